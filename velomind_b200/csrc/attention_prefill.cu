// Prefill attention for bfloat16: causal (optionally windowed) attention of the step's new tokens over
// the paged cache, on the tensor cores, with the online softmax kept in float32.
//
// Arithmetic as in attention_generic.cu (reference: examples/common/llama/llama_graph.cpp:97-103,
// src/cpu/ops/fused_attention.cpp:84-135).  One CTA owns 64 consecutive new tokens of one sequence and
// one query head.  It has NG groups of four warps; a group's warps own 16 query rows each, and the groups
// share the key blocks of the tile among them (group g takes blocks g, g + NG, ...), so that the tiles at
// the end of a long prompt, which see the most keys, are not a chain NG times longer than the rest.  Keys
// and values arrive one cache page per group (64 tokens of one kv head, contiguous) at a time through
// cp.async into double-buffered shared memory; Q K^T and P V run on mma.sync m16n8k16 (bf16 in, float32
// accumulate); at the end the groups' partial results are merged through shared memory.
//
// Sizes: head size D in {16, 32, ..., 128} (template), any head count and group size; the sequences of a
// step may have any lengths.  Other head sizes are refused (the caller falls back to the generic kernel).
#include "common.cuh"

namespace {

constexpr int BM = 64;      // query rows per CTA
constexpr int BN = 64;      // keys per block = one cache page
static_assert(BN == VM_PAGE_TOKENS, "a key block is one page");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = pred ? 16 : 0;                       // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float c[4], const unsigned a[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (ex2.approx: 2^-inf = 0, relative error about 2^-22)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int D, int NG>
__global__ void __launch_bounds__(128 * NG)
attn_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                        const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ positions, const int* __restrict__ cu_tokens, int B,
                        __nv_bfloat16* __restrict__ out, int H, int Hkv, float scale_log2, int window, int n_pages,
                        int* __restrict__ err) {
    constexpr int DP = D + 8;                  // padded row: 2D+16 bytes, an odd number of 16-byte units -> no ldmatrix conflicts
    constexpr int CH = D / 8;                  // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [BM][DP]
    __nv_bfloat16* sK = sQ + BM * DP;                                    // [2][NG][BN][DP]
    __nv_bfloat16* sV = sK + 2 * NG * BN * DP;                           // [2][NG][BN][DP]
    constexpr int THREADS = 128 * NG;

    // ---- which 64 tokens of which sequence
    // (the last tiles of a sequence see the most keys: they are started first)
    int tile = gridDim.x - 1 - blockIdx.x, seq = 0, t0 = 0, n_rows = 0;
    for (; seq < B; ++seq) {
        const int a = cu_tokens[seq], b = cu_tokens[seq + 1];
        const int nt = (b - a + BM - 1) / BM;
        if (tile < nt) { t0 = a + tile * BM; n_rows = min(BM, b - t0); break; }
        tile -= nt;
    }
    if (seq >= B) return;
    const int h = blockIdx.y, hk = h / (H / Hkv);
    const int tid = threadIdx.x, lane = tid & 31;
    const int grp = tid >> 7, warp = (tid >> 5) & 3;       // group of four warps; warp inside its group
    const int pos0 = positions[t0];
    const int hi = pos0 + n_rows - 1;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int blk_lo = lo / BN, blk_hi = hi / BN;
    const size_t page_stride = (size_t)Hkv * BN * D;
    const int* table = block_table + (size_t)seq * max_blocks;

    // ---- Q tile -> shared (rows past the sequence's end are zero)
    for (int c = tid; c < BM * CH; c += THREADS) {
        const int r = c / CH, ch = c - r * CH;
        cp_async16(sQ + r * DP + ch * 8, q + (size_t)(t0 + (r < n_rows ? r : 0)) * q_row_stride + (size_t)h * D + ch * 8, r < n_rows);
    }
    auto load_kv = [&](int step, int buf) {                // the NG blocks of one step, by all threads
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
            const int blk = blk_lo + step * NG + gi;
            if (blk > blk_hi) break;
            int page = (blk < max_blocks) ? table[blk] : -1;
            const bool ok = (page >= 0 && page < n_pages);
            if (!ok) { if (tid == 0 && err) atomicExch(err, 3); page = 0; }
            const __nv_bfloat16* kg = kpages + (size_t)page * page_stride + (size_t)hk * BN * D;
            const __nv_bfloat16* vg = vpages + (size_t)page * page_stride + (size_t)hk * BN * D;
            __nv_bfloat16* ks = sK + (size_t)(buf * NG + gi) * BN * DP;
            __nv_bfloat16* vs = sV + (size_t)(buf * NG + gi) * BN * DP;
            for (int c = tid; c < BN * CH; c += THREADS) {
                const int r = c / CH, ch = c - r * CH;
                cp_async16(ks + r * DP + ch * 8, kg + r * D + ch * 8, ok);
                cp_async16(vs + r * DP + ch * 8, vg + r * D + ch * 8, ok);
            }
        }
    };
    const int n_steps = (blk_hi - blk_lo + NG) / NG;
    load_kv(0, 0);
    cp_async_commit();

    // ---- per-thread state: rows g and g+8 of the warp's 16 rows
    const int g = lane >> 2, t4 = lane & 3;
    const int row_a = warp * 16 + g, row_b = row_a + 8;
    const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;
    const int lo_a = (window > 0) ? pos_a - window + 1 : 0, lo_b = (window > 0) ? pos_b - window + 1 : 0;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    unsigned qa[D / 16][4];
    bool q_loaded = false;
    const int warp_max_pos = pos0 + warp * 16 + 15;

    for (int step = 0; step < n_steps; ++step) {
        const int buf = step & 1;
        const int blk = blk_lo + step * NG + grp;          // this group's block of the step
        if (step + 1 < n_steps) load_kv(step + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (!q_loaded) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                ldmatrix_x4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3],
                            sQ + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * DP + kk * 16 + 8 * (lane >> 4));
            q_loaded = true;
        }
        const int key0 = blk * BN;
        if (blk <= blk_hi && key0 <= warp_max_pos && warp * 16 < n_rows) {      // this warp has a row that may see this page
            const __nv_bfloat16* ks = sK + (size_t)(buf * NG + grp) * BN * DP;
            const __nv_bfloat16* vs = sV + (size_t)(buf * NG + grp) * BN * DP;
            float s[BN / 8][4];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < BN / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, ks + (nb * 8 + (lane & 7) + 8 * (lane >> 4)) * DP + kk * 16 + 8 * ((lane >> 3) & 1));
                    mma_bf16(s[nb], qa[kk], b0, b1);
                    mma_bf16(s[nb + 1], qa[kk], b2, b3);
                }
            }
            // ---- mask (only where a block touches the diagonal, the window's edge or rows past the end), then the
            //      online softmax in base 2 on the RAW scores: p = 2^(s * c - m * c) is one FMA and one ex2 per score
            const bool interior = (key0 + BN - 1 <= pos0 + warp * 16) && (window <= 0 || key0 >= pos0 + warp * 16 + 15 - window + 1);
            if (!interior) {
#pragma unroll
                for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + nb * 8 + 2 * t4 + e;
                        if (!(key <= pos_a && key >= lo_a)) s[nb][e] = -INFINITY;
                        if (!(key <= pos_b && key >= lo_b)) s[nb][2 + e] = -INFINITY;
                    }
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                mx_a = fmaxf(mx_a, fmaxf(s[nb][0], s[nb][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[nb][2], s[nb][3]));
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);               // running maxima of the raw scores
            const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a, use_b = (mn_b == -INFINITY) ? 0.f : mn_b;   // row sees nothing yet
            const float al_a = fast_exp2((m_a - use_a) * scale_log2), al_b = fast_exp2((m_b - use_b) * scale_log2);
            const float off_a = -use_a * scale_log2, off_b = -use_b * scale_log2;
            float sum_a = 0.f, sum_b = 0.f;
            unsigned pa[BN / 16][4];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                const float p0 = fast_exp2(fmaf(s[nb][0], scale_log2, off_a)), p1 = fast_exp2(fmaf(s[nb][1], scale_log2, off_a));
                const float p2 = fast_exp2(fmaf(s[nb][2], scale_log2, off_b)), p3 = fast_exp2(fmaf(s[nb][3], scale_log2, off_b));
                sum_a += p0 + p1; sum_b += p2 + p3;
                pa[nb >> 1][(nb & 1) * 2 + 0] = pack_bf16(p0, p1);
                pa[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l_a = l_a * al_a + sum_a; l_b = l_b * al_b + sum_b;          // per-thread partial sums; quads are joined at the end
            m_a = mn_a; m_b = mn_b;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
            // ---- O += P V
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < D / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * DP + nb * 8 + 8 * (lane >> 4));
                    mma_bf16(o[nb], pa[kk], b0, b1);
                    mma_bf16(o[nb + 1], pa[kk], b2, b3);
                }
            }
        }
        __syncthreads();          // everyone is done with `buf` before the next iteration's prefetch overwrites it
    }
    cp_async_wait<0>();

    // ---- finish: join the quad's partial sums, merge the groups, normalise, store
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (NG > 1) {
        // groups 1.. leave (o, m, l) of their rows in shared memory (the key/value buffers are free now)
        constexpr int RW = D + 2;
        float* xch = reinterpret_cast<float*>(sK);          // [NG - 1][BM][RW]
        __syncthreads();
        if (grp > 0) {
            float* ra = xch + ((size_t)(grp - 1) * BM + row_a) * RW;
            float* rb = xch + ((size_t)(grp - 1) * BM + row_b) * RW;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                const int d = i * 8 + 2 * t4;
                ra[d] = o[i][0]; ra[d + 1] = o[i][1]; rb[d] = o[i][2]; rb[d + 1] = o[i][3];
            }
            if (t4 == 0) { ra[D] = m_a; ra[D + 1] = l_a; rb[D] = m_b; rb[D + 1] = l_b; }
        }
        __syncthreads();
        if (grp > 0) return;
#pragma unroll
        for (int og = 0; og < NG - 1; ++og) {
            const float* ra = xch + ((size_t)og * BM + row_a) * RW;
            const float* rb = xch + ((size_t)og * BM + row_b) * RW;
            const float ma2 = ra[D], mb2 = rb[D];
            const float Ma = fmaxf(m_a, ma2), Mb = fmaxf(m_b, mb2);
            const float ua = (Ma == -INFINITY) ? 0.f : Ma, ub = (Mb == -INFINITY) ? 0.f : Mb;
            const float fa = fast_exp2((m_a - ua) * scale_log2), fa2 = fast_exp2((ma2 - ua) * scale_log2);
            const float fb = fast_exp2((m_b - ub) * scale_log2), fb2 = fast_exp2((mb2 - ub) * scale_log2);
            l_a = l_a * fa + ra[D + 1] * fa2; l_b = l_b * fb + rb[D + 1] * fb2;
            m_a = Ma; m_b = Mb;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                const int d = i * 8 + 2 * t4;
                o[i][0] = o[i][0] * fa + ra[d] * fa2; o[i][1] = o[i][1] * fa + ra[d + 1] * fa2;
                o[i][2] = o[i][2] * fb + rb[d] * fb2; o[i][3] = o[i][3] * fb + rb[d + 1] * fb2;
            }
        }
    }
    const float inv_a = 1.f / l_a, inv_b = 1.f / l_b;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int d = i * 8 + 2 * t4;
        if (row_a < n_rows)
            *reinterpret_cast<unsigned*>(out + ((size_t)(t0 + row_a) * H + h) * D + d) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
        if (row_b < n_rows)
            *reinterpret_cast<unsigned*>(out + ((size_t)(t0 + row_b) * H + h) * D + d) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

template <int D, int NG>
int launch_prefill_ng(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                      int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, void* out, int H, int Hkv,
                      float scale, int window, int n_pages, int* err, cudaStream_t stream) {
    constexpr int DP = D + 8;
    size_t smem = (size_t)(BM + 4 * NG * BN) * DP * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)(NG - 1) * BM * (D + 2) * sizeof(float) + (size_t)BM * DP * sizeof(__nv_bfloat16);
    if (merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<D, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, H);
    attn_prefill_mma_kernel<D, NG><<<grid, 128 * NG, smem, stream>>>(
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)kpages, (const __nv_bfloat16*)vpages, block_table,
        max_blocks, positions, cu_tokens, B, (__nv_bfloat16*)out, H, Hkv, scale * 1.4426950408889634f, window, n_pages, err);
    return vm_launch_status();
}

// `long_tiles`: some tile of the step sees many key blocks (a long prompt): split its blocks over two warp groups
template <int D>
int launch_prefill(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                   int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, void* out, int H, int Hkv,
                   float scale, int window, int n_pages, int* err, int groups, cudaStream_t stream) {
    if (groups >= 4 && D <= 64)
        return launch_prefill_ng<D, 4>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, cu_tokens, B, n_tiles,
                                       out, H, Hkv, scale, window, n_pages, err, stream);
    if (groups >= 2)
        return launch_prefill_ng<D, 2>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, cu_tokens, B, n_tiles,
                                       out, H, Hkv, scale, window, n_pages, err, stream);
    return launch_prefill_ng<D, 1>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, cu_tokens, B, n_tiles,
                                   out, H, Hkv, scale, window, n_pages, err, stream);
}

}  // namespace

// n_tiles = sum over the step's sequences of ceil(new tokens / 64), computed by the host.
// groups: warp groups (1, 2 or 4) that share a tile's key blocks; more for steps whose tiles see many keys.
VM_API int vm_attention_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                     const int* block_table, int max_blocks, const int* positions, const int* cu_tokens,
                                     int B, int n_tiles, void* out, int H, int Hkv, int D, float scale, int window,
                                     int n_pages, int* err, int groups, cudaStream_t stream) {
    if (n_tiles <= 0 || B <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || (q_row_stride % 8) != 0) return VM_ERR_UNSUPPORTED;
#define VM_PREFILL_CASE(DD)                                                                                          \
    case DD:                                                                                                         \
        return launch_prefill<DD>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, cu_tokens, B,  \
                                  n_tiles, out, H, Hkv, scale, window, n_pages, err, groups, stream);
    switch (D) {
        VM_PREFILL_CASE(16) VM_PREFILL_CASE(32) VM_PREFILL_CASE(48) VM_PREFILL_CASE(64)
        VM_PREFILL_CASE(80) VM_PREFILL_CASE(96) VM_PREFILL_CASE(112) VM_PREFILL_CASE(128)
        default: return VM_ERR_UNSUPPORTED;
    }
#undef VM_PREFILL_CASE
}
