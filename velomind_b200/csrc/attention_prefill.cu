// Prefill attention for bfloat16: causal (optionally windowed) attention of the step's new tokens over
// the paged cache, on the tensor cores, with the online softmax kept in float32.
//
// Arithmetic as in attention_generic.cu (reference: examples/common/llama/llama_graph.cpp:97-103,
// src/cpu/ops/fused_attention.cpp:84-135).  One CTA owns 64 consecutive new tokens of one sequence and
// one query head; its four warps own 16 query rows each.  Keys and values arrive one cache page
// (64 tokens of one kv head, contiguous) at a time through cp.async into double-buffered shared
// memory; Q K^T and P V run on mma.sync m16n8k16 (bf16 in, float32 accumulate).
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
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int D>
__global__ void __launch_bounds__(128)
attn_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                        const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ positions, const int* __restrict__ cu_tokens, int B,
                        __nv_bfloat16* __restrict__ out, int H, int Hkv, float scale_log2, int window, int n_pages,
                        int* __restrict__ err) {
    constexpr int DP = D + 8;                  // padded row: 2D+16 bytes, an odd number of 16-byte units -> no ldmatrix conflicts
    constexpr int CH = D / 8;                  // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [BM][DP]
    __nv_bfloat16* sK = sQ + BM * DP;                                    // [2][BN][DP]
    __nv_bfloat16* sV = sK + 2 * BN * DP;                                // [2][BN][DP]

    // ---- which 64 tokens of which sequence
    int tile = blockIdx.x, seq = 0, t0 = 0, n_rows = 0;
    for (; seq < B; ++seq) {
        const int a = cu_tokens[seq], b = cu_tokens[seq + 1];
        const int nt = (b - a + BM - 1) / BM;
        if (tile < nt) { t0 = a + tile * BM; n_rows = min(BM, b - t0); break; }
        tile -= nt;
    }
    if (seq >= B) return;
    const int h = blockIdx.y, hk = h / (H / Hkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos0 = positions[t0];
    const int hi = pos0 + n_rows - 1;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int blk_lo = lo / BN, blk_hi = hi / BN;
    const size_t page_stride = (size_t)Hkv * BN * D;
    const int* table = block_table + (size_t)seq * max_blocks;

    // ---- Q tile -> shared (rows past the sequence's end are zero)
    for (int c = tid; c < BM * CH; c += 128) {
        const int r = c / CH, ch = c - r * CH;
        cp_async16(sQ + r * DP + ch * 8, q + (size_t)(t0 + (r < n_rows ? r : 0)) * q_row_stride + (size_t)h * D + ch * 8, r < n_rows);
    }
    auto load_kv = [&](int blk, int buf) {
        int page = (blk < max_blocks) ? table[blk] : -1;
        const bool ok = (page >= 0 && page < n_pages);
        if (!ok) { if (tid == 0 && err) atomicExch(err, 3); page = 0; }
        const __nv_bfloat16* kg = kpages + (size_t)page * page_stride + (size_t)hk * BN * D;
        const __nv_bfloat16* vg = vpages + (size_t)page * page_stride + (size_t)hk * BN * D;
        __nv_bfloat16* ks = sK + buf * BN * DP;
        __nv_bfloat16* vs = sV + buf * BN * DP;
        for (int c = tid; c < BN * CH; c += 128) {
            const int r = c / CH, ch = c - r * CH;
            cp_async16(ks + r * DP + ch * 8, kg + r * D + ch * 8, ok);
            cp_async16(vs + r * DP + ch * 8, vg + r * D + ch * 8, ok);
        }
    };
    load_kv(blk_lo, 0);
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

    for (int blk = blk_lo; blk <= blk_hi; ++blk) {
        const int buf = (blk - blk_lo) & 1;
        if (blk + 1 <= blk_hi) load_kv(blk + 1, buf ^ 1);
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
        if (key0 <= warp_max_pos && warp * 16 < n_rows) {          // this warp has a row that may see this page
            const __nv_bfloat16* ks = sK + buf * BN * DP;
            const __nv_bfloat16* vs = sV + buf * BN * DP;
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
            // ---- mask, online softmax (base 2)
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + nb * 8 + 2 * t4 + e;
                    const float va = (key <= pos_a && key >= lo_a) ? s[nb][e] * scale_log2 : -INFINITY;
                    const float vb = (key <= pos_b && key >= lo_b) ? s[nb][2 + e] * scale_log2 : -INFINITY;
                    s[nb][e] = va; s[nb][2 + e] = vb;
                    mx_a = fmaxf(mx_a, va); mx_b = fmaxf(mx_b, vb);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a, use_b = (mn_b == -INFINITY) ? 0.f : mn_b;   // row sees nothing yet
            const float al_a = exp2f(m_a - use_a), al_b = exp2f(m_b - use_b);
            float sum_a = 0.f, sum_b = 0.f;
            unsigned pa[BN / 16][4];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                const float p0 = exp2f(s[nb][0] - use_a), p1 = exp2f(s[nb][1] - use_a);
                const float p2 = exp2f(s[nb][2] - use_b), p3 = exp2f(s[nb][3] - use_b);
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

    // ---- finish: join the quad's partial sums, normalise, store
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
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

template <int D>
int launch_prefill(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                   int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, void* out, int H, int Hkv,
                   float scale, int window, int n_pages, int* err, cudaStream_t stream) {
    constexpr int DP = D + 8;
    const size_t smem = (size_t)(BM + 4 * BN) * DP * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, H);
    attn_prefill_mma_kernel<D><<<grid, 128, smem, stream>>>(
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)kpages, (const __nv_bfloat16*)vpages, block_table,
        max_blocks, positions, cu_tokens, B, (__nv_bfloat16*)out, H, Hkv, scale * 1.4426950408889634f, window, n_pages, err);
    return vm_launch_status();
}

}  // namespace

// n_tiles = sum over the step's sequences of ceil(new tokens / 64), computed by the host.
VM_API int vm_attention_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                     const int* block_table, int max_blocks, const int* positions, const int* cu_tokens,
                                     int B, int n_tiles, void* out, int H, int Hkv, int D, float scale, int window,
                                     int n_pages, int* err, cudaStream_t stream) {
    if (n_tiles <= 0 || B <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || (q_row_stride % 8) != 0) return VM_ERR_UNSUPPORTED;
#define VM_PREFILL_CASE(DD)                                                                                          \
    case DD:                                                                                                         \
        return launch_prefill<DD>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, cu_tokens, B,  \
                                  n_tiles, out, H, Hkv, scale, window, n_pages, err, stream);
    switch (D) {
        VM_PREFILL_CASE(16) VM_PREFILL_CASE(32) VM_PREFILL_CASE(48) VM_PREFILL_CASE(64)
        VM_PREFILL_CASE(80) VM_PREFILL_CASE(96) VM_PREFILL_CASE(112) VM_PREFILL_CASE(128)
        default: return VM_ERR_UNSUPPORTED;
    }
#undef VM_PREFILL_CASE
}
