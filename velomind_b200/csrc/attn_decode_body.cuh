// Device body of the split-KV decode attention (see attention_decode.cu).
#pragma once
#include "mma.cuh"

namespace vmad {

constexpr int DEC_ROWS = 16;           // query heads per CTA (the M of the tensor-core tile); more heads per kv head take more CTAs
constexpr int MAX_SPLITS = 16;         // the merge keeps one value per split in registers

// One warp works on one cache page (64 keys) at a time: K and V of the page go to the warp's own shared
// memory with cp.async, S = Q K^T and O += P V run on mma.sync m16n8k16 with the G query heads of the kv
// head as the rows of the tile (padded to 16), the softmax state is float32 in base 2.
// (split, group_y, b) of (n_splits, n_group_y, B) is what (blockIdx, gridDim) are for the stand-alone kernel.
template <int D, int DEC_WARPS, bool PDL>
__device__ __forceinline__ void
attn_decode_body(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                 const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                 const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                 int* __restrict__ counters, int H, int Hkv, float scale_log2, int window, int n_pages,
                 int* __restrict__ err, const int split, const int n_splits, const int group_y, const int n_group_y,
                 const int b, unsigned char* smem_raw) {
    constexpr int DP = D + 8;              // padded row: an odd number of 16-byte units -> conflict-free ldmatrix
    constexpr int CH = D / 8;              // 16-byte chunks per row
    constexpr int RW = D + 2;              // a result row: D sums, then the running max and the running sum
    constexpr int BN = VM_PAGE_TOKENS;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);                    // [16][DP]
    __nv_bfloat16* sKV = sQ + DEC_ROWS * DP;                                            // [warps][K,V][64][DP]
    float* res = reinterpret_cast<float*>(sKV + DEC_WARPS * 2 * BN * DP);               // [warps][16][RW]
    if (PDL) vm_pdl_launch_dependents();
    // Before the wait this kernel reads what OLDER steps and kernels wrote: positions, the block table and the cache
    // rows of earlier tokens.  That is sound because the kernel launched directly before it (the one that writes the
    // new token's row) lets its dependents start only after its own wait, when everything older is complete.  The
    // new row and the queries, which that kernel writes, are fetched after the wait.
    const int G = H / Hkv;
    const int groups_per_kv = (G + DEC_ROWS - 1) / DEC_ROWS;
    const int hk = group_y / groups_per_kv, gg = group_y - hk * groups_per_kv;
    const int h0 = hk * G + gg * DEC_ROWS;                 // first query head of this CTA
    const int ng = min(DEC_ROWS, G - gg * DEC_ROWS);       // query heads of this CTA
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = positions[b];                          // one token per sequence: token index == sequence index
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_page = lo / BN, last_page = pos / BN;
    const int pages = last_page - first_page + 1;
    const int per_split = (pages + n_splits - 1) / n_splits;
    const int page_a = first_page + split * per_split, page_b = min(last_page + 1, page_a + per_split);
    const size_t page_stride = (size_t)Hkv * BN * D;
    const int* table = block_table + (size_t)b * max_blocks;
    __nv_bfloat16* ks = sKV + (size_t)warp * 2 * BN * DP;
    __nv_bfloat16* vs = ks + BN * DP;
    const int new_row = pos - last_page * BN;              // the row of the last page that this step's token takes

    // the calling warp fetches K and V of one page; skip >= 0: all rows but that one
    auto load_page = [&](int blk, int skip) -> bool {
        const int page = (blk < max_blocks) ? table[blk] : -1;
        if (page < 0 || page >= n_pages) { if (lane == 0 && err) atomicExch(err, 3); return false; }
        const __nv_bfloat16* kg = kpages + (size_t)page * page_stride + (size_t)hk * BN * D;
        const __nv_bfloat16* vg = vpages + (size_t)page * page_stride + (size_t)hk * BN * D;
#pragma unroll 4
        for (int c = lane; c < BN * CH; c += 32) {
            const int r = c / CH, ch = c - r * CH;
            if (r != skip) {
                vm_cp_async16(ks + r * DP + ch * 8, kg + r * D + ch * 8);
                vm_cp_async16(vs + r * DP + ch * 8, vg + r * D + ch * 8);
            }
        }
        return true;
    };
    int blk = page_a + warp;
    bool have = (blk < page_b) && load_page(blk, PDL && blk == last_page ? new_row : -1);
    vm_cp_async_commit();
    if (PDL) {
        vm_pdl_wait();
        if (have && blk == last_page && lane < 2 * CH) {   // the new token's key and value
            const int page = table[blk];
            const size_t at = (size_t)page * page_stride + ((size_t)hk * BN + new_row) * D + (lane % CH) * 8;
            if (lane < CH) vm_cp_async16(ks + new_row * DP + lane * 8, kpages + at);
            else vm_cp_async16(vs + new_row * DP + (lane - CH) * 8, vpages + at);
        }
    }
    // ---- the queries of this CTA's heads (rows past the last head are zero)
    for (int c = tid; c < DEC_ROWS * CH; c += DEC_WARPS * 32) {
        const int r = c / CH, ch = c - r * CH;
        if (r < ng) vm_cp_async16(sQ + r * DP + ch * 8, q + (size_t)b * q_row_stride + (size_t)(h0 + r) * D + ch * 8);
        else *reinterpret_cast<uint4*>(sQ + r * DP + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    vm_cp_async_commit();
    vm_cp_async_wait_all();
    __syncthreads();                                       // the queries (fetched by all threads) are in place

    const int g = lane >> 2, t4 = lane & 3;
    unsigned qa[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        vm_ldmatrix_x4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3],
                       sQ + ((lane & 7) + 8 * ((lane >> 3) & 1)) * DP + kk * 16 + 8 * (lane >> 4));
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;     // rows g and g + 8 of the tile
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    while (blk < page_b) {
        if (have) {
            const int key0 = blk * BN;
            float s[BN / 8][4];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < BN / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    vm_ldmatrix_x4(b0, b1, b2, b3, ks + (nb * 8 + (lane & 7) + 8 * (lane >> 4)) * DP + kk * 16 + 8 * ((lane >> 3) & 1));
                    vm_mma_bf16_16816(s[nb], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
                    vm_mma_bf16_16816(s[nb + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b2, b3);
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + nb * 8 + 2 * t4 + e;
                    const bool ok = (key <= pos && key >= lo);
                    const float va = ok ? s[nb][e] * scale_log2 : -INFINITY;
                    const float vb = ok ? s[nb][2 + e] * scale_log2 : -INFINITY;
                    s[nb][e] = va; s[nb][2 + e] = vb;
                    mx_a = fmaxf(mx_a, va); mx_b = fmaxf(mx_b, vb);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a, use_b = (mn_b == -INFINITY) ? 0.f : mn_b;
            const float al_a = exp2f(m_a - use_a), al_b = exp2f(m_b - use_b);
            float sum_a = 0.f, sum_b = 0.f;
            unsigned pa[BN / 16][4];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                const float p0 = exp2f(s[nb][0] - use_a), p1 = exp2f(s[nb][1] - use_a);
                const float p2 = exp2f(s[nb][2] - use_b), p3 = exp2f(s[nb][3] - use_b);
                sum_a += p0 + p1; sum_b += p2 + p3;
                pa[nb >> 1][(nb & 1) * 2 + 0] = vm_pack_bf16(p0, p1);
                pa[nb >> 1][(nb & 1) * 2 + 1] = vm_pack_bf16(p2, p3);
            }
            l_a = l_a * al_a + sum_a; l_b = l_b * al_b + sum_b;        // per-thread partial sums; the quad is joined below
            m_a = mn_a; m_b = mn_b;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < D / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    vm_ldmatrix_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * DP + nb * 8 + 8 * (lane >> 4));
                    vm_mma_bf16_16816(o[nb], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    vm_mma_bf16_16816(o[nb + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        }
        blk += DEC_WARPS;
        if (blk < page_b) {
            __syncwarp();                                  // every lane is done with the page before it is overwritten
            have = load_page(blk, -1);
            vm_cp_async_commit();
            vm_cp_async_wait_all();
            __syncwarp();
        }
    }
    // ---- this warp's result rows: join the quad's sums; res[warp][row] = (o[D], m, l)
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    {
        float* ra = res + ((size_t)warp * DEC_ROWS + g) * RW;
        float* rb = res + ((size_t)warp * DEC_ROWS + g + 8) * RW;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const int d = i * 8 + 2 * t4;
            ra[d] = o[i][0]; ra[d + 1] = o[i][1]; rb[d] = o[i][2]; rb[d + 1] = o[i][3];
        }
        if (t4 == 0) { ra[D] = m_a; ra[D + 1] = l_a; rb[D] = m_b; rb[D + 1] = l_b; }
    }
    __syncthreads();
    if (n_splits == 1) {
        // one CTA holds all keys of the sequence: the warps' rows are joined straight into the output
        for (int i = tid; i < ng * D; i += DEC_WARPS * 32) {
            const int r = i / D, d = i - r * D;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, res[((size_t)w * DEC_ROWS + r) * RW + D]);
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) {
                const float* rr = res + ((size_t)w * DEC_ROWS + r) * RW;
                const float f = (rr[D] == -INFINITY) ? 0.f : exp2f(rr[D] - M);
                acc += f * rr[d]; L += f * rr[D + 1];
            }
            out[((size_t)b * H + (h0 + r)) * D + d] = __float2bfloat16_rn(acc / L);
        }
        __syncthreads();                                   // shared memory may be reused for another item
        return;
    }
    // partial[b, h, split, :] = (o[D], m, l), merged over the warps (max and sums in base 2)
    for (int i = tid; i < ng * D; i += DEC_WARPS * 32) {
        const int r = i / D, d = i - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, res[((size_t)w * DEC_ROWS + r) * RW + D]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* rr = res + ((size_t)w * DEC_ROWS + r) * RW;
            const float f = (rr[D] == -INFINITY) ? 0.f : exp2f(rr[D] - M);
            acc += f * rr[d]; L += f * rr[D + 1];
        }
        float* dst = partial + (((size_t)b * H + (h0 + r)) * n_splits + split) * RW;
        dst[d] = acc;
        if (d == 0) { dst[D] = M; dst[D + 1] = L; }
    }
    // ---- the last CTA of this (sequence, head group) to arrive merges the splits; nobody waits
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(&counters[(size_t)b * n_group_y + group_y], 1);
        is_last = (old == n_splits - 1);
        if (is_last) counters[(size_t)b * n_group_y + group_y] = 0;     // ready for the next launch
    }
    __syncthreads();
    if (is_last) {
    __threadfence();
    for (int i = tid; i < ng * D; i += DEC_WARPS * 32) {
        const int r = i / D, d = i - r * D;
        const float* src = partial + ((size_t)b * H + (h0 + r)) * n_splits * RW;
        // all loads first (independent of each other), then the arithmetic: one memory latency, not n_splits
        float ms[MAX_SPLITS], ls[MAX_SPLITS], os[MAX_SPLITS];
#pragma unroll
        for (int s2 = 0; s2 < MAX_SPLITS; ++s2) {
            if (s2 < n_splits) {
                ms[s2] = __ldcg(src + (size_t)s2 * RW + D);
                ls[s2] = __ldcg(src + (size_t)s2 * RW + D + 1);
                os[s2] = __ldcg(src + (size_t)s2 * RW + d);
            } else { ms[s2] = -INFINITY; ls[s2] = 0.f; os[s2] = 0.f; }
        }
        float M = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < MAX_SPLITS; ++s2) M = fmaxf(M, ms[s2]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < MAX_SPLITS; ++s2) {
            const float f = (ms[s2] == -INFINITY) ? 0.f : exp2f(ms[s2] - M);
            acc += f * os[s2];
            L += f * ls[s2];
        }
        out[((size_t)b * H + (h0 + r)) * D + d] = __float2bfloat16_rn(acc / L);
    }
    }
    __syncthreads();                                       // shared memory may be reused for another item
}

template <int D, int WARPS>
__host__ __device__ constexpr size_t attn_decode_smem_bytes() {
    return (size_t)(DEC_ROWS + WARPS * 2 * VM_PAGE_TOKENS) * (D + 8) * sizeof(__nv_bfloat16)
           + (size_t)WARPS * DEC_ROWS * (D + 2) * sizeof(float);
}

}  // namespace vmad
