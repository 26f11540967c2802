// Prefill attention for bfloat16 and head size 64 on the fifth-generation tensor cores (tcgen05): causal
// (optionally windowed) attention of the step's new tokens over the paged cache, online softmax in float32.
//
// Arithmetic as in attention_generic.cu (reference: examples/common/llama/llama_graph.cpp:97-103,
// src/cpu/ops/fused_attention.cpp:84-135).  mma.sync, which attention_prefill.cu uses, runs on this GPU at a
// fraction of the tensor cores' rate and that kernel is bound by it; here both products of a key block are single
// tcgen05.mma chains with their accumulators in tensor memory.
//
// One CTA of 128 threads owns 128 consecutive new tokens of one sequence and one query head; thread r owns query
// row r: tensor-memory lane r holds its scores and its P V sums, so the softmax needs no exchange between
// threads.  Per block of 64 keys (one cache page):
//   S = Q K^T      M 128, N 64, K 64: four tcgen05.mma (kind::f16) from shared memory (Q and K both K-major,
//                  128-byte rows, 128-byte swizzle) into tensor-memory columns 0..63
//   softmax        each thread reads its row with tcgen05.ld, masks, keeps the running maximum and sum, and writes
//                  its 64 probabilities as bf16 into a K-major swizzled P tile in shared memory
//   PV             M 128, N 64 (head size), K 64 (keys): four tcgen05.mma with V as the MN-major B operand (the
//                  cache keeps a key's 64 values contiguous) into columns 64..127; each thread adds its row to its
//                  output registers, which it rescales itself when the maximum moves
// The softmax, not the products, is what a tile costs (64 x 128 exponentials and as many roundings per block go through
// one SM's special-function units), and the last tiles of a long prompt see the most keys.  So a tile may belong to a
// CLUSTER of NC CTAs (1 to 4) on NC SMs: CTA c takes the tile's key blocks c, c + NC, ..., and at the end the CTAs
// exchange their rows (sums, maximum, denominator) through distributed shared memory, each joining and storing every
// NC-th row of the tile.
// Q, K and V reach shared memory through cp.async with the swizzle applied to the destination (the next page is in
// flight while this one is worked on).  The one mbarrier wait (completion of the MMAs, signalled by tcgen05.commit)
// is bounded: when it gives up, the CTA raises error word 4, drains its copies, frees its tensor memory and returns.
#include "tc05.cuh"

namespace {

constexpr int TA_BM = 128, TA_BN = 64, TA_D = 64, TA_THREADS = 128;
static_assert(TA_BN == VM_PAGE_TOKENS, "a key block is one page");
constexpr uint32_t TA_TMEM_COLS = 128;                                       // per group: scores 0..63, P V 64..127
constexpr int TA_Q_BYTES = TA_BM * 128, TA_KV_BYTES = TA_BN * 128, TA_P_BYTES = TA_BM * 128;
constexpr int TA_WORK_BYTES = 4 * TA_KV_BYTES + TA_P_BYTES;                  // K[2], V[2], P
constexpr int TA_SMEM = TA_Q_BYTES + TA_WORK_BYTES + 128;                    // + barrier, tensor-memory slot, flag
constexpr int TA_RW = TA_D + 4;                                              // floats of an exchanged row: sums, maximum, denominator, padding
static_assert(TA_RW * 4 * (TA_BM + 3) <= TA_WORK_BYTES, "the exchanged rows must fit into the K, V and P buffers");

template <int NC>
__global__ void __launch_bounds__(TA_THREADS)
attn_prefill_tc_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                       const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                       const int* __restrict__ positions, const int* __restrict__ cu_tokens, int B,
                       __nv_bfloat16* __restrict__ out, int H, int Hkv, float scale_log2, int window, int n_pages,
                       int* __restrict__ err) {
    constexpr int D = TA_D, BN = TA_BN;
    // instruction descriptors: float32 accumulate (bits 4-5 = 1), A and B bf16 (bits 7-9 and 10-12 = 1), B MN-major
    // (bit 16) for P V, N >> 3 in bits 17-22, M >> 4 in bits 24-28
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TA_BM >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(TA_BM >> 4) << 24);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, gt = tid, warp = tid >> 5;
    int grp = 0;                                                    // this CTA's place in its cluster
    if (NC > 1) { unsigned r; asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); grp = (int)r; }
    constexpr int NG = NC;
    unsigned char* sQ = smem_raw;
    unsigned char* sK = sQ + TA_Q_BYTES;                            // [2][64 keys][128 bytes]
    unsigned char* sV = sK + 2 * TA_KV_BYTES;                       // [2][64 keys][128 bytes]
    unsigned char* sP = sV + 2 * TA_KV_BYTES;                       // [128 rows][128 bytes]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sQ + TA_Q_BYTES + TA_WORK_BYTES);
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 1);
    int& abort_flag = *reinterpret_cast<int*>(bars + 2);

    // ---- which 128 tokens of which sequence (the last tiles of a sequence see the most keys: they start first)
    int tile = (int)(gridDim.x / NC) - 1 - (int)(blockIdx.x / NC), seq = 0, t0 = 0, n_rows = 0;
    for (; seq < B; ++seq) {
        const int a = cu_tokens[seq], b = cu_tokens[seq + 1];
        const int nt = (b - a + TA_BM - 1) / TA_BM;
        if (tile < nt) { t0 = a + tile * TA_BM; n_rows = min(TA_BM, b - t0); break; }
        tile -= nt;
    }
    if (seq >= B) return;                                   // (before any barrier or allocation: the whole cluster leaves)
    const int h = blockIdx.y, hk = h / (H / Hkv);
    const int pos0 = positions[t0];
    const int hi = pos0 + n_rows - 1;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int blk_lo = lo / BN, blk_hi = hi / BN;
    const int n_blocks = blk_hi - blk_lo + 1;
    const int n_steps = (n_blocks - grp + NG - 1) / NG;            // this group's blocks: grp, grp + NG, ...
    const size_t page_stride = (size_t)Hkv * BN * D;
    const int* table = block_table + (size_t)seq * max_blocks;
    if (tid == 0) {
        abort_flag = (ta_u32(smem_raw) & 1023u) ? 1 : 0;    // misaligned tiles would give wrong sums: give up instead
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ta_u32(&bars[0])) : "memory");     // scores done
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ta_u32(&bars[3])) : "memory");     // P V done
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 32) {                                         // one warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ta_u32(&tmem_slot)), "r"(TA_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // ---- Q tile -> shared, swizzled (rows past the sequence's end are zero)
    for (int c = tid; c < TA_BM * 8; c += TA_THREADS) {
        const int r = c >> 3, ch = c & 7;
        ta_cp_async16(ta_u32(sQ) + r * 128 + ((ch ^ (r & 7)) << 4),
                      q + (size_t)(t0 + (r < n_rows ? r : 0)) * q_row_stride + (size_t)h * D + ch * 8, r < n_rows);
    }
    auto load_page = [&](int step, bool values) {           // K or V of this CTA's block `step` into buffer step & 1
        if (step >= n_steps) return;
        const int blk = blk_lo + grp + step * NG;
        int page = (blk < max_blocks) ? table[blk] : -1;
        const bool ok = (page >= 0 && page < n_pages);
        if (!ok) { if (gt == 0 && err) atomicExch(err, 3); page = 0; }
        const __nv_bfloat16* src = (values ? vpages : kpages) + (size_t)page * page_stride + (size_t)hk * BN * D;
        const uint32_t dst = ta_u32(values ? sV : sK) + (step & 1) * TA_KV_BYTES;
        for (int c = gt; c < BN * 8; c += TA_THREADS) {
            const int r = c >> 3, ch = c & 7;
            ta_cp_async16(dst + r * 128 + ((ch ^ (r & 7)) << 4), src + r * D + ch * 8, ok);
        }
    };
    // copy groups, always in this order: [Q, K(0)], [K(1)], [V(0)], then per step i: [K(i+2)], [V(i+1)]
    load_page(0, false);
    ta_commit_group();
    load_page(1, false);
    ta_commit_group();
    load_page(0, true);
    ta_commit_group();
    ta_wait_group<2>();                                     // Q and K(0) have landed
    ta_fence_async_smem();
    ta_fence_before();
    __syncthreads();                                        // Q, K(0), the barriers and the allocation
    ta_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_p = &abort_flag;
    const uint32_t bar_s = ta_u32(&bars[0]), bar_pv = ta_u32(&bars[3]);

    // ---- this thread's query row
    const int row = gt;
    const int pos_r = pos0 + row;
    const int lo_r = (window > 0) ? pos_r - window + 1 : 0;
    const uint32_t t_s = tmem_base + ((uint32_t)(warp * 32) << 16);         // this warp's 32 lanes; scores in columns 0..63
    const uint32_t t_pv = t_s + 64;                                         // P V in columns 64..127
    float m = -INFINITY, l = 0.f;
    float2 o[D / 2];                                        // the row's output sums, in pairs (packed float32 arithmetic)
#pragma unroll
    for (int d = 0; d < D / 2; ++d) o[d] = make_float2(0.f, 0.f);
    uint32_t phase_s = 0, phase_pv = 0;
    bool ok = !*abort_p;
    const uint64_t dq = ta_desc(ta_u32(sQ)), dp = ta_desc(ta_u32(sP));
    auto issue_s = [&](int step) {                          // S = Q K(step)^T: +32 bytes per k step, +2 in the descriptors' units
        ta_fence_after();
        const uint64_t dk = ta_desc(ta_u32(sK) + (step & 1) * TA_KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) ta_mma(tmem_base, dq + 2 * k, dk + 2 * k, IDESC_S, k > 0 ? 1u : 0u);
        ta_commit(bar_s);
    };
    if (ok && n_steps > 0 && gt == 0) issue_s(0);

    // The steps overlap: while the threads work on the scores of block i, the tensor cores already multiply Q with
    // K(i+1) (the scores of block i are in registers by then) and finish P(i-1) V(i-1), which is only added to the
    // output rows after the probabilities of block i are known.
    for (int step = 0; ok && step < n_steps; ++step) {
        ta_wait(bar_s, phase_s, abort_p);                   // (on failure the flag is set and seen after the next barrier)
        phase_s ^= 1u;
        ta_fence_after();
        uint32_t sv[2][32];
        ta_ld32(t_s, sv[0]);
        ta_ld32(t_s + 32, sv[1]);
        load_page(step + 2, false);                         // K(step)'s buffer is free: the product that read it is done
        ta_commit_group();
        ta_ld_wait();
        ta_wait_group<2>();                                 // K(step + 1) has landed (newer: V(step), K(step + 2))
        ta_fence_async_smem();
        ta_fence_before();
        __syncthreads();                                    // every thread has its scores: the columns may be written again
        if (*abort_p) { ok = false; break; }
        if (gt == 0 && step + 1 < n_steps) issue_s(step + 1);

        // ---- this row's 64 scores: mask, online softmax in base 2 on the raw scores
        const int key0 = (blk_lo + grp + step * NG) * BN;
        float mx = -INFINITY;
        const bool interior = (key0 + BN - 1 <= pos_r) && (key0 >= lo_r);
        if (!interior) {
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                const int key = key0 + j;
                if (!(key <= pos_r && key >= lo_r)) sv[j >> 5][j & 31] = 0xff800000u;     // -inf
            }
        }
#pragma unroll
        for (int j = 0; j < 64; j += 2) mx = ta_max3(mx, __uint_as_float(sv[j >> 5][j & 31]), __uint_as_float(sv[(j + 1) >> 5][(j + 1) & 31]));
        const float mn = fmaxf(m, mx);
        const float use = (mn == -INFINITY) ? 0.f : mn;     // the row sees nothing yet
        const float alpha = ta_exp2((m - use) * scale_log2);
        const float off = -use * scale_log2;
        float2 p_sum = make_float2(0.f, 0.f);              // (even and odd columns apart: two values per instruction)
        const float2 scale2 = make_float2(scale_log2, scale_log2), off2 = make_float2(off, off);
        uint32_t pw[32];                                    // the probabilities, two bf16 per word
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[j >> 5][j & 31]), __uint_as_float(sv[(j + 1) >> 5][(j + 1) & 31])),
                                        scale2, off2);
            const float2 p = make_float2(ta_exp2(x.x), ta_exp2(x.y));
            p_sum = __fadd2_rn(p_sum, p);
            pw[j >> 1] = vm_pack_bf16(p.x, p.y);
        }
        l = l * alpha + (p_sum.x + p_sum.y);
        m = mn;
        // ---- the previous block's P V is done by now: add it, then rescale; its P tile and its V buffer are free
        if (step > 0) {
            ta_wait(bar_pv, phase_pv, abort_p);
            phase_pv ^= 1u;
            ta_fence_after();
            ta_ld32(t_pv, sv[0]);
            ta_ld32(t_pv + 32, sv[1]);
            ta_ld_wait();
#pragma unroll
            for (int d = 0; d < D; d += 2)
                o[d >> 1] = __fadd2_rn(o[d >> 1], make_float2(__uint_as_float(sv[d >> 5][d & 31]), __uint_as_float(sv[(d + 1) >> 5][(d + 1) & 31])));
        }
        load_page(step + 1, true);                          // V(step + 1) into the buffer V(step - 1) was in
        ta_commit_group();
        if (alpha != 1.f) {
            const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
            for (int d = 0; d < D / 2; ++d) o[d] = __fmul2_rn(o[d], alpha2);
        }
        unsigned char* prow = sP + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)                         // eight probabilities (16 bytes) per store, swizzled like the rest
            *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
        ta_wait_group<2>();                                 // V(step) has landed (newer: K(step + 2), V(step + 1))
        ta_fence_async_smem();                              // P and V are read by the tensor cores
        ta_fence_before();
        __syncthreads();
        if (*abort_p) { ok = false; break; }
        if (gt == 0) {                                      // P: +32 bytes per 16 keys; V: 16 key rows = 2048 bytes = +128
            ta_fence_after();
            const uint64_t dv = ta_desc(ta_u32(sV) + (step & 1) * TA_KV_BYTES);
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) ta_mma(tmem_base + 64, dp + 2 * k, dv + 128 * k, IDESC_PV, k > 0 ? 1u : 0u);
            ta_commit(bar_pv);
        }
    }
    if (ok && n_steps > 0) {                                // the last block's P V
        ta_wait(bar_pv, phase_pv, abort_p);
        ta_fence_after();
        uint32_t sv[2][32];
        ta_ld32(t_pv, sv[0]);
        ta_ld32(t_pv + 32, sv[1]);
        ta_ld_wait();
#pragma unroll
        for (int d = 0; d < D; d += 2)
            o[d >> 1] = __fadd2_rn(o[d >> 1], make_float2(__uint_as_float(sv[d >> 5][d & 31]), __uint_as_float(sv[(d + 1) >> 5][(d + 1) & 31])));
    }
    ta_wait_group<0>();
    ta_fence_before();
    __syncthreads();
    if (*abort_p) ok = false;

    if (NC == 1) {
        if (ok && row < n_rows) {
            const float inv = 1.f / l;
            __nv_bfloat16* orow = out + ((size_t)(t0 + row) * H + h) * D;
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                uint4 w;
                w.x = vm_pack_bf16(o[4 * c].x * inv, o[4 * c].y * inv); w.y = vm_pack_bf16(o[4 * c + 1].x * inv, o[4 * c + 1].y * inv);
                w.z = vm_pack_bf16(o[4 * c + 2].x * inv, o[4 * c + 2].y * inv); w.w = vm_pack_bf16(o[4 * c + 3].x * inv, o[4 * c + 3].y * inv);
                *reinterpret_cast<uint4*>(orow + 8 * c) = w;
            }
        }
    } else {
        // ---- the cluster's CTAs exchange their rows: CTA c joins and stores the rows r of the tile with r % NC == c.  Every CTA's K, V and P buffers are free once all CTAs are past this barrier; they receive the rows
        // as xch[source CTA][row][TA_RW].  (A CTA that gave up still takes part in the barriers; its rows are garbage,
        // the error word says so.)
        constexpr int RPR = (TA_BM + NC - 1) / NC;                      // rows joined per CTA: row r belongs to CTA r % NC
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        {
            const unsigned dest = (unsigned)(row % NC);
            const uint32_t local = ta_u32(sK) + (uint32_t)(((grp * RPR) + (row / NC)) * TA_RW * 4);
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(dest));
#pragma unroll
            for (int c = 0; c < D / 4; ++c)
                asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote + 16 * c), "f"(o[2 * c].x), "f"(o[2 * c].y),
                             "f"(o[2 * c + 1].x), "f"(o[2 * c + 1].y) : "memory");
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote + 4 * D), "f"(m), "f"(l), "f"(0.f), "f"(0.f) : "memory");
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        {
            constexpr int CPT = D / 2;                                  // two threads share a row, 32 columns each
            const int r = tid >> 1, c0 = (tid & 1) * CPT;
            const int trow = r * NC + grp;                              // the row's place in the tile
            if (!*abort_p && r < RPR && trow < n_rows) {
                const float* xch = reinterpret_cast<const float*>(sK);
                float M = -INFINITY;
#pragma unroll
                for (int g = 0; g < NC; ++g) M = fmaxf(M, xch[(size_t)(g * RPR + r) * TA_RW + D]);
                const float u = (M == -INFINITY) ? 0.f : M;
                float acc[CPT], L = 0.f;
#pragma unroll
                for (int d = 0; d < CPT; ++d) acc[d] = 0.f;
#pragma unroll
                for (int g = 0; g < NC; ++g) {
                    const float* src = xch + (size_t)(g * RPR + r) * TA_RW;
                    const float f = ta_exp2((src[D] - u) * scale_log2);
                    L += src[D + 1] * f;
#pragma unroll
                    for (int d = 0; d < CPT; ++d) acc[d] += src[c0 + d] * f;
                }
                const float inv = 1.f / L;
                __nv_bfloat16* orow = out + ((size_t)(t0 + trow) * H + h) * D + c0;
#pragma unroll
                for (int c = 0; c < CPT / 8; ++c) {
                    uint4 w;
                    w.x = vm_pack_bf16(acc[8 * c] * inv, acc[8 * c + 1] * inv); w.y = vm_pack_bf16(acc[8 * c + 2] * inv, acc[8 * c + 3] * inv);
                    w.z = vm_pack_bf16(acc[8 * c + 4] * inv, acc[8 * c + 5] * inv); w.w = vm_pack_bf16(acc[8 * c + 6] * inv, acc[8 * c + 7] * inv);
                    *reinterpret_cast<uint4*>(orow + 8 * c) = w;
                }
            }
        }
        // nobody leaves while a peer may still write into its shared memory: the second barrier above is past all writes
    }
    if (!ok && tid == 0 && err) atomicExch(err, 4);
    ta_fence_before();
    __syncthreads();
    if (tid < 32) {
        ta_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(TA_TMEM_COLS) : "memory");
    }
}

template <int NC>
int ta_launch(int n_tiles, int H, cudaStream_t stream, const __nv_bfloat16* q, int q_row_stride, const __nv_bfloat16* kpages,
              const __nv_bfloat16* vpages, const int* block_table, int max_blocks, const int* positions, const int* cu_tokens,
              int B, __nv_bfloat16* out, int Hkv, float scale_log2, int window, int n_pages, int* err) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles * NC, H); cfg.blockDim = dim3(TA_THREADS); cfg.dynamicSmemBytes = TA_SMEM; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = NC; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = NC > 1 ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attn_prefill_tc_kernel<NC>, q, q_row_stride, kpages, vpages, block_table, max_blocks,
                                       positions, cu_tokens, B, out, H, Hkv, scale_log2, window, n_pages, err);
    if (e != cudaSuccess) return (int)e;
    return vm_launch_status();
}

}  // namespace

// n_tiles = sum over the step's sequences of ceil(new tokens / 128), computed by the host.  Head size 64 only;
// out [T, H*64] must be 16-byte aligned, q rows too (q_row_stride % 8 == 0).  groups (1 to 4): CTAs of a cluster
// that take a tile's key blocks in turn; more for steps whose tiles see many keys.
VM_API int vm_attention_prefill_tc_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                        const int* block_table, int max_blocks, const int* positions, const int* cu_tokens,
                                        int B, int n_tiles, void* out, int H, int Hkv, int D, float scale, int window,
                                        int n_pages, int* err, int groups, cudaStream_t stream) {
    if (n_tiles <= 0 || B <= 0) return 0;
    if (D != TA_D || H <= 0 || Hkv <= 0 || H % Hkv != 0 || (q_row_stride % 8) != 0) return VM_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(kpages) |
         reinterpret_cast<uintptr_t>(vpages)) & 15) return VM_ERR_UNSUPPORTED;
    const float sl = scale * 1.4426950408889634f;
    const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)kpages, *vv = (const __nv_bfloat16*)vpages;
    if (groups >= 4)
        return ta_launch<4>(n_tiles, H, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, cu_tokens, B,
                            (__nv_bfloat16*)out, Hkv, sl, window, n_pages, err);
    if (groups == 3)
        return ta_launch<3>(n_tiles, H, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, cu_tokens, B,
                            (__nv_bfloat16*)out, Hkv, sl, window, n_pages, err);
    if (groups >= 2)
        return ta_launch<2>(n_tiles, H, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, cu_tokens, B,
                            (__nv_bfloat16*)out, Hkv, sl, window, n_pages, err);
    return ta_launch<1>(n_tiles, H, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, cu_tokens, B,
                        (__nv_bfloat16*)out, Hkv, sl, window, n_pages, err);
}
