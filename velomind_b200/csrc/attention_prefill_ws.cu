// Prefill attention for bfloat16 and head size 64 on the fifth-generation tensor cores, warp-specialised: causal
// (optionally windowed) attention of the step's new tokens over the paged cache, online softmax in float32.
//
// Arithmetic as in attention_generic.cu (reference: examples/common/llama/llama_graph.cpp:97-103,
// src/cpu/ops/fused_attention.cpp:84-135).  What a key block costs on this GPU is its softmax (64 exponentials per row go
// through the special-function units) and the latencies between the steps, not its two products, so the kernel keeps
// every scheduler of an SM busy with softmax rows of several tiles and takes everything else off those warps:
//
//   * A CTA owns NT tiles (2 or 3) of 128 query rows that share one kv head: NH query heads of the group at the same
//     rows, times NR consecutive row tiles.  Keys and values are fetched once for all of them.
//   * Warps 0 .. 4 NT - 1 are softmax warps: thread r of a tile owns query row r, tensor-memory lane r holds its scores
//     and its output sums.  Warps 4 NT .. 5 NT - 1 issue the products, one warp per tile (an mbarrier wait costs a
//     couple of hundred cycles here even when the barrier is complete, so the tiles' chains of waits run side by side).
//     Warp 5 NT copies: the query tiles, then a key page and its value page per block arrive through TMA (tensor maps
//     over the query rows and the page pools, 128-byte swizzle), the pages into a ring of four stages.  In these warps
//     every lane walks the loop and one elected lane issues.
//   * Per key block (one cache page of 64 keys) and tile:  S = Q K^T (M 128, N 64, K 64: four tcgen05.mma) into the
//     tile's score columns; the row's thread reads its 64 scores, and as soon as they are in registers the scores of
//     the NEXT block are multiplied into the same columns while the thread masks, exponentiates and writes the
//     probabilities as bf16 into the tile's P buffer; O += P V (V is the MN-major B operand) accumulates in tensor
//     memory, so a row's thread touches its output only at the end, or when its maximum moved far.
//   * The maximum used in the exponent is only raised when the new one exceeds it by more than 8 in the exponent's
//     units (the probabilities then stay below 2^8; numerator and denominator carry the same factor, so the result is
//     the same); raising it rescales the row's sums in tensor memory.
//   * The tiles of a long prompt see very different numbers of keys.  A cluster of NC CTAs (1 to 8) takes a PAIR of
//     row-tile groups, the i-th from the end and the i-th from the start, and deals its CTAs out to the two groups in
//     proportion to their key blocks; the n CTAs of a group take its key blocks r, r + n, ... .  Every CTA of the launch
//     thus walks about the same number of key blocks, with one set of query tiles.  At the end the CTAs of a group
//     exchange their rows (sums, maximum, denominator): each lays its rows out in its own shared memory and sends CTA c
//     the rows c joins (a contiguous range per tile) with one bulk copy per tile into c's shared memory, completion
//     counted on c's mbarrier; c joins and stores its rows.
//
// Every mbarrier wait is bounded.  When one gives up, the CTA raises error word 4, still takes part in its cluster's
// barriers, waits (bounded) for its copies in flight, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "tc05.cuh"

namespace {

constexpr int WS_BM = 128, WS_BN = 64, WS_D = 64, WS_STAGES = 4;
static_assert(WS_BN == VM_PAGE_TOKENS, "a key block is one page");
constexpr int WS_QTILE = WS_BM * 128;                      // bytes of a Q or P tile (128 rows of 128 bytes)
constexpr int WS_KVTILE = WS_BN * 128;                     // bytes of a K or V page of one head
constexpr int WS_RW = WS_D + 4;                            // floats of an exchanged row: sums, maximum, denominator, padding
constexpr int WS_MAX_NC = 8;
constexpr int WS_INLINE_SEQS = 16;

struct WsParams {
    const __nv_bfloat16* q; int q_row_stride;
    const int* block_table; int max_blocks;
    const int* positions; const int* cu_tokens; int B;
    __nv_bfloat16* out; int H, Hkv, NH;
    float scale_log2, rescale_gap;                         // rescale_gap: how far (in raw scores) the maximum may run ahead
    int window, n_pages; int* err;
    int n_inline;                                          // > 0: the offsets of cu_tokens ride along in inline_cu (they are shape, known
    int inline_cu[WS_INLINE_SEQS + 1];                     //      to the host at launch): the walk over the sequences loads nothing
};

struct WsSlot { int valid, head, t0, n_rows, pos0, blk_lo, blk_hi; };

// Tile `s` of row-tile group `rtg`: NH heads at the same rows, then the next row tile.
__device__ __forceinline__ WsSlot ws_slot(const WsParams& p, int NR, int rtg, int s, int head0, int tok_a, int tok_b, int n_rt, int pos_a) {
    WsSlot sl;
    const int rt = rtg * NR + s / p.NH;
    sl.valid = rt < n_rt;
    sl.head = head0 + s % p.NH;
    sl.t0 = tok_a + rt * WS_BM;
    sl.n_rows = min(WS_BM, tok_b - sl.t0);
    sl.pos0 = pos_a + rt * WS_BM;                          // a sequence's new tokens have consecutive positions
    const int hi = sl.pos0 + sl.n_rows - 1;
    const int lo = (p.window > 0 && sl.pos0 - p.window + 1 > 0) ? sl.pos0 - p.window + 1 : 0;
    sl.blk_lo = lo / WS_BN;
    sl.blk_hi = hi / WS_BN;
    return sl;
}

__device__ __forceinline__ void ws_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// bounded wait that ignores the give-up flag (for the copies still in flight after giving up)
__device__ __forceinline__ void ws_drain_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < TA_WAIT_LIMIT; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return;
    }
}

// rows of a tile that CTA c of a cluster of nc joins: a contiguous range of up to ceil(128 / nc)
__host__ __device__ constexpr int ws_rpr(int nc) { return (WS_BM + nc - 1) / nc; }
__device__ __forceinline__ int ws_own_rows(int c, int rpr) { const int n = WS_BM - c * rpr; return n < 0 ? 0 : (n > rpr ? rpr : n); }

template <int NT> __host__ __device__ constexpr int ws_threads() { return (5 * NT + 1) * 32; }
template <int NT> __host__ __device__ constexpr int ws_tile_bytes() { return 2 * NT * WS_QTILE + 2 * WS_STAGES * WS_KVTILE; }
template <int NT> __host__ __device__ constexpr int ws_stage_bytes() { return NT * WS_BM * WS_RW * 4; }            // a CTA's own rows, laid out for sending
__host__ __device__ constexpr int ws_max_rows_in() { int m = 0; for (int c = 2; c <= WS_MAX_NC; ++c) { const int v = c * ws_rpr(c); if (v > m) m = v; } return m; }
template <int NT> __host__ __device__ constexpr int ws_recv_bytes() { return NT * ws_max_rows_in() * WS_RW * 4; }  // the rows it receives
template <int NT> __host__ __device__ constexpr int ws_smem_bytes() {
    return (ws_tile_bytes<NT>() > ws_stage_bytes<NT>() + ws_recv_bytes<NT>() ? ws_tile_bytes<NT>() : ws_stage_bytes<NT>() + ws_recv_bytes<NT>()) + 512;
}
static_assert(ws_smem_bytes<3>() <= 227 * 1024, "three tiles per CTA must fit an SM's shared memory");

template <int NT>
__global__ void __launch_bounds__((5 * NT + 1) * 32) __maxnreg__(NT <= 2 ? 168 : 128)
attn_prefill_ws_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const WsParams p) {
    constexpr int ST = WS_STAGES, NSOFT = NT * 128, D = WS_D, BN = WS_BN;
    constexpr uint32_t TMEM_COLS = NT == 1 ? 128u : (NT == 2 ? 256u : 512u);        // per tile: scores 0..63, output sums 64..127
    // instruction descriptors: float32 accumulate (bits 4-5 = 1), A and B bf16 (bits 7-9 and 10-12 = 1), B MN-major
    // (bit 16) for P V, N >> 3 in bits 17-22, M >> 4 in bits 24-28
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(WS_BM >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(WS_BM >> 4) << 24);
    constexpr int B_QFULL = 0, B_SFULL = NT, B_SFREE = 2 * NT, B_PFULL = 3 * NT, B_PVDONE = 4 * NT;
    constexpr int B_KVFULL = 5 * NT, B_KVEMPTY = B_KVFULL + ST, B_XCH = B_KVEMPTY + ST, N_BARS = B_XCH + 1;
    static_assert(N_BARS * 8 + 16 <= 512, "the bookkeeping behind the tiles");
    constexpr int TILE_BYTES = ws_tile_bytes<NT>(), STAGE_BYTES = ws_stage_bytes<NT>();
    constexpr int BOOK = ws_smem_bytes<NT>() - 512;                // the bookkeeping sits behind everything else

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* sQ = smem_raw;                                   // [NT][128 rows][128 bytes]
    unsigned char* sP = sQ + NT * WS_QTILE;                         // [NT][128 rows][128 bytes]
    unsigned char* sKV = sP + NT * WS_QTILE;                        // [ST][K: 64 keys x 128 bytes | V: 64 keys x 128 bytes]
    static_assert(TILE_BYTES == 2 * NT * WS_QTILE + ST * 2 * WS_KVTILE, "layout");
    float* xstage = reinterpret_cast<float*>(smem_raw);             // after a pass: [NT][128 rows][WS_RW], this CTA's rows
    float* xrecv = reinterpret_cast<float*>(smem_raw + STAGE_BYTES);   // [source CTA][NT][rows it joins][WS_RW]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + BOOK);
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + N_BARS);
    int& abort_flag = *reinterpret_cast<int*>(bars + N_BARS + 1);
    const uint32_t bar0 = ta_u32(bars);
#define WS_BAR(i) (bar0 + 8u * (uint32_t)(i))

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);          // (a value the compiler knows to be the same in all lanes)
    unsigned ncu = 1, grpu = 0;
    asm("mov.u32 %0, %%cluster_nctarank;" : "=r"(ncu));
    asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(grpu));
    const int NC = (int)ncu, grp = (int)grpu;

    // ---- which pair of row-tile groups of which sequence
    const int G = p.H / p.Hkv, NR = NT / p.NH;
    int unit = (int)blockIdx.x / NC, seq = 0, tok_a = 0, tok_b = 0, n_rt = 0, n_rtg = 0;
    for (; seq < p.B; ++seq) {
        if (p.n_inline > 0) { tok_a = p.inline_cu[seq]; tok_b = p.inline_cu[seq + 1]; }
        else { tok_a = p.cu_tokens[seq]; tok_b = p.cu_tokens[seq + 1]; }
        n_rt = (tok_b - tok_a + WS_BM - 1) / WS_BM;
        n_rtg = (n_rt + NR - 1) / NR;
        const int units = (n_rtg + 1) / 2;
        if (unit < units) break;
        unit -= units;
    }
    if (seq >= p.B) return;                                 // (before any barrier or allocation: the whole cluster leaves)
    // (broadcasts: every lane holds the same values anyway; this way the compiler knows it too)
    unit = __shfl_sync(0xffffffffu, unit, 0); seq = __shfl_sync(0xffffffffu, seq, 0);
    tok_a = __shfl_sync(0xffffffffu, tok_a, 0); tok_b = __shfl_sync(0xffffffffu, tok_b, 0);
    n_rt = __shfl_sync(0xffffffffu, n_rt, 0); n_rtg = __shfl_sync(0xffffffffu, n_rtg, 0);
    const int per_kv = G / p.NH;
    const int hk = (int)blockIdx.y / per_kv, head0 = hk * G + ((int)blockIdx.y % per_kv) * p.NH;
    const int pos_a = __shfl_sync(0xffffffffu, p.positions[tok_a], 0);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    // ---- the cluster's two groups and this CTA's place: CTAs 0 .. nA-1 walk group A (more keys), the others group B
    int blk_lo, blk_hi;
    auto block_range = [&](int g) {
        blk_lo = 0x7fffffff; blk_hi = -1;
#pragma unroll
        for (int s = 0; s < NT; ++s) {
            const WsSlot sl = ws_slot(p, NR, g, s, head0, tok_a, tok_b, n_rt, pos_a);
            if (sl.valid) { blk_lo = min(blk_lo, sl.blk_lo); blk_hi = max(blk_hi, sl.blk_hi); }
        }
    };
    const int rtgA = n_rtg - 1 - unit, rtgB = unit;
    int nA = NC;
    if (rtgA != rtgB && NC > 1) {
        block_range(rtgB);
        const int bB = blk_hi - blk_lo + 1;
        block_range(rtgA);
        const int bA = blk_hi - blk_lo + 1;
        int nB = (NC * bB + (bA + bB) / 2) / (bA + bB);
        nB = nB < 1 ? 1 : (nB > NC - 1 ? NC - 1 : nB);
        nA = NC - nB;
    }
    // (a cluster of one CTA walks its two groups one after the other: see the loop below)
    const int n_pass = (rtgA != rtgB && NC == 1) ? 2 : 1;
    const bool in_a = grp < nA;
    const int n_grp = in_a ? nA : NC - nA;                  // CTAs that share this CTA's group
    const int rank = in_a ? grp : grp - nA, base = in_a ? 0 : nA;
    const int RPR = ws_rpr(n_grp);                          // rows of a tile that one CTA of the group joins

    if (tid == 0) {
        abort_flag = (ta_u32(smem_raw) & 1023u) ? 1 : 0;    // misaligned tiles would give wrong sums: give up instead
#pragma unroll
        for (int s = 0; s < NT; ++s) {
            ta_bar_init(WS_BAR(B_QFULL + s), 1); ta_bar_init(WS_BAR(B_SFULL + s), 1); ta_bar_init(WS_BAR(B_SFREE + s), 4);
            ta_bar_init(WS_BAR(B_PFULL + s), 4); ta_bar_init(WS_BAR(B_PVDONE + s), 1);
        }
#pragma unroll
        for (int st = 0; st < ST; ++st) { ta_bar_init(WS_BAR(B_KVFULL + st), 1); ta_bar_init(WS_BAR(B_KVEMPTY + st), NT); }
        ta_bar_init(WS_BAR(B_XCH), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5 * NT) {                                   // one warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ta_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    ta_fence_before();
    __syncthreads();
    ta_fence_after();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_slot, 0);
    volatile int* abort_p = &abort_flag;
    bool ok = !*abort_p;

    // state that outlives a pass: how often each barrier has been used (its parity follows)
    uint32_t n_sfull = 0, n_pvdone = 0;                     // softmax threads: waits done on their tile's barriers
    uint32_t n_kv = 0, n_kv_done = 0;                       // copy warp: pages sent; product warps: pages awaited / released
    uint32_t s_cnt = 0, pv_cnt = 0, q_cnt = 0;              // product warps: products issued for their tile, query tiles awaited

    for (int ps = 0; ps < n_pass; ++ps) {
        const int rtg = (n_pass == 2) ? (ps == 0 ? rtgA : rtgB) : (in_a ? rtgA : rtgB);
        block_range(rtg);
        const int n_blocks = blk_hi - blk_lo + 1;
        const int n_my = n_blocks > rank ? (n_blocks - rank + n_grp - 1) / n_grp : 0;      // this CTA's blocks: rank, rank + n_grp, ...

        // this thread's row (softmax warps); the sums it ends the pass with
        const int my_s = warp >> 2, row = (warp & 3) * 32 + lane;
        uint32_t o[2][32];                                  // (as the tensor memory hands them out: float32 bit patterns)
        float m_ref = -INFINITY, l = 0.f;
        bool my_valid = false;

        if (warp < 4 * NT) {
            // =============================================================== softmax warps
            const WsSlot sl = ws_slot(p, NR, rtg, my_s, head0, tok_a, tok_b, n_rt, pos_a);
            my_valid = sl.valid;
            const uint32_t t_s = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)my_s * 128u;
            const uint32_t t_o = t_s + 64u;
            const int pos_r = sl.pos0 + row;
            const int lo_r = (p.window > 0) ? pos_r - p.window + 1 : 0;
            bool has_o = false, pending = false;            // a P V has been issued in this pass; its completion is not yet awaited
            for (int it = 0; ok && it < n_my; ++it) {
                const int blk = blk_lo + rank + it * n_grp;
                if (!(sl.valid && blk >= sl.blk_lo && blk <= sl.blk_hi)) continue;
                ok = __all_sync(0xffffffffu, ta_spin(WS_BAR(B_SFULL + my_s), n_sfull & 1u, abort_p));
                if (!ok) break;
                ++n_sfull;
                ta_fence_after();
                uint32_t sv[2][32];
                ta_ld32(t_s, sv[0]);
                ta_ld32(t_s + 32, sv[1]);
                ta_ld_wait();
                ta_fence_before();
                __syncwarp();
                if (lane == 0) ta_bar_arrive(WS_BAR(B_SFREE + my_s));          // the score columns may be written again
                // ---- mask, maximum
                const int key0 = blk * BN;
                if (!((key0 + BN - 1 <= pos_r) && (key0 >= lo_r))) {
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        const int key = key0 + j;
                        if (!(key <= pos_r && key >= lo_r)) sv[j >> 5][j & 31] = 0xff800000u;     // -inf
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};        // four chains: the maxima do not wait for one another
#pragma unroll
                for (int j = 0; j < 64; j += 8) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        mx4[c] = ta_max3(mx4[c], __uint_as_float(sv[(j + 2 * c) >> 5][(j + 2 * c) & 31]), __uint_as_float(sv[(j + 2 * c + 1) >> 5][(j + 2 * c + 1) & 31]));
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                // ---- the reference maximum moves only when the new one is far ahead (or it is the first)
                const bool grow = mx > m_ref + p.rescale_gap;
                float alpha = 1.f;
                if (grow) { alpha = ta_exp2((m_ref - mx) * p.scale_log2); l *= alpha; m_ref = mx; }
                const bool rescale = has_o && __any_sync(0xffffffffu, grow);
                // ---- probabilities in base 2 on the raw scores
                const float off = (m_ref == -INFINITY) ? 0.f : -m_ref * p.scale_log2;
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), off2 = make_float2(off, off);
                float2 p_sum = make_float2(0.f, 0.f), p_sum2 = make_float2(0.f, 0.f);
                uint32_t pw[32];
#pragma unroll
                for (int j = 0; j < 64; j += 4) {
                    const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(sv[j >> 5][j & 31]), __uint_as_float(sv[(j + 1) >> 5][(j + 1) & 31])), scale2, off2);
                    const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(sv[(j + 2) >> 5][(j + 2) & 31]), __uint_as_float(sv[(j + 3) >> 5][(j + 3) & 31])), scale2, off2);
                    const float2 e0 = make_float2(ta_exp2(x0.x), ta_exp2(x0.y)), e1 = make_float2(ta_exp2(x1.x), ta_exp2(x1.y));
                    p_sum = __fadd2_rn(p_sum, e0);
                    p_sum2 = __fadd2_rn(p_sum2, e1);
                    pw[j >> 1] = vm_pack_bf16(e0.x, e0.y);
                    pw[(j >> 1) + 1] = vm_pack_bf16(e1.x, e1.y);
                }
                l += (p_sum.x + p_sum.y) + (p_sum2.x + p_sum2.y);
                if (pending) {                              // the previous block's P V is done: it has read the P tile, the sums are whole
                    ok = __all_sync(0xffffffffu, ta_spin(WS_BAR(B_PVDONE + my_s), n_pvdone & 1u, abort_p));
                    if (!ok) break;
                    ++n_pvdone; pending = false;
                }
                if (rescale) {                              // (after the probabilities: the scores' registers are free by now)
                    ta_fence_after();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t ov[32];
                        ta_ld32(t_o + 32 * half, ov);
                        ta_ld_wait();
#pragma unroll
                        for (int d = 0; d < 32; ++d) ov[d] = __float_as_uint(__uint_as_float(ov[d]) * alpha);
                        ta_st32(t_o + 32 * half, ov);
                    }
                    ta_st_wait();
                    ta_fence_before();
                }
                unsigned char* prow = sP + my_s * WS_QTILE + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
                ta_fence_async_smem();                      // P is read by the tensor cores
                __syncwarp();
                if (lane == 0) ta_bar_arrive(WS_BAR(B_PFULL + my_s));
                has_o = true; pending = true;
            }
            // ---- the row's sums
            if (ok && pending) {
                ok = __all_sync(0xffffffffu, ta_spin(WS_BAR(B_PVDONE + my_s), n_pvdone & 1u, abort_p));
                if (ok) { ++n_pvdone; pending = false; }
            }
            if (ok && has_o) {
                ta_fence_after();
                ta_ld32(t_o, o[0]);
                ta_ld32(t_o + 32, o[1]);
                ta_ld_wait();
                ta_fence_before();
            } else {
#pragma unroll
                for (int d = 0; d < 32; ++d) o[0][d] = o[1][d] = 0u;
            }
            if (n_grp == 1 && ok && sl.valid && row < sl.n_rows) {
                const float inv = 1.f / l;
                __nv_bfloat16* orow = p.out + ((size_t)(sl.t0 + row) * p.H + sl.head) * D;
#pragma unroll
                for (int c = 0; c < D / 8; ++c) {
                    const uint32_t* v = &o[c >> 2][(c & 3) * 8];
                    uint4 w;
                    w.x = vm_pack_bf16(__uint_as_float(v[0]) * inv, __uint_as_float(v[1]) * inv);
                    w.y = vm_pack_bf16(__uint_as_float(v[2]) * inv, __uint_as_float(v[3]) * inv);
                    w.z = vm_pack_bf16(__uint_as_float(v[4]) * inv, __uint_as_float(v[5]) * inv);
                    w.w = vm_pack_bf16(__uint_as_float(v[6]) * inv, __uint_as_float(v[7]) * inv);
                    *reinterpret_cast<uint4*>(orow + 8 * c) = w;
                }
            }
        } else if (warp < 5 * NT) {
            // =============================================================== products of tile ts (the whole warp walks the
            // loop; one elected lane issues)
            const int ts = warp - 4 * NT;
            const WsSlot sl = ws_slot(p, NR, rtg, ts, head0, tok_a, tok_b, n_rt, pos_a);
            if (ok) {
                if (sl.valid) ok = __all_sync(0xffffffffu, ta_spin(WS_BAR(B_QFULL + ts), q_cnt & 1u, abort_p));
                ta_fence_after();
                const uint64_t dq = ta_desc(ta_u32(sQ) + ts * WS_QTILE), dp = ta_desc(ta_u32(sP) + ts * WS_QTILE);
                const uint32_t t_s = tmem_base + (uint32_t)ts * 128u, t_o = t_s + 64u;
                bool first_pv = true;
                auto issue_s = [&](int it) -> bool {        // S = Q K(it)^T, once the page has landed
                    const int blk = blk_lo + rank + it * n_grp;
                    const uint32_t st = n_kv % ST;
                    if (!__all_sync(0xffffffffu, ta_spin(WS_BAR(B_KVFULL + st), (n_kv / ST) & 1u, abort_p))) return false;
                    ++n_kv;
                    if (!(sl.valid && blk >= sl.blk_lo && blk <= sl.blk_hi)) return true;
                    if (s_cnt > 0 && !__all_sync(0xffffffffu, ta_spin(WS_BAR(B_SFREE + ts), (s_cnt - 1) & 1u, abort_p))) return false;
                    ta_fence_after();                       // (the tile's previous scores are in their threads' registers)
                    const uint64_t dk = ta_desc(ta_u32(sKV) + st * 2 * WS_KVTILE);
                    if (ta_elect_one()) {
#pragma unroll
                        for (int k = 0; k < D / 16; ++k) ta_mma(t_s, dq + 2 * k, dk + 2 * k, IDESC_S, k > 0 ? 1u : 0u);
                        ta_commit(WS_BAR(B_SFULL + ts));
                    }
                    ++s_cnt;
                    return true;
                };
                auto issue_pv = [&](int it) -> bool {       // O += P V(it); the page is released once every tile's product is done
                    const int blk = blk_lo + rank + it * n_grp;
                    const uint32_t st = n_kv_done % ST;
                    if (sl.valid && blk >= sl.blk_lo && blk <= sl.blk_hi) {
                        if (!__all_sync(0xffffffffu, ta_spin(WS_BAR(B_PFULL + ts), pv_cnt & 1u, abort_p))) return false;
                        ta_fence_after();
                        const uint64_t dv = ta_desc(ta_u32(sKV) + st * 2 * WS_KVTILE + WS_KVTILE);
                        if (ta_elect_one()) {
                            if (first_pv) {
#pragma unroll
                                for (int k = 0; k < BN / 16; ++k) ta_mma(t_o, dp + 2 * k, dv + 128 * k, IDESC_PV, k > 0 ? 1u : 0u);
                            } else {
#pragma unroll
                                for (int k = 0; k < BN / 16; ++k)   // P: +32 bytes per 16 keys; V: 16 key rows = 2048 bytes = +128
                                    ta_mma(t_o, dp + 2 * k, dv + 128 * k, IDESC_PV, 1u);
                            }
                            ta_commit(WS_BAR(B_PVDONE + ts));
                        }
                        ++pv_cnt; first_pv = false;
                    }
                    if (ta_elect_one()) ta_commit(WS_BAR(B_KVEMPTY + st));
                    ++n_kv_done;
                    return true;
                };
                if (ok && n_my > 0) ok = issue_s(0);
                for (int it = 0; ok && it < n_my; ++it) {
                    if (it + 1 < n_my) ok = issue_s(it + 1);
                    if (ok) ok = issue_pv(it);
                }
            }
            q_cnt += sl.valid ? 1u : 0u;
            __syncwarp();
        } else {
            // =============================================================== copies: the key page and the value page of this CTA's
            // blocks (the whole warp walks the loop; one elected lane issues)
            if (ok) {
                // the query tiles (rows past the sequence's end are whatever follows them, or zeros past the last token: such rows
                // are computed and never stored)
#pragma unroll
                for (int s = 0; s < NT; ++s) {
                    const WsSlot sl = ws_slot(p, NR, rtg, s, head0, tok_a, tok_b, n_rt, pos_a);
                    if (sl.valid && ta_elect_one()) {
                        ta_bar_expect_tx(WS_BAR(B_QFULL + s), WS_QTILE);
                        ta_tma_load_2d(ta_u32(sQ) + s * WS_QTILE, &map_q, sl.head * D, sl.t0, WS_BAR(B_QFULL + s));
                    }
                }
                int page_next = -1;
                if (n_my > 0) { const int blk = blk_lo + rank; page_next = (blk < p.max_blocks) ? table[blk] : -1; }
                for (int it = 0; it < n_my; ++it) {
                    int page = page_next;
                    if (it + 1 < n_my) { const int blk = blk_lo + rank + (it + 1) * n_grp; page_next = (blk < p.max_blocks) ? table[blk] : -1; }
                    if (page < 0 || page >= p.n_pages) { if (lane == 0 && p.err) atomicExch(p.err, 3); page = 0; }
                    const int y = (page * p.Hkv + hk) * BN;
                    const uint32_t st = n_kv % ST;
                    if (n_kv >= ST) { ok = __all_sync(0xffffffffu, ta_spin(WS_BAR(B_KVEMPTY + st), (n_kv / ST - 1) & 1u, abort_p)); if (!ok) break; }
                    if (ta_elect_one()) {
                        ta_bar_expect_tx(WS_BAR(B_KVFULL + st), 2 * WS_KVTILE);
                        ta_tma_load_2d(ta_u32(sKV) + st * 2 * WS_KVTILE, &map_k, 0, y, WS_BAR(B_KVFULL + st));
                        ta_tma_load_2d(ta_u32(sKV) + st * 2 * WS_KVTILE + WS_KVTILE, &map_v, 0, y, WS_BAR(B_KVFULL + st));
                    }
                    ++n_kv;
                }
            }
            __syncwarp();
        }

        if (NC > 1) {
            // ---- the CTAs of a group exchange their rows.  Every CTA's tiles are free once all CTAs of the cluster are
            // past the first barrier; the rows this CTA walked go into xstage, the rows it joins arrive in xrecv from the
            // others of its group.  (A CTA that gave up still takes part in the barriers and sends; its rows are garbage,
            // the error word says so.)
            __syncwarp();
            ws_cluster_sync();
            if (n_grp > 1) {
                if (warp < 4 * NT && my_valid) {
                    float4* dst = reinterpret_cast<float4*>(xstage + (size_t)(my_s * WS_BM + row) * WS_RW);
#pragma unroll
                    for (int c = 0; c < D / 4; ++c)
                        dst[c] = make_float4(__uint_as_float(o[c >> 3][(c & 7) * 4]), __uint_as_float(o[c >> 3][(c & 7) * 4 + 1]),
                                             __uint_as_float(o[c >> 3][(c & 7) * 4 + 2]), __uint_as_float(o[c >> 3][(c & 7) * 4 + 3]));
                    dst[D / 4] = make_float4(m_ref, l, 0.f, 0.f);
                }
                ta_fence_async_smem();                      // the rows are read by bulk copies
                __syncthreads();
                int n_valid = 0;
#pragma unroll
                for (int s = 0; s < NT; ++s) n_valid += ws_slot(p, NR, rtg, s, head0, tok_a, tok_b, n_rt, pos_a).valid ? 1 : 0;
                const int my_rows = ws_own_rows(rank, RPR);
                if (tid == 0) ta_bar_expect_tx(WS_BAR(B_XCH), (uint32_t)((n_grp - 1) * n_valid * my_rows * WS_RW * 4));
                if (tid < (n_grp - 1) * NT) {               // one bulk copy per destination CTA and tile
                    const int dest = tid / NT + (tid / NT >= rank ? 1 : 0), s = tid % NT;
                    const int rows = ws_own_rows(dest, RPR);
                    if (rows > 0 && ws_slot(p, NR, rtg, s, head0, tok_a, tok_b, n_rt, pos_a).valid) {
                        const uint32_t src = ta_u32(xstage + (size_t)(s * WS_BM + dest * RPR) * WS_RW);
                        const uint32_t dst_local = ta_u32(xrecv + (size_t)((rank * NT + s) * RPR) * WS_RW);
                        uint32_t dst, rbar;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(dst_local), "r"((unsigned)(base + dest)));
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(WS_BAR(B_XCH)), "r"((unsigned)(base + dest)));
                        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst), "r"(src), "r"((uint32_t)(rows * WS_RW * 4)), "r"(rbar) : "memory");
                    }
                }
                const bool got = __all_sync(0xffffffffu, ta_spin(WS_BAR(B_XCH), 0u, abort_p));
                if (got && warp < 4 * NT && !*abort_p) {
                    const int qd = tid & 3;                                     // four threads share a row, 16 columns each
                    const int r0 = rank * RPR;
                    for (int ri = tid >> 2; ri < NT * my_rows; ri += NSOFT / 4) {
                        const int s2 = ri / my_rows, idx = ri - s2 * my_rows;
                        const int trow = r0 + idx;                              // the row's place in its tile
                        const WsSlot sl = ws_slot(p, NR, rtg, s2, head0, tok_a, tok_b, n_rt, pos_a);
                        if (!sl.valid || trow >= sl.n_rows) continue;
                        const float* mine = xstage + (size_t)(s2 * WS_BM + trow) * WS_RW;
                        const float* theirs = xrecv + (size_t)(s2 * RPR + idx) * WS_RW;       // + source rank * NT * RPR rows
                        const size_t hop = (size_t)NT * RPR * WS_RW;
                        // maxima and denominators of all sources first, then the sums with every source's loads in flight
                        float mg[WS_MAX_NC], fg[WS_MAX_NC];
                        float M = -INFINITY;
#pragma unroll
                        for (int g = 0; g < WS_MAX_NC; ++g) {
                            mg[g] = -INFINITY;
                            if (g < n_grp) { mg[g] = (g == rank) ? mine[D] : theirs[g * hop + D]; M = fmaxf(M, mg[g]); }
                        }
                        const float u = (M == -INFINITY) ? 0.f : M;
                        float acc[16], L = 0.f;
#pragma unroll
                        for (int d = 0; d < 16; ++d) acc[d] = 0.f;
#pragma unroll
                        for (int g = 0; g < WS_MAX_NC; ++g) fg[g] = (g < n_grp) ? ta_exp2((mg[g] - u) * p.scale_log2) : 0.f;
#pragma unroll
                        for (int g = 0; g < WS_MAX_NC; ++g) {
                            if (g < n_grp) {
                                const float* src = (g == rank) ? mine : theirs + g * hop;
                                L += src[D + 1] * fg[g];
                                const float4* s4 = reinterpret_cast<const float4*>(src + qd * 16);
#pragma unroll
                                for (int c = 0; c < 4; ++c) {
                                    const float4 v = s4[c];
                                    acc[4 * c] += v.x * fg[g]; acc[4 * c + 1] += v.y * fg[g]; acc[4 * c + 2] += v.z * fg[g]; acc[4 * c + 3] += v.w * fg[g];
                                }
                            }
                        }
                        const float inv = 1.f / L;
                        __nv_bfloat16* orow = p.out + ((size_t)(sl.t0 + trow) * p.H + sl.head) * D + qd * 16;
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            uint4 w;
                            w.x = vm_pack_bf16(acc[8 * c] * inv, acc[8 * c + 1] * inv); w.y = vm_pack_bf16(acc[8 * c + 2] * inv, acc[8 * c + 3] * inv);
                            w.z = vm_pack_bf16(acc[8 * c + 4] * inv, acc[8 * c + 5] * inv); w.w = vm_pack_bf16(acc[8 * c + 6] * inv, acc[8 * c + 7] * inv);
                            *reinterpret_cast<uint4*>(orow + 8 * c) = w;
                        }
                    }
                }
            }
            __syncwarp();
            ws_cluster_sync();                              // everybody has its rows: every CTA's copies have been read
        }
        if (n_pass > 1) __syncthreads();                     // (a cluster of one: the next pass overwrites the query tiles)
        if (*abort_p) ok = false;
    }

    if (warp == 5 * NT && lane == 0 && *abort_p) {          // gave up: the copies still in flight land before the CTA leaves
        for (uint32_t back = 0; back < (uint32_t)ST && back < n_kv; ++back) { const uint32_t c = n_kv - 1 - back; ws_drain_wait(WS_BAR(B_KVFULL + c % ST), (c / ST) & 1u); }
    }
    if (tid == 0 && *abort_p && p.err) atomicExch(p.err, 4);
    ta_fence_before();
    __syncthreads();
    if (warp == 5 * NT) {
        ta_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
#undef WS_BAR
}

// ---------------------------------------------------------------- host side
typedef CUresult (*WsEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

WsEncodeTiledFn ws_encode_fn() {
    static WsEncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<WsEncodeTiledFn>(ptr);
    }
    return fn;
}

// The page pool of one cache tensor as rows of 64 values: [n_pages * Hkv * 64 keys][64]; a box is one head's page.
// Maps are kept (a step asks for the same two per layer every time).
int ws_page_map(CUtensorMap* out, const void* base, long long rows) {
    struct Entry { const void* base; long long rows; int device; CUtensorMap map; };
    static std::mutex lock;
    static Entry cache[256];
    static int used = 0, next = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return VM_ERR_BAD_ARG;
    std::lock_guard<std::mutex> guard(lock);
    for (int i = 0; i < used; ++i)
        if (cache[i].base == base && cache[i].rows == rows && cache[i].device == dev) { *out = cache[i].map; return 0; }
    WsEncodeTiledFn fn = ws_encode_fn();
    if (fn == nullptr) return VM_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)WS_D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)WS_D * 2};
    cuuint32_t box[2] = {(cuuint32_t)WS_D, (cuuint32_t)WS_BN};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return VM_ERR_BAD_ARG;
    const int at = used < 256 ? used++ : (next++ % 256);
    cache[at] = Entry{base, rows, dev, map};
    *out = map;
    return 0;
}

// The step's query rows [T][H * 64 of q_row_stride values]; a box is one head's 128 rows.
int ws_query_map(CUtensorMap* out, const void* q, long long T, int H, int q_row_stride) {
    struct Entry { const void* q; long long T; int H, stride, device; CUtensorMap map; };
    static std::mutex lock;
    static Entry cache[64];
    static int used = 0, next = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return VM_ERR_BAD_ARG;
    std::lock_guard<std::mutex> guard(lock);
    for (int i = 0; i < used; ++i)
        if (cache[i].q == q && cache[i].T == T && cache[i].H == H && cache[i].stride == q_row_stride && cache[i].device == dev) { *out = cache[i].map; return 0; }
    WsEncodeTiledFn fn = ws_encode_fn();
    if (fn == nullptr) return VM_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)H * WS_D, (cuuint64_t)T};
    cuuint64_t strides[1] = {(cuuint64_t)q_row_stride * 2};
    cuuint32_t box[2] = {(cuuint32_t)WS_D, (cuuint32_t)WS_BM};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return VM_ERR_BAD_ARG;
    const int at = used < 64 ? used++ : (next++ % 64);
    cache[at] = Entry{q, T, H, q_row_stride, dev, map};
    *out = map;
    return 0;
}

// Clusters of `nc` CTAs of this kernel that the GPU holds at once (asked once per size).
template <int NT>
int ws_active_clusters(int nc) {
    static int cached[WS_MAX_NC + 1] = {};
    if (cached[nc] != 0) return cached[nc];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nc * 64, 1); cfg.blockDim = dim3(ws_threads<NT>()); cfg.dynamicSmemBytes = ws_smem_bytes<NT>();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nc; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, attn_prefill_ws_kernel<NT>, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = vm_sm_count() / nc;
        if (n <= 0) n = 1;
    }
    cached[nc] = n;
    return n;
}

template <int NT>
int ws_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const WsParams& p, long long units, int grid_y, int est_blocks, int groups,
              cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_ws_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, ws_smem_bytes<NT>());
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int nc = groups;
    if (nc <= 0) {
        // As many CTAs per cluster as make the step shortest, in key blocks of one CTA (about 1.75 us each, measured): waves of
        // clusters times what a CTA walks plus what it pays once.  A lone CTA walks its pair of tile groups one after the other
        // and pays 3 (set-up, two pipeline fills); the CTAs of a cluster are dealt out to the two groups as the kernel does it
        // (the pair with the most uneven groups decides: `est_blocks` against 2) and pay 10 (launch of a cluster, set-up,
        // fill, the exchange of rows with its two barriers).
        double best = 0;
        for (int c = 1; c <= WS_MAX_NC; ++c) {
            const long long active = ws_active_clusters<NT>(c);
            const long long waves = (units * grid_y + active - 1) / active;
            double blocks, fixed;
            if (c == 1) { blocks = est_blocks + 2; fixed = 3; }
            else {
                int nb = (c * 2 + (est_blocks + 2) / 2) / (est_blocks + 2);
                nb = nb < 1 ? 1 : (nb > c - 1 ? c - 1 : nb);
                const int na = c - nb;
                blocks = (est_blocks + na - 1) / na;
                if ((2 + nb - 1) / nb > blocks) blocks = (2 + nb - 1) / nb;
                fixed = 10;
            }
            const double cost = (double)waves * (fixed + blocks);
            if (nc <= 0 || cost < best) { best = cost; nc = c; }
        }
    }
    if (nc > WS_MAX_NC) nc = WS_MAX_NC;
    if (units * nc > 0x7fffffffLL) return VM_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(units * nc), (unsigned)grid_y); cfg.blockDim = dim3(ws_threads<NT>());
    cfg.dynamicSmemBytes = ws_smem_bytes<NT>(); cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nc; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attn_prefill_ws_kernel<NT>, mq, mk, mv, p);
    if (e != cudaSuccess) return (int)e;
    return vm_launch_status();
}

}  // namespace

// host_cu_tokens [B + 1] (host memory) are the same offsets as cu_tokens (device): the launch is shaped from them.
// Head size 64 only; out [T, H*64] and q rows must be 16-byte aligned (q_row_stride % 8 == 0).  groups: CTAs of a
// cluster that take a tile group's key blocks in turn (1 to 8), 0: chosen from the step's shape.
VM_API int vm_attention_prefill_ws_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                        const int* block_table, int max_blocks, const int* positions, const int* cu_tokens,
                                        const int* host_cu_tokens, int B, void* out, int H, int Hkv, int D, float scale, int window,
                                        int n_pages, int* err, int groups, cudaStream_t stream) {
    if (B <= 0 || host_cu_tokens == nullptr) return B <= 0 ? 0 : VM_ERR_BAD_ARG;
    if (D != WS_D || H <= 0 || Hkv <= 0 || H % Hkv != 0 || (q_row_stride % 8) != 0 || scale <= 0.f || n_pages <= 0 || max_blocks <= 0)
        return VM_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(kpages) |
         reinterpret_cast<uintptr_t>(vpages)) & 15) return VM_ERR_UNSUPPORTED;
    const long long rows = (long long)n_pages * Hkv * WS_BN;
    if (rows > 0x7fffffffLL) return VM_ERR_UNSUPPORTED;
    // tiles per CTA: the heads of a kv group at the same rows first, consecutive row tiles of a head when the group is small
    const int G = H / Hkv;
    const int NH = G % 3 == 0 ? 3 : (G % 2 == 0 ? 2 : 1);
    const int NT = NH == 1 ? 3 : NH;                        // (one head: three consecutive row tiles of it)
    const int NR = NT / NH;
    long long units = 0;
    for (int b = 0; b < B; ++b) {
        const int n = host_cu_tokens[b + 1] - host_cu_tokens[b];
        if (n < 0) return VM_ERR_BAD_ARG;
        const int n_rt = (n + WS_BM - 1) / WS_BM, n_rtg = (n_rt + NR - 1) / NR;
        units += (n_rtg + 1) / 2;
    }
    if (units <= 0) return 0;
    CUtensorMap mq, mk, mv;
    int rc = ws_query_map(&mq, q, host_cu_tokens[B], H, q_row_stride);
    if (rc) return rc;
    rc = ws_page_map(&mk, kpages, rows);
    if (rc) return rc;
    rc = ws_page_map(&mv, vpages, rows);
    if (rc) return rc;
    WsParams p{};
    p.q = (const __nv_bfloat16*)q; p.q_row_stride = q_row_stride; p.block_table = block_table; p.max_blocks = max_blocks;
    p.positions = positions; p.cu_tokens = cu_tokens; p.B = B; p.out = (__nv_bfloat16*)out; p.H = H; p.Hkv = Hkv; p.NH = NH;
    p.scale_log2 = scale * 1.4426950408889634f; p.rescale_gap = 8.0f / p.scale_log2;
    p.window = window; p.n_pages = n_pages; p.err = err;
    p.n_inline = 0;
    if (B <= WS_INLINE_SEQS) {
        p.n_inline = B;
        for (int b = 0; b <= B; ++b) p.inline_cu[b] = host_cu_tokens[b];
    }
    int est = max_blocks;                                   // key blocks a pair of tile groups walks, bounded by the table's width
    if (window > 0 && window / WS_BN + 2 < est) est = 2 * (window / WS_BN + 2);
    const int grid_y = Hkv * (G / NH);
    if (NT == 3) return ws_launch<3>(mq, mk, mv, p, units, grid_y, est, groups, stream);
    return ws_launch<2>(mq, mk, mv, p, units, grid_y, est, groups, stream);
}
