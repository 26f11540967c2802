// The weight-streaming products (skinny_gemm.cu) for LARGE weight matrices: the same work items, prologue and epilogues
// as skinny_run, organised around memory bandwidth instead of around the latency of one short chain.
//
// skinny_run fetches its weights straight into registers; each warp alternates between requesting a group of blocks and
// multiplying them, and the prologue is redone by every CTA while those registers are held.  That is right when a product
// reads one to three megabytes (a launch is then one chain of memory latencies), and slow when it reads tens of megabytes:
// two thousand dependent instructions per warp at a quarter of the memory bandwidth.  Here warps of their own stream the
// weight rows of the CTA's work items through a ring of shared-memory stages with bulk asynchronous copies (one copy per
// weight row and stage, 2 KB each, completion counted on an mbarrier), which keeps 60 to 190 KB per SM in flight whatever
// the eight multiplying warps are doing, starts before the wait on the predecessor kernel (weights are constants) and
// costs the multiplying warps two 16-byte shared-memory loads per two mma.sync.  The prologue reads every row's value of
// a column by the same thread, so one round of loads covers all rows.  Copying warps, multiplying warps, their work items,
// ring, sums and barriers are a pipeline; a CTA is one pipeline (two CTAs per SM) or two that share the staged rows.
//
// Work item, column permutation, accumulation order inside a warp, join of the eight warps and epilogues are those of
// skinny_run; so are the results, up to the order in which a warp's k blocks are summed.
#pragma once
#include "skinny_body.cuh"
#include "tc05.cuh"

namespace vmsk {

constexpr int SS_CW = SK_WARPS;                           // warps that multiply, per pipeline
constexpr int SS_KC = 1024;                              // values of K per stage
constexpr int SS_W_PITCH = SS_KC * 2 + 64;               // bytes between weight rows of a stage, == 64 (mod 128)
constexpr int SS_MAX_STAGES = 8;
constexpr int SS_TWIN_MIN_A_BYTES = 32 * 1024;            // from this size of the A tile on one CTA with two pipelines stages it once per SM

// byte offsets of the kernel's shared memory (`groups` pipelines share the A tile; each has its ring, sums and barriers)
struct StreamLayout { int ring, red, part, inv, bars, total, red_group; };
__host__ __device__ inline StreamLayout stream_layout(int M, int K, int rows, int stage_rows, int stages, int groups) {
    StreamLayout L;
    L.ring = (M * skinny_pitch(K) + 127) / 128 * 128;                        // after the A tile: M rows of K bf16
    L.red = L.ring + groups * stages * stage_rows * SS_W_PITCH;              // [group][buffer][warp][row][16] partial sums
    // (up to 16 rows: two buffers of the live rows, rounded up to 8, used by alternate work items; else one of all rows)
    L.red_group = (rows == 16 ? 2 * ((M + 7) / 8 * 8) : rows) * SS_CW * 16 * (int)sizeof(float);
    L.part = L.red + groups * L.red_group;                                   // [warp][row] partial sums of squares
    L.inv = L.part + groups * SS_CW * rows * (int)sizeof(float);             // [row] 1/rms
    L.bars = L.inv + rows * (int)sizeof(float);                              // per group full[8], empty[8]; then two flags
    L.total = L.bars + groups * 2 * SS_MAX_STAGES * 8 + 16;
    return L;
}

__device__ __forceinline__ uint64_t ss_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
// `bytes` (a multiple of 16) from global to this CTA's shared memory, both 16-byte aligned; completion is counted on `bar`
__device__ __forceinline__ void ss_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
template <int ID, int THREADS> __device__ __forceinline__ void ss_bar_sync() { asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(THREADS) : "memory"); }
// the barrier of pipeline `grp` (0 or 1) among its multiplying threads
template <int THREADS> __device__ __forceinline__ void ss_pipeline_sync(int grp) {
    if (grp == 0) ss_bar_sync<2, THREADS>(); else ss_bar_sync<3, THREADS>();
}

// NGRP pipelines per CTA (1: two CTAs share an SM; 2: one CTA has the SM and stages the A tile once for both), each of
// eight multiplying warps and PW copying warps with its own work items, ring, sums and barriers.
template <int MT, int NGRP, int PW>
__global__ void __launch_bounds__(NGRP * (SS_CW + PW) * 32, (MT == 1 && NGRP == 1) ? 2 : 1)
skinny_stream_kernel(const SkinnyParams p) {
    constexpr int SS_CONSUMERS = SS_CW, SS_CONSUMER_THREADS = SS_CW * 32, ALL_CONSUMER_THREADS = NGRP * SS_CONSUMER_THREADS;
    extern __shared__ __align__(128) unsigned char ss_smem[];
    unsigned char* const smem = ss_smem;
    constexpr int ROWS = 16 * MT;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int warp_all = tid >> 5;
    const bool copies = warp_all >= NGRP * SS_CW;
    // this warp's pipeline, and its index among the pipeline's warps of its kind
    const int grp = NGRP == 1 ? 0 : (copies ? (warp_all - NGRP * SS_CW) / PW : warp_all / SS_CW);
    const int warp = NGRP == 1 ? (copies ? warp_all - SS_CW : warp_all) : (copies ? (warp_all - NGRP * SS_CW) % PW : warp_all % SS_CW);
    const bool two = (p.tiles == 2);
    const int stage_rows = two ? 16 : 8;
    const int stage_bytes = stage_rows * SS_W_PITCH;
    const int S = p.stages;
    const StreamLayout L = stream_layout(p.M, p.K, ROWS, stage_rows, S, NGRP);
    unsigned char* sA = smem;
    float* red = reinterpret_cast<float*>(smem + L.red + grp * L.red_group);
    float* part = reinterpret_cast<float*>(smem + L.part);
    float* inv = reinterpret_cast<float*>(smem + L.inv);
    const uint32_t bars = ta_u32(smem + L.bars) + (uint32_t)(grp * 2 * SS_MAX_STAGES * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.bars + NGRP * 2 * SS_MAX_STAGES * 8);
    volatile int* never_set = abort_flag + 1;
#define SS_FULL(s) (bars + 8u * (uint32_t)(s))
#define SS_EMPTY(s) (bars + 8u * (uint32_t)(SS_MAX_STAGES + (s)))
    if (tid == 0) {
        const uint32_t all = ta_u32(smem + L.bars);
        for (int gi = 0; gi < NGRP; ++gi)
            for (int s = 0; s < S; ++s) {
                ta_bar_init(all + 8u * (uint32_t)(gi * 2 * SS_MAX_STAGES + s), PW);
                ta_bar_init(all + 8u * (uint32_t)(gi * 2 * SS_MAX_STAGES + SS_MAX_STAGES + s), SS_CONSUMERS);
            }
        *abort_flag = 0; *never_set = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // (the kernel that writes the cache lets its successor, the attention, start only after its own wait: see common.cuh)
    if (p.epi != EPI_ROPE_KV) vm_pdl_launch_dependents();
    // a pipeline takes the work items first, first + stride, ...
    const int first = (int)blockIdx.x * NGRP + grp, stride = (int)gridDim.x * NGRP;
    const int my_items = first < p.n_items ? (p.n_items - 1 - first) / stride + 1 : 0;
    const int chunks = (p.K + SS_KC - 1) / SS_KC;
    int n_issued = 0;

    if (copies) {
        // ---- the copying warps: each fetches its share of a stage's weight rows, a lane a row.  Weights are constants of the
        //      model, so these warps do not wait for the predecessor kernel: the ring is full when the multiplying warps get
        //      there.
        const uint64_t policy = ss_policy_evict_first();           // every weight byte is used once per step
        const uint32_t ring = ta_u32(smem + L.ring) + (uint32_t)(grp * S * stage_bytes);
        const int rows_pw = stage_rows / PW;
        const int my_row = warp * rows_pw + lane;                  // (lanes past rows_pw copy nothing)
        int n = 0;
        bool ok = true;
        for (int it = 0; it < my_items && ok; ++it) {
            const SkinnyCols c = skinny_cols(p, first + it * stride);
            const __nv_bfloat16* src = p.W + (size_t)(my_row < 8 ? c.nA + my_row : c.nB + my_row - 8) * p.K;
            for (int ch = 0; ch < chunks; ++ch) {
                const int s = n % S;
                if (n >= S) ok = ta_wait(SS_EMPTY(s), (uint32_t)((n / S) - 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const int kc0 = ch * SS_KC, kc = min(SS_KC, p.K - kc0);
                if (lane == 0) ta_bar_expect_tx(SS_FULL(s), (uint32_t)(rows_pw * kc * 2));
                if (lane < rows_pw)
                    ss_bulk_load(ring + (uint32_t)(s * stage_bytes + my_row * SS_W_PITCH), src + kc0, (uint32_t)(kc * 2), SS_FULL(s), policy);
                ++n;
            }
        }
        n_issued = n;
    } else {
        // ---- the multiplying warps
        vm_pdl_wait();                                          // from here on: data written by earlier kernels
        if (p.epi == EPI_ROPE_KV) vm_pdl_launch_dependents();
        const int a_pitch = p.row_bytes;
        // this thread's place in the epilogue: one (row, column-in-tile) of the work item
        // (an epilogue has ROWS x 8 such places; with more threads than that, groups of threads take the work items' epilogues
        // in turn, so that the others are already multiplying the next item, and the partial sums have two buffers)
        constexpr int EG = ROWS * 8, NG = SS_CONSUMER_THREADS / EG;
        const int ptid = tid - grp * SS_CONSUMER_THREADS;         // index among the pipeline's multiplying threads
        const int e_row = (ptid % EG) >> 3, e_c = ptid & 7, e_grp = ptid / EG;
        const int red_rows = NG > 1 ? (p.M + 7) / 8 * 8 : ROWS;
        int row_pos = 0, row_page = -1;
        if (p.epi == EPI_ROPE_KV && e_row < p.M) {
            row_pos = p.positions[e_row];
            if (p.kpages != nullptr) {
                const int blk = row_pos / VM_PAGE_TOKENS;
                row_page = (blk < p.max_blocks) ? p.block_table[(size_t)p.seq_of_token[e_row] * p.max_blocks + blk] : -1;
            }
        }
        // ---- stage A once for all work items of the CTA (all its multiplying threads, of every pipeline)
        if (p.pro == PRO_NONE) {
            const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.A);
            const int per_row = p.K / 8;
            for (int r = 0; r < p.M; ++r)
                for (int ch = tid; ch < per_row; ch += ALL_CONSUMER_THREADS)
                    vm_cp_async16(sA + (size_t)r * a_pitch + ch * 16, A + (size_t)r * p.K + ch * 8);
            vm_cp_async_commit();
            vm_cp_async_wait_all();
        } else {
            // x * w as bf16; the row's 1/rms multiplies the float32 sums in the epilogue (a row scale commutes with the
            // product).  A thread owns columns: it reads the norm weight once and the values of all rows in one round.
            const float* h = static_cast<const float*>(p.A);
            const int quads = p.K / 4;
            float ss[ROWS];
#pragma unroll
            for (int r = 0; r < ROWS; ++r) ss[r] = 0.f;
#pragma unroll 2
            for (int q = tid; q < quads; q += ALL_CONSUMER_THREADS) {
                const float4 w = reinterpret_cast<const float4*>(p.norm_w)[q];
#pragma unroll
                for (int r0 = 0; r0 < ROWS; r0 += 8) {
                    if (r0 >= p.M) break;
                    float4 x[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (r0 + u < p.M) x[u] = __ldcg(reinterpret_cast<const float4*>(h + (size_t)(r0 + u) * p.K) + q);   // from L2: another SM wrote it
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (r0 + u < p.M) {
                            ss[r0 + u] += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
                            uint2 v;
                            v.x = vm_pack_bf16(x[u].x * w.x, x[u].y * w.y);
                            v.y = vm_pack_bf16(x[u].z * w.z, x[u].w * w.w);
                            *reinterpret_cast<uint2*>(sA + (size_t)(r0 + u) * a_pitch + q * 8) = v;
                        }
                }
            }
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (r < p.M) {
                    const float v = vm_warp_sum(ss[r]);
                    if (lane == 0) part[warp_all * ROWS + r] = v;
                }
        }
        ss_bar_sync<1, ALL_CONSUMER_THREADS>();                   // A is there
        if (p.pro == PRO_RMSNORM) {
            if (tid < p.M) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < NGRP * SS_CONSUMERS; ++w) sum += part[w * ROWS + tid];
                inv[tid] = 1.0f / sqrtf(sum / (float)p.K + p.eps);
            }
            // (one pipeline: read by the epilogue after the join's barrier, which all its threads pass; two: the second
            // pipeline's join does not wait for thread tid of the first, so all meet once more)
            if (NGRP > 1) ss_bar_sync<1, ALL_CONSUMER_THREADS>();
        }

        int n = 0;
        bool ok = true;
        for (int it = 0; it < my_items; ++it) {
            const SkinnyCols cols = skinny_cols(p, first + it * stride);
            const int nA = cols.nA, nB = cols.nB, head = cols.head;
            const bool rotate = p.epi == EPI_ROPE_KV && head < p.H + p.Hkv && p.rot_dim > 0;
            const bool e_live = e_row < p.M && e_grp == it % NG;
            float* const red_it = red + (NG > 1 ? (size_t)(it & 1) * SS_CONSUMERS * red_rows * 16 : 0);
            // what the epilogue adds to or multiplies with is requested now: its latency passes under the product
            float freq = 0.f, res_a = 0.f, res_b = 0.f;
            if (rotate) freq = p.inv_freq[(nA - head * p.D) + e_c];
            if (p.epi == EPI_RESIDUAL && e_live) {
                const float* o = p.h + (size_t)e_row * p.N;
                res_a = __ldcg(o + nA + e_c);
                if (two) res_b = __ldcg(o + nB + e_c);
            }
            float acc[MT][2][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int t = 0; t < 2; ++t) acc[mt][t][0] = acc[mt][t][1] = acc[mt][t][2] = acc[mt][t][3] = 0.f;

            for (int ch = 0; ch < chunks; ++ch, ++n) {
                const int s = n % S;
                if (ok) ok = ta_wait(SS_FULL(s), (uint32_t)(n / S) & 1u, abort_flag);
                const int kc0 = ch * SS_KC, blocks = min(SS_KC, p.K - kc0) >> 5;
                const unsigned char* wbase = smem + L.ring + (grp * S + s) * stage_bytes + g * SS_W_PITCH + t4 * 16;
                const unsigned char* abase = sA + kc0 * 2 + t4 * 16;
#pragma unroll 2
                for (int b = warp; b < blocks; b += SS_CONSUMERS) {
                    const uint4 wa = *reinterpret_cast<const uint4*>(wbase + b * 64);
                    uint4 wb = make_uint4(0u, 0u, 0u, 0u);
                    if (two) wb = *reinterpret_cast<const uint4*>(wbase + 8 * SS_W_PITCH + b * 64);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint4 a_lo = make_uint4(0u, 0u, 0u, 0u), a_hi = a_lo;          // rows past M: zeros, never read
                        if (mt * 16 + g < p.M) a_lo = *reinterpret_cast<const uint4*>(abase + (size_t)(mt * 16 + g) * a_pitch + b * 64);
                        if (mt * 16 + g + 8 < p.M) a_hi = *reinterpret_cast<const uint4*>(abase + (size_t)(mt * 16 + g + 8) * a_pitch + b * 64);
                        vm_mma_bf16_16816(acc[mt][0], a_lo.x, a_hi.x, a_lo.y, a_hi.y, wa.x, wa.y);
                        vm_mma_bf16_16816(acc[mt][0], a_lo.z, a_hi.z, a_lo.w, a_hi.w, wa.z, wa.w);
                        if (two) {
                            vm_mma_bf16_16816(acc[mt][1], a_lo.x, a_hi.x, a_lo.y, a_hi.y, wb.x, wb.y);
                            vm_mma_bf16_16816(acc[mt][1], a_lo.z, a_hi.z, a_lo.w, a_hi.w, wb.z, wb.w);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) ta_bar_arrive(SS_EMPTY(s));       // this warp has read the stage
            }
            // ---- join the warps' partial sums: red[warp][row][col], col 0..7 = tile A, 8..15 = tile B
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int row = mt * 16 + g + 8 * half;
                        if (row < p.M && (t == 0 || two))
                            *reinterpret_cast<float2*>(&red_it[((size_t)warp * red_rows + row) * 16 + t * 8 + 2 * t4]) =
                                make_float2(acc[mt][t][2 * half], acc[mt][t][2 * half + 1]);
                    }
            ss_pipeline_sync<SS_CONSUMER_THREADS>(grp);          // this pipeline's sums are there
            if (e_live && !*abort_flag) {
                const int row = e_row, c = e_c;
                float vA = 0.f, vB = 0.f;
#pragma unroll
                for (int w = 0; w < SS_CONSUMERS; ++w) {
                    vA += red_it[((size_t)w * red_rows + row) * 16 + c];
                    if (two) vB += red_it[((size_t)w * red_rows + row) * 16 + 8 + c];
                }
                if (p.pro == PRO_RMSNORM) { const float rs = inv[row]; vA *= rs; vB *= rs; }
                switch (p.epi) {
                    case EPI_STORE_BF16: {
                        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride;
                        o[nA + c] = __float2bfloat16_rn(vA);
                        if (two) o[nB + c] = __float2bfloat16_rn(vB);
                    } break;
                    case EPI_STORE_F32: {
                        float* o = static_cast<float*>(p.out) + (size_t)row * p.out_stride;
                        o[nA + c] = vA;
                        if (two) o[nB + c] = vB;
                    } break;
                    case EPI_RESIDUAL: {
                        float* o = p.h + (size_t)row * p.N;
                        o[nA + c] = res_a + vA;
                        if (two) o[nB + c] = res_b + vB;
                    } break;
                    case EPI_SWIGLU: {
                        const float sig = 1.0f / (1.0f + expf(-vA));
                        static_cast<__nv_bfloat16*>(p.out)[(size_t)row * p.out_stride + nA + c] = __float2bfloat16_rn((sig * vA) * vB);
                    } break;
                    case EPI_ROPE_KV: {
                        float ya = vA, yb = vB;
                        int da, db;                                 // the two columns' places inside the head
                        if (rotate) {
                            da = (nA - head * p.D) + c; db = da + p.D / 2;
                            float sn, co;
                            sincosf((float)row_pos * freq, &sn, &co);
                            ya = vA * co - vB * sn;
                            yb = vB * co + vA * sn;
                        } else { da = (nA - head * p.D) + c; db = da + 8; }
                        if (head < p.H) {
                            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride + (size_t)head * p.D;
                            o[da] = __float2bfloat16_rn(ya); o[db] = __float2bfloat16_rn(yb);
                        } else if (p.kpages != nullptr) {
                            if (row_page < 0 || row_page >= p.n_pages) { if (p.err) atomicExch(p.err, VM_ERRWORD_CACHE_WRITE); break; }
                            const bool is_k = head < p.H + p.Hkv;
                            const int hk = is_k ? head - p.H : head - p.H - p.Hkv;
                            __nv_bfloat16* dst = (is_k ? p.kpages : p.vpages) + (size_t)row_page * ((size_t)p.Hkv * VM_PAGE_TOKENS * p.D)
                                                 + ((size_t)hk * VM_PAGE_TOKENS + row_pos % VM_PAGE_TOKENS) * p.D;
                            dst[da] = __float2bfloat16_rn(ya); dst[db] = __float2bfloat16_rn(yb);
                        }
                    } break;
                }
            }
            if (NG == 1) ss_pipeline_sync<SS_CONSUMER_THREADS>(grp);                 // the sums' one buffer is reused by the next item
        }
    }
    // ---- a wait that ran out: nothing more was stored; copies still in flight into this CTA's shared memory are waited
    //      for (again with a limit) before the CTA ends, and the step's error word says what happened
    __syncthreads();
    if (*abort_flag && copies) {
        if (lane == 0) {
            for (int k = max(0, n_issued - S); k < n_issued; ++k) ta_wait(SS_FULL(k % S), (uint32_t)(k / S) & 1u, never_set);
            if (p.err) atomicExch(p.err, VM_ERRWORD_BARRIER_WAIT);
        }
    }
#undef SS_FULL
#undef SS_EMPTY
}

// Launch for `items` work items (p.tiles, p.epi and the epilogue's fields set by the caller).  VM_ERR_UNSUPPORTED when the
// A tile and two stages per pipeline do not fit into shared memory or M is over 32: the caller then takes skinny_launch.
// form 0: the launcher's choice; 1: two CTAs of one pipeline per SM; 2: one CTA of two pipelines per SM.  Measured at hidden
// 2,048 (gate/up, 4 / 8 rows: 14.6 / 15.7 us as two CTAs, 13.9 / 14.7 us as one; down at K = 8,192, 8 rows: 15.2 / 11.7 us) and
// at hidden 960 (gate/up, 1 / 4 / 8 / 16 rows: 5.2 / 5.5 / 6.4 / 8.6 against 5.6 / 6.2 / 6.6 / 8.2 us): one CTA pays when the
// rows it stages once instead of twice are many.  Inside a decode step it also starts later than a CTA of half its size (it
// needs a whole SM to be free): the 1.7B shape at batch 1 lost 5 % with the down projection in this form (951 -> 900 tokens/s,
// although the kernel alone is as fast), and gains 7 % at batch 8 with three of its four products in it.
inline int skinny_stream_launch(SkinnyParams p, int items, cudaStream_t stream, int form = 0) {
    if (p.M <= 0 || items <= 0) return 0;
    if (p.M > 32 || p.K % 32 != 0 || p.K <= 0) return VM_ERR_UNSUPPORTED;
    const int MT = p.M <= 16 ? 1 : 2;
    const int rows = 16 * MT, stage_rows = p.tiles == 2 ? 16 : 8, stage_bytes = stage_rows * SS_W_PITCH;
    constexpr int SM_BYTES = 227 * 1024, CTA_RESERVED = 1024;
    // stages per pipeline in each form
    const int s_pair = (SM_BYTES / 2 - CTA_RESERVED - stream_layout(p.M, p.K, rows, stage_rows, 0, 1).total) / stage_bytes;       // two CTAs per SM
    const int s_twin = MT == 1 ? (SM_BYTES - CTA_RESERVED - stream_layout(p.M, p.K, rows, stage_rows, 0, 2).total) / stage_bytes / 2 : 0;   // one CTA, two pipelines
    const int s_lone = (SM_BYTES - CTA_RESERVED - stream_layout(p.M, p.K, rows, stage_rows, 0, 1).total) / stage_bytes;           // one CTA, one pipeline
    int groups = 1, per_sm = 1, S = s_lone;
    const bool twin_preferred = p.M * skinny_pitch(p.K) >= SS_TWIN_MIN_A_BYTES;
    if (MT == 1 && form != 1 && s_twin >= 2 && (form == 2 || twin_preferred || s_pair < 2)) { groups = 2; S = s_twin; }
    else if (MT == 1 && form != 2 && s_pair >= 2) { per_sm = 2; S = s_pair; }
    if (S > SS_MAX_STAGES) S = SS_MAX_STAGES;
    if (S < 2) return VM_ERR_UNSUPPORTED;
    const int sms = vm_sm_count() > 0 ? vm_sm_count() : 1;
    const int want = (items + groups - 1) / groups;
    const int grid = want < sms * per_sm ? want : sms * per_sm;
    p.n_items = items; p.stages = S; p.row_bytes = skinny_pitch(p.K);
    const size_t smem = (size_t)stream_layout(p.M, p.K, rows, stage_rows, S, groups).total;
#define VM_SS_CASE(X, G, P)                                                                                           \
    {                                                                                                                 \
        static bool configured = false;                                                                               \
        if (!configured) {                                                                                            \
            cudaError_t e = cudaFuncSetAttribute(skinny_stream_kernel<X, G, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_BYTES - CTA_RESERVED); \
            if (e != cudaSuccess) return (int)e;                                                                      \
            configured = true;                                                                                        \
        }                                                                                                             \
        vm_launch_pdl(skinny_stream_kernel<X, G, P>, dim3(grid), dim3(G * (SS_CW + P) * 32), smem, stream, p);        \
    }
    if (MT == 2) VM_SS_CASE(2, 1, 4) else if (groups == 2) VM_SS_CASE(1, 2, 2) else VM_SS_CASE(1, 1, 2)
#undef VM_SS_CASE
    return vm_launch_status();
}

}  // namespace vmsk
