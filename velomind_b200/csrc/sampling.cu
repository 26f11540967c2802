// Sampling on the device: greedy, temperature and nucleus (top-p), one block per row of logits.
//
// Rules of the reference's sampler (examples/common/llama/llama_engine.cpp:668-726):
//   * temperature <= 0 or top_p <= 0: greedy; NaN is skipped, the first maximum wins, all-NaN gives -1;
//   * otherwise p_i = exp((x_i - max) / T) in float, normalised by a sum kept in double; the nucleus is
//     the smallest set of most probable tokens whose mass reaches top_p; draw r uniform in [0, mass) and
//     walk the nucleus until the running sum reaches r.
// Differences, on purpose: the uniform number comes from Philox-4x32-10 keyed by (seed; stream, step)
// instead of one std::mt19937 shared by all draws, so a request's tokens do not depend on what else is
// in the batch; the walk goes in index order, not in sorted order, and every token that ties with the
// least probable nucleus member belongs to the nucleus (same distribution; no sort of the vocabulary).
#include "common.cuh"

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ double block_sum_d(double v, double* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum_d(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double t = (lane < (int)((blockDim.x + 31) >> 5)) ? red[lane] : 0.0;
    return warp_sum_d(t);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
        const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
        c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
        k0 += W0; k1 += W1;
    }
}

struct ArgBest { float v; int i; };

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {   // larger value; on a tie the lower index
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// CACHED: the row's unnormalised probabilities are computed once and kept in dynamic shared memory (V floats; NaN
// logits are marked by -1), so the passes of the nucleus search read shared memory; otherwise every pass recomputes them
// from the logits in global memory (vocabularies too large for shared memory).
template <bool CACHED>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const long long* __restrict__ seed, const long long* __restrict__ stream_id,
              const long long* __restrict__ step, long long step_add, int* __restrict__ out) {
    extern __shared__ __align__(16) float sraw[];
    __shared__ double redd[32];
    __shared__ float redv[32];
    __shared__ int redi[32];
    __shared__ double sums[SAMPLE_THREADS];
    __shared__ int s_choice;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * row_stride;
    const float temp = temperature ? temperature[row] : 0.f;
    const float tp = top_p ? top_p[row] : 1.f;

    // ---- maximum (NaN skipped) with its first index; four values per load where the row is 16-byte aligned
    ArgBest best{-INFINITY, -1};
    int scalar_from = 0;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const int V4 = V >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        constexpr int U = 4;
        for (int i0 = tid; i0 < V4; i0 += SAMPLE_THREADS * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * SAMPLE_THREADS;
                v[u] = (i < V4) ? x4[i] : make_float4(NAN, NAN, NAN, NAN);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = 4 * (i0 + u * SAMPLE_THREADS);
                if (v[u].x == v[u].x) best = better(best, ArgBest{v[u].x, i});
                if (v[u].y == v[u].y) best = better(best, ArgBest{v[u].y, i + 1});
                if (v[u].z == v[u].z) best = better(best, ArgBest{v[u].z, i + 2});
                if (v[u].w == v[u].w) best = better(best, ArgBest{v[u].w, i + 3});
            }
        }
        scalar_from = V4 << 2;
    }
    for (int i = scalar_from + tid; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v != v) continue;
        best = better(best, ArgBest{v, i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) { redv[warp] = best.v; redi[warp] = best.i; }
    __syncthreads();
    best = ArgBest{-INFINITY, -1};
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) best = better(best, ArgBest{redv[k], redi[k]});
    if (!(temp > 0.f) || !(tp > 0.f) || best.i < 0) {
        if (tid == 0) out[row] = best.i;
        return;
    }
    // the reference takes the max over FINITE values only (an all -inf/+inf row gives -1)
    float max_v = best.v;
    if (isinf(max_v)) {
        float fm = -INFINITY; int any = 0;
        for (int i = tid; i < V; i += blockDim.x) { const float v = x[i]; if (isfinite(v)) { fm = fmaxf(fm, v); any = 1; } }
        fm = vm_warp_max(fm); any = __any_sync(0xffffffffu, any);
        __syncthreads();
        if (lane == 0) { redv[warp] = fm; redi[warp] = any; }
        __syncthreads();
        fm = -INFINITY; any = 0;
        for (int k = 0; k < (int)(blockDim.x >> 5); ++k) { fm = fmaxf(fm, redv[k]); any |= redi[k]; }
        if (!any) { if (tid == 0) out[row] = -1; return; }
        max_v = fm;
    }
    const float inv_t = 1.0f / temp;
    // unnormalised probability of token i, or a negative number for a NaN logit
    auto raw_of = [&](int i) -> float {
        const float v = x[i];
        return (v != v) ? -1.f : expf((v - max_v) * inv_t);
    };
    auto raw = [&](int i) -> float { return CACHED ? sraw[i] : raw_of(i); };
    double part = 0.0;
    for (int i = tid; i < V; i += blockDim.x) {
        const float r = raw_of(i);
        if (CACHED) sraw[i] = r;
        part += (double)(r < 0.f ? 0.f : r);
    }
    const double total = block_sum_d(part, redd);          // (its barriers also publish the cached values)
    const float inv_sum = (float)(1.0 / total);
    // normalised probability; negative for a NaN logit (never in the nucleus)
    auto prob = [&](int i) -> float { const float r = raw(i); return r < 0.f ? -1.f : r * inv_sum; };

    // ---- nucleus threshold: the largest tau with sum{p_i >= tau} >= top_p (bisection on the float bits)
    // Search: four-way instead of two-way, three thresholds per pass over the probabilities (16 passes, not 31; measured
    // at 49,152 tokens: 7 and 15 thresholds per pass are no faster), and only what lies between the thresholds is summed again.
    float tau = 0.f;
    if (tp < 1.0f) {
        float pmax = 0.f;
        for (int i = tid; i < V; i += blockDim.x) pmax = fmaxf(pmax, prob(i));
        pmax = vm_warp_max(pmax);
        __syncthreads();
        if (lane == 0) redv[warp] = pmax;
        __syncthreads();
        pmax = 0.f;
        for (int k = 0; k < (int)(blockDim.x >> 5); ++k) pmax = fmaxf(pmax, redv[k]);
        uint32_t lo = 0u, hi = __float_as_uint(pmax) + 1u;   // cond(lo) holds or tau stays 0; cond(hi) fails
        constexpr int WAYS = 3;
        double* many = sums;                                  // [warps][WAYS] partial sums (sums[] is free until the walk)
        double above = 0.0;                                   // the mass of p >= hi: known from the pass that lowered hi
        while (hi - lo > 1u) {
            const uint32_t stepw = (hi - lo + WAYS) / (WAYS + 1);      // thresholds lo + j * stepw, j = 1..WAYS, below hi
            float th[WAYS];
            double sj[WAYS];
#pragma unroll
            for (int j = 0; j < WAYS; ++j) {
                const unsigned long long t = (unsigned long long)lo + (unsigned long long)(j + 1) * stepw;
                th[j] = (t < (unsigned long long)hi) ? __uint_as_float((uint32_t)t) : INFINITY;
                sj[j] = 0.0;
            }
            const float f_lo = __uint_as_float(lo + stepw), f_hi = __uint_as_float(hi);
            for (int i = tid; i < V; i += blockDim.x) {
                const float p = prob(i);
                if (p >= f_lo && p < f_hi) {                 // only what lies between the thresholds is summed again
                    const double pd = (double)p;
#pragma unroll
                    for (int j = 0; j < WAYS; ++j) if (p >= th[j]) sj[j] += pd;
                }
            }
#pragma unroll
            for (int j = 0; j < WAYS; ++j) sj[j] = warp_sum_d(sj[j]);
            __syncthreads();
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < WAYS; ++j) many[warp * WAYS + j] = sj[j];
            }
            __syncthreads();
            if (warp == 0 && lane < WAYS) {                   // one thread per threshold joins the warps, in warp order
                double sum = 0.0;
                for (int k = 0; k < (int)(blockDim.x >> 5); ++k) sum += many[k * WAYS + lane];
                redd[lane] = sum;
            }
            __syncthreads();
            uint32_t new_lo = lo, new_hi = hi;
            double new_above = above;
#pragma unroll
            for (int j = 0; j < WAYS; ++j) {
                const unsigned long long t = (unsigned long long)lo + (unsigned long long)(j + 1) * stepw;
                if (t < (unsigned long long)new_hi) {
                    const double sum = above + redd[j];       // mass of p >= t: what lies above hi, plus [t, hi)
                    if (sum >= (double)tp) new_lo = (uint32_t)t; else { new_hi = (uint32_t)t; new_above = sum; }
                }
            }
            lo = new_lo; hi = new_hi; above = new_above;
        }
        tau = __uint_as_float(lo);
        __syncthreads();
    }

    // ---- mass of the nucleus and the walk in index order
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int i0 = min(V, tid * chunk), i1 = min(V, i0 + chunk);
    double mine = 0.0;
    for (int i = i0; i < i1; ++i) { const float p = prob(i); if (p >= 0.f && p >= tau) mine += (double)p; }
    // exclusive running sums over the threads' chunks: a scan inside each warp, then over the warps' totals
    double incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    __syncthreads();
    if (lane == 31) redd[warp] = incl;
    if (tid == 0) s_choice = 0x7fffffff;
    __syncthreads();
    double offset = 0.0, mass = 0.0;
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) { const double t = redd[k]; if (k < warp) offset += t; mass += t; }
    sums[tid] = offset + incl - mine;
    __syncthreads();
    uint32_t c[4];
    const unsigned long long st = (unsigned long long)((step ? step[row] : 0) + step_add), sid = (unsigned long long)(stream_id ? stream_id[row] : 0);
    const unsigned long long sd = (unsigned long long)(seed ? seed[row] : 0);
    c[0] = (uint32_t)st; c[1] = (uint32_t)(st >> 32); c[2] = (uint32_t)sid; c[3] = (uint32_t)(sid >> 32);
    philox4x32_10(c, (uint32_t)sd, (uint32_t)(sd >> 32));
    const float u = (float)(c[0] >> 8) * (1.0f / 16777216.0f);
    const double r = (double)u * mass;
    // the chunk in which the running sum first reaches r walks its members
    const double before = sums[tid];
    if (before <= r) {
        double acc = before;
        for (int i = i0; i < i1; ++i) {
            const float p = prob(i);
            if (p >= 0.f && p >= tau) {
                acc += (double)p;
                if (acc >= r) { atomicMin(&s_choice, i); break; }
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int choice = s_choice;
        if (choice == 0x7fffffff) {       // rounding left the running sum short of r: the last member
            choice = -1;
            for (int i = V - 1; i >= 0; --i) { const float p = prob(i); if (p >= 0.f && p >= tau) { choice = i; break; } }
        }
        out[row] = choice;
    }
}

// ---------------------------------------------------------------- the same sampler, a cluster of eight CTAs per row
// A decode batch has few rows and one CTA per row leaves the GPU idle while it walks a vocabulary of tens of thousands
// several times.  Here eight CTAs (a thread-block cluster) share a row: each keeps an eighth of the row's probabilities
// in shared memory, every pass sums its own eighth, and the eight partial results meet through distributed shared
// memory (every CTA writes its number into every CTA's table, one hardware cluster barrier, every CTA adds the eight
// numbers in rank order: the same sum everywhere, so all eight take the same decisions).  Same rules, same results.
// What a step costs here is its cluster barrier (2 to 3 us), so there are as few as possible: the largest probability is
// known without asking (the maximum's own), the nucleus search counts as it sums and, as soon as at most SC_CAND_MAX
// probabilities are left between its bounds, every CTA receives all of them and finishes the search by itself, and the CTA
// in whose range the drawn number falls writes the token without a last exchange.
constexpr int SC_CTAS = 8, SC_THREADS = 256, SC_WARPS = SC_THREADS / 32, SC_WAYS = 7;
constexpr int SC_VALS = 16;                       // numbers per exchange: SC_WAYS sums and SC_WAYS + 1 counts
constexpr int SC_CAND_MAX = 2048;                 // the search goes on inside every CTA once this few probabilities are left

__device__ __forceinline__ void sc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void sc_put(double* slot_local, unsigned to_rank, double v) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(slot_local)), "r"(to_rank));
    asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(remote), "d"(v) : "memory");
}

struct ScShared {
    double gather[2][SC_CTAS][SC_VALS];       // [exchange parity][source CTA][value]
    double warp_d[SC_WARPS][SC_VALS];
    float warp_v[SC_WARPS];
    int warp_i[SC_WARPS];
    double prefix[SC_THREADS];
    int choice;
    int scan[SC_WARPS];
    float cand[SC_CAND_MAX];                  // the probabilities still in question, the same list in every CTA
};

// Every CTA contributes up to SC_VALS numbers; the caller reads sh.gather[parity][source][k] after the call.
__device__ __forceinline__ void sc_all_gather(ScShared& sh, int parity, unsigned rank, const double (&mine)[SC_VALS], int n) {
    if (threadIdx.x < SC_CTAS * SC_VALS) {
        const unsigned to = threadIdx.x / SC_VALS;
        const int k = threadIdx.x % SC_VALS;
        double v = 0.0;
#pragma unroll
        for (int j = 0; j < SC_VALS; ++j) if (j == k) v = mine[j];      // (no dynamic indexing of registers)
        if (k < n) sc_put(&sh.gather[parity][rank][k], to, v);
    }
    sc_cluster_sync();
}

// Sum of n (<= SC_VALS) per-thread doubles over the CTA; every thread gets the sums (warps joined in warp order).
__device__ __forceinline__ void sc_block_sum(ScShared& sh, double (&v)[SC_VALS], int n) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < SC_VALS; ++k) if (k < n) v[k] = warp_sum_d(v[k]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < SC_VALS; ++k) if (k < n) sh.warp_d[warp][k] = v[k];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SC_VALS; ++k) {
        if (k < n) {
            double t = 0.0;
#pragma unroll
            for (int w = 0; w < SC_WARPS; ++w) t += sh.warp_d[w][k];
            v[k] = t;
        }
    }
}

__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, long long row_stride, int V, int slice,
                      const float* __restrict__ temperature, const float* __restrict__ top_p,
                      const long long* __restrict__ seed, const long long* __restrict__ stream_id,
                      const long long* __restrict__ step, long long step_add, int* __restrict__ out) {
    extern __shared__ __align__(16) float sraw[];                   // this CTA's slice of unnormalised probabilities
    __shared__ ScShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned rank;
    asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int row = blockIdx.x / SC_CTAS;
    const float* x = logits + (size_t)row * row_stride;
    const int i0 = min(V, (int)rank * slice), i1 = min(V, i0 + slice), n = i1 - i0;       // this CTA's tokens [i0, i1)
    const float temp = temperature ? temperature[row] : 0.f;
    const float tp = top_p ? top_p[row] : 1.f;
    int parity = 0;
    double mine[SC_VALS];

    // ---- maximum (NaN skipped) with its first index
    ArgBest best{-INFINITY, -1};
    for (int i = i0 + tid; i < i1; i += SC_THREADS) {
        const float v = x[i];
        if (v == v) best = better(best, ArgBest{v, i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) { sh.warp_v[warp] = best.v; sh.warp_i[warp] = best.i; }
    __syncthreads();
    best = ArgBest{-INFINITY, -1};
    for (int k = 0; k < SC_WARPS; ++k) best = better(best, ArgBest{sh.warp_v[k], sh.warp_i[k]});
    mine[0] = (double)best.v; mine[1] = (double)best.i;
    sc_all_gather(sh, parity, rank, mine, 2);
    best = ArgBest{-INFINITY, -1};
    for (int c = 0; c < SC_CTAS; ++c) best = better(best, ArgBest{(float)sh.gather[parity][c][0], (int)sh.gather[parity][c][1]});
    parity ^= 1;
    if (!(temp > 0.f) || !(tp > 0.f) || best.i < 0) {
        if (rank == 0 && tid == 0) out[row] = best.i;
        return;                                    // (uniform over the cluster; nobody writes into a peer after the barrier above)
    }
    // the reference takes the max over FINITE values only (an all -inf/+inf row gives -1)
    float max_v = best.v;
    if (isinf(max_v)) {                            // (uniform over the cluster)
        float fm = -INFINITY; int any = 0;
        for (int i = i0 + tid; i < i1; i += SC_THREADS) { const float v = x[i]; if (isfinite(v)) { fm = fmaxf(fm, v); any = 1; } }
        fm = vm_warp_max(fm); any = __any_sync(0xffffffffu, any);
        __syncthreads();
        if (lane == 0) { sh.warp_v[warp] = fm; sh.warp_i[warp] = any; }
        __syncthreads();
        fm = -INFINITY; any = 0;
        for (int k = 0; k < SC_WARPS; ++k) { fm = fmaxf(fm, sh.warp_v[k]); any |= sh.warp_i[k]; }
        mine[0] = (double)fm; mine[1] = (double)any;
        sc_all_gather(sh, parity, rank, mine, 2);
        fm = -INFINITY; any = 0;
        for (int c = 0; c < SC_CTAS; ++c) { fm = fmaxf(fm, (float)sh.gather[parity][c][0]); any |= (int)sh.gather[parity][c][1]; }
        parity ^= 1;
        if (!any) { if (rank == 0 && tid == 0) out[row] = -1; return; }
        max_v = fm;
    }
    // ---- unnormalised probabilities of this slice (negative for a NaN logit) and their sum
    const float inv_t = 1.0f / temp;
    double part = 0.0;
    for (int j = tid; j < n; j += SC_THREADS) {
        const float v = x[i0 + j];
        const float r = (v != v) ? -1.f : expf((v - max_v) * inv_t);
        sraw[j] = r;
        part += (double)(r < 0.f ? 0.f : r);
    }
    mine[0] = part;
    sc_block_sum(sh, mine, 1);
    sc_all_gather(sh, parity, rank, mine, 1);
    double total = 0.0;
    for (int c = 0; c < SC_CTAS; ++c) total += sh.gather[parity][c][0];
    parity ^= 1;
    const float inv_sum = (float)(1.0 / total);
    auto prob = [&](int j) -> float { const float r = sraw[j]; return r < 0.f ? -1.f : r * inv_sum; };

    // ---- nucleus threshold: the largest tau with sum{p_i >= tau} >= top_p (eight-way search on the float bits)
    float tau = 0.f;
    const int chunk = (n + SC_THREADS - 1) / SC_THREADS;
    const int j0 = min(n, tid * chunk), j1 = min(n, j0 + chunk);            // this thread's tokens of the slice, in index order
    if (tp < 1.0f) {
        const float pmax = 1.0f * inv_sum;                    // the probability of the maximum itself (its exponential is 1)
        uint32_t lo = 0u, hi = __float_as_uint(pmax) + 1u;   // cond(lo) holds or tau stays 0; cond(hi) fails
        double above = 0.0;                                   // the mass of p >= hi: known from the pass that lowered hi
        long long left = (long long)V;                        // probabilities in [lo, hi), an upper bound before the first pass
        // One pass: the masses above SC_WAYS thresholds between lo and hi (only what lies between the bounds is summed again)
        // and, with `count`, how many probabilities lie above each and above lo.  `each` yields the probabilities to look at.
        // thresholds of a pass, ascending, as float bits (a threshold at or beyond hi stands for "none")
        auto uniform = [&](uint32_t (&tb)[SC_WAYS]) {
            const uint32_t stepw = (hi - lo + SC_WAYS) / (SC_WAYS + 1);
#pragma unroll
            for (int k = 0; k < SC_WAYS; ++k) {
                const unsigned long long t = (unsigned long long)lo + (unsigned long long)(k + 1) * stepw;
                tb[k] = (t < (unsigned long long)hi) ? (uint32_t)t : 0xffffffffu;
            }
        };
        auto decide = [&](const double (&S)[SC_VALS], const uint32_t (&tb)[SC_WAYS], bool count) {      // S: the cluster's (or the list's) sums
            uint32_t new_lo = lo, new_hi = hi;
            double new_above = above;
            double c_lo = S[SC_WAYS], c_hi = 0.0;             // counts above the new bounds
#pragma unroll
            for (int k = 0; k < SC_WAYS; ++k) {
                if (tb[k] < new_hi) {
                    const double sum = above + S[k];          // mass of p >= t: what lies above hi, plus [t, hi)
                    if (sum >= (double)tp) { new_lo = tb[k]; c_lo = S[SC_WAYS + 1 + k]; }
                    else { new_hi = tb[k]; new_above = sum; c_hi = S[SC_WAYS + 1 + k]; }
                }
            }
            lo = new_lo; hi = new_hi; above = new_above;
            if (count) left = (long long)(c_lo - c_hi);
        };
        while (hi - lo > 1u && left > SC_CAND_MAX) {          // (the same trip count in every CTA: the sums are the same)
            uint32_t tb[SC_WAYS];
            float th[SC_WAYS];
            double sj[SC_VALS];
#pragma unroll
            for (int k = 0; k < SC_VALS; ++k) sj[k] = 0.0;
            // while no threshold has held yet, a pass asks at every second power of two below the upper bound (a pass that cuts
            // the float bits evenly would spend itself on sixteen binades per step, and nearly everything lies in a few)
            const int e_top = (int)((hi - 1u) >> 23);
            if (lo == 0u && e_top > 2 * SC_WAYS) {
#pragma unroll
                for (int k = 0; k < SC_WAYS; ++k) tb[k] = (uint32_t)(e_top - 2 * (SC_WAYS - k)) << 23;
            } else {
                uniform(tb);
            }
#pragma unroll
            for (int k = 0; k < SC_WAYS; ++k) th[k] = (tb[k] < hi) ? __uint_as_float(tb[k]) : INFINITY;
            const float f_lo = __uint_as_float(lo), f_hi = __uint_as_float(hi);
            for (int j = tid; j < n; j += SC_THREADS) {
                const float p = prob(j);
                if (p >= f_lo && p < f_hi) {
                    const double pd = (double)p;
                    sj[SC_WAYS] += 1.0;
#pragma unroll
                    for (int k = 0; k < SC_WAYS; ++k) if (p >= th[k]) { sj[k] += pd; sj[SC_WAYS + 1 + k] += 1.0; }
                }
            }
            sc_block_sum(sh, sj, 2 * SC_WAYS + 1);
            sc_all_gather(sh, parity, rank, sj, 2 * SC_WAYS + 1);
            double S[SC_VALS];
#pragma unroll
            for (int k = 0; k < SC_VALS; ++k) {
                S[k] = 0.0;
                if (k < 2 * SC_WAYS + 1) for (int c = 0; c < SC_CTAS; ++c) S[k] += sh.gather[parity][c][k];
            }
            parity ^= 1;
            decide(S, tb, true);
        }
        if (hi - lo > 1u) {
            // ---- few are left: every CTA gets all of them (each CTA's in index order, the CTAs in rank order) ...
            const float f_lo = __uint_as_float(lo), f_hi = __uint_as_float(hi);
            int mine_n = 0;
            for (int j = j0; j < j1; ++j) { const float p = prob(j); mine_n += (p >= f_lo && p < f_hi) ? 1 : 0; }
            int incl_n = mine_n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int up = __shfl_up_sync(0xffffffffu, incl_n, o); if (lane >= o) incl_n += up; }
            __syncthreads();
            if (lane == 31) sh.scan[warp] = incl_n;
            __syncthreads();
            int warp_before = 0, cta_n = 0;
            for (int k = 0; k < SC_WARPS; ++k) { const int t = sh.scan[k]; if (k < warp) warp_before += t; cta_n += t; }
            mine[0] = (double)cta_n;
            sc_all_gather(sh, parity, rank, mine, 1);
            int cta_before_n = 0, total_n = 0;
            for (int c = 0; c < SC_CTAS; ++c) { const int t = (int)sh.gather[parity][c][0]; if (c < (int)rank) cta_before_n += t; total_n += t; }
            parity ^= 1;
            total_n = min(total_n, SC_CAND_MAX);              // (it is at most that: the counts said so)
            int at = cta_before_n + warp_before + incl_n - mine_n;
            const unsigned cand_local = (unsigned)__cvta_generic_to_shared(sh.cand);
            for (int j = j0; j < j1; ++j) {
                const float p = prob(j);
                if (p >= f_lo && p < f_hi) {
                    if (at < SC_CAND_MAX) {
#pragma unroll
                        for (unsigned to = 0; to < (unsigned)SC_CTAS; ++to) {
                            unsigned remote;
                            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(cand_local + 4u * (unsigned)at), "r"(to));
                            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(p) : "memory");
                        }
                    }
                    ++at;
                }
            }
            sc_cluster_sync();
            // ---- ... and finishes the search on the list, with no further exchange
            while (hi - lo > 1u) {
                uint32_t tb[SC_WAYS];
                float th[SC_WAYS];
                double sj[SC_VALS];
#pragma unroll
                for (int k = 0; k < SC_VALS; ++k) sj[k] = 0.0;
                uniform(tb);
#pragma unroll
                for (int k = 0; k < SC_WAYS; ++k) th[k] = (tb[k] < hi) ? __uint_as_float(tb[k]) : INFINITY;
                const float g_lo = th[0], g_hi = __uint_as_float(hi);
                for (int j = tid; j < total_n; j += SC_THREADS) {
                    const float p = sh.cand[j];
                    if (p >= g_lo && p < g_hi) {
                        const double pd = (double)p;
#pragma unroll
                        for (int k = 0; k < SC_WAYS; ++k) if (p >= th[k]) sj[k] += pd;
                    }
                }
                sc_block_sum(sh, sj, SC_WAYS);
                decide(sj, tb, false);
            }
        }
        tau = __uint_as_float(lo);
    }

    // ---- mass of the nucleus and the walk in index order: running sums over the threads' chunks, the CTAs in rank order
    double my_mass = 0.0;
    for (int j = j0; j < j1; ++j) { const float p = prob(j); if (p >= 0.f && p >= tau) my_mass += (double)p; }
    double incl = my_mass;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    __syncthreads();
    if (lane == 31) sh.warp_d[warp][0] = incl;
    if (tid == 0) sh.choice = 0x7fffffff;
    __syncthreads();
    double offset = 0.0, cta_mass = 0.0;
    for (int k = 0; k < SC_WARPS; ++k) { const double t = sh.warp_d[k][0]; if (k < warp) offset += t; cta_mass += t; }
    mine[0] = cta_mass;
    sc_all_gather(sh, parity, rank, mine, 1);
    double mass = 0.0, cta_before = 0.0;
    for (int c = 0; c < SC_CTAS; ++c) { const double t = sh.gather[parity][c][0]; if (c < (int)rank) cta_before += t; mass += t; }
    parity ^= 1;
    uint32_t c4[4];
    const unsigned long long st = (unsigned long long)((step ? step[row] : 0) + step_add), sid = (unsigned long long)(stream_id ? stream_id[row] : 0);
    const unsigned long long sd = (unsigned long long)(seed ? seed[row] : 0);
    c4[0] = (uint32_t)st; c4[1] = (uint32_t)(st >> 32); c4[2] = (uint32_t)sid; c4[3] = (uint32_t)(sid >> 32);
    philox4x32_10(c4, (uint32_t)sd, (uint32_t)(sd >> 32));
    const float u = (float)(c4[0] >> 8) * (1.0f / 16777216.0f);
    const double r = (double)u * mass;
    // the chunk in which the running sum first reaches r walks its members; the last member overall is kept as well
    const double before = cta_before + offset + incl - my_mass;
    int last_member = -1;
    for (int j = j1 - 1; j >= j0; --j) { const float p = prob(j); if (p >= 0.f && p >= tau) { last_member = i0 + j; break; } }
    if (before <= r) {
        double acc = before;
        for (int j = j0; j < j1; ++j) {
            const float p = prob(j);
            if (p >= 0.f && p >= tau) {
                acc += (double)p;
                if (acc >= r) { atomicMin(&sh.choice, i0 + j); break; }
            }
        }
    }
    last_member = max(last_member, __shfl_xor_sync(0xffffffffu, last_member, 16));
    last_member = max(last_member, __shfl_xor_sync(0xffffffffu, last_member, 8));
    last_member = max(last_member, __shfl_xor_sync(0xffffffffu, last_member, 4));
    last_member = max(last_member, __shfl_xor_sync(0xffffffffu, last_member, 2));
    last_member = max(last_member, __shfl_xor_sync(0xffffffffu, last_member, 1));
    __syncthreads();
    if (lane == 0) sh.warp_i[warp] = last_member;
    __syncthreads();
    last_member = -1;
    for (int k = 0; k < SC_WARPS; ++k) last_member = max(last_member, sh.warp_i[k]);
    // the CTA in whose range of the running sum r falls writes the token (exactly one does: the ranges tile [0, mass)); should
    // rounding have left its threads' running sums short of r, its last member
    if (tid == 0 && cta_before <= r && (r < cta_before + cta_mass || (cta_mass > 0.0 && cta_before + cta_mass >= mass)))
        out[row] = (sh.choice == 0x7fffffff) ? last_member : sh.choice;
}

constexpr int SAMPLE_CACHE_LIMIT = 200 * 1024;      // bytes of dynamic shared memory for a row's probabilities
constexpr int SC_CLUSTER_MIN_VOCAB = 8192;        // from this many tokens on, and ...
constexpr int SC_CLUSTER_MAX_ROWS = 64;           // ... up to this many rows, a cluster of CTAs samples a row

// The Philox counter of row r is step[r] + step_add: a caller whose rows all move on by the same number of draws
// leaves its parameter block on the device untouched.
VM_API int vm_sample(const float* logits, long long row_stride, int R, int V, const float* temperature,
                     const float* top_p, const long long* seed, const long long* stream_id, const long long* step,
                     long long step_add, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return VM_ERR_BAD_ARG;
    const size_t cache = (size_t)V * sizeof(float);
    if (V >= SC_CLUSTER_MIN_VOCAB && R <= SC_CLUSTER_MAX_ROWS) {
        // large vocabulary, few rows: eight CTAs per row
        const int slice = ((V + SC_CTAS - 1) / SC_CTAS + 3) / 4 * 4;
        const size_t smem = (size_t)slice * sizeof(float);
        if (smem <= SAMPLE_CACHE_LIMIT) {
            static bool configured_c = false;
            if (!configured_c) {
                cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMPLE_CACHE_LIMIT);
                if (e != cudaSuccess) return (int)e;
                configured_c = true;
            }
            sample_cluster_kernel<<<R * SC_CTAS, SC_THREADS, smem, stream>>>(logits, row_stride, V, slice, temperature, top_p, seed,
                                                                           stream_id, step, step_add, out);
            return vm_launch_status();
        }
    }
    if (cache <= SAMPLE_CACHE_LIMIT) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMPLE_CACHE_LIMIT);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        sample_kernel<true><<<R, SAMPLE_THREADS, cache, stream>>>(logits, row_stride, V, temperature, top_p, seed, stream_id, step, step_add, out);
    } else {
        sample_kernel<false><<<R, SAMPLE_THREADS, 0, stream>>>(logits, row_stride, V, temperature, top_p, seed, stream_id, step, step_add, out);
    }
    return vm_launch_status();
}

// ---------------------------------------------------------------- feeding sampled tokens back on the device
// After a decode step has been sampled: the sampled token becomes the next step's input, every sequence moves one
// place on, the draw counters advance, and the token is kept in `history[iteration, :]` for the host to read later.
// With this the host can queue several decode steps without waiting for the tokens of each.
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ tokens, int* __restrict__ positions,
                                      int* __restrict__ ctx_len, long long* __restrict__ draw_step, int* __restrict__ history,
                                      int* __restrict__ iteration, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    const int it = *iteration;
    if (b < B) {
        const int tok = sampled[b];
        tokens[b] = tok < 0 ? 0 : tok;          // a row without a valid choice keeps the step well-formed; the host sees -1
        positions[b] += 1;
        ctx_len[b] += 1;
        draw_step[b] += 1;
        history[(size_t)it * B + b] = tok;
    }
    __syncthreads();
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        // every block reads `iteration` before this block (the last one to start in practice) bumps it; with one block
        // (B <= 1024) the barrier above makes that exact
        *iteration = it + 1;
    }
}

VM_API int vm_decode_advance(const int* sampled, int* tokens, int* positions, int* ctx_len, long long* draw_step,
                             int* history, int* iteration, int B, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (B > 1024) return VM_ERR_UNSUPPORTED;     // one block, so that the iteration counter is read by all before it moves
    decode_advance_kernel<<<1, ((B + 31) / 32) * 32, 0, stream>>>(sampled, tokens, positions, ctx_len, draw_step, history, iteration, B);
    return vm_launch_status();
}
