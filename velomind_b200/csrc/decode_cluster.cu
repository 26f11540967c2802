// All layers of a decode step in one launch of thread-block clusters; nothing is synchronised across the grid.
//
// The sequences of a decode batch do not depend on one another, so every cluster of CS CTAs takes a few rows
// (sequences) of the batch through ALL layers by itself.  Inside a cluster the output columns of each matrix
// product are split over the CTAs; every CTA keeps a full copy of the rows' activations in shared memory and
// receives the other CTAs' columns through distributed shared memory (st.shared::cluster), with one
// mbarrier-based cluster barrier per phase.  A layer has five phases:
//
//   1  x = rmsnorm(h) (src/cpu/ops/rmsnorm.cpp:42-59); q,k,v = x Wqkv^T; rotary (rotary_embedding.cpp:30-44);
//      the new k and v go to the cache pages (llama_graph.cpp:210-215) and, with q, to every CTA
//   2  attention over the cached keys of the rows (src/cuda/ops/attention.cu: softmax(q k^T * scale) v), split
//      over (row, kv head, part); every part's (sums, max, denominator) goes to every CTA
//   3  every CTA joins the parts and the new token's own key into the attention rows; h += att Wo^T
//   4  x = rmsnorm(h); act = silu(x Wg^T) * (x Wu^T) (llama_graph.cpp:22-28)
//   5  h += act Wd^T
//
// The weights are the kernel's stream: they are packed once, at load time, into the order in which each CTA
// rank consumes them (engine/cluster.py), as ready-made mma.sync A fragments (the weights are the 16-row
// operand, the few activation rows the 8-column one), and a producer thread per CTA keeps a ring of
// shared-memory stages full with one bulk copy (cp.async.bulk) per stage, far ahead of the phase barriers: the
// stream never waits for a barrier, only for ring space.  The cached K and V pages of phase 2 come through the
// same ring.  Every wait has an iteration limit, after which the thread reports error 6 and stops waiting (the
// results are then garbage and the host raises); no thread leaves before the closing cluster barrier.
#include "mma.cuh"

namespace {

constexpr int CL_WARPS = 8;                       // consumer warps; warp 8 is the producer
constexpr int CL_THREADS = (CL_WARPS + 1) * 32;
constexpr int CL_MAX_STAGES = 16;
constexpr int CL_KS_MAX = 4;                      // k32 blocks of one unit in one stage, at most
constexpr int CL_FRAG = 1024;                     // bytes of the two A fragments (16 weight rows x 32 k) of a k32 block for 32 lanes
constexpr int CL_WAIT_LIMIT = 1 << 21;
constexpr int CL_ERR_WAIT = 6;
constexpr int CL_SMEM_LIMIT = 227 * 1024;         // dynamic shared memory of a CTA

struct ClLayer {                                  // 32 bytes per layer; laid out by engine/cluster.py
    const unsigned char* w;                       // packed weight stream of the layer: [cs][rank_stride] bytes
    const __nv_bfloat16* k;                       // cache pages of the layer [n_pages, Hkv, 64, D]
    const __nv_bfloat16* v;
    float eps1, eps2;
};

struct ClParams {
    const ClLayer* layers; int n_layers;
    int B, rpc, cs;                               // batch rows, rows per cluster, CTAs per cluster
    int hid, H, Hkv, D, I, V;
    float scale_log2; int window;
    const float* inv_freq; int rot;
    const int* tokens; const int* positions; const int* table; int max_blocks, n_pages;
    const void* embed; int embed_f32;
    float* h_out; int* err;
    unsigned long long* trace;                    // optional [phases][CTAs][2]: each CTA's arrival at and release from every phase barrier (ns)
    long long rank_stride;
    int ks_target;                                // k32 blocks of a warp's unit per ring stage, at most (see choose_split)
    int P;                                        // parts per (row, kv head) in phase 2
    int stage_bytes, n_stages;
    int o_h, o_xa, o_qa, o_part, o_res, o_ipart, o_wst, o_cs, o_pos, o_tab, o_snew, o_red, o_nred, o_layers, o_ring;   // shared memory offsets
    int hp, xap, qap;                             // row pitches in elements of h (float), xa and qa (bf16)
};

// ---------------------------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ unsigned su32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint64_t* b, int n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(su32(b)), "r"(n));
}
__device__ __forceinline__ void mb_expect(uint64_t* b, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(su32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mb_arrive(uint64_t* b, int n) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(su32(b)), "r"(n) : "memory");
}
__device__ __forceinline__ bool mb_try(uint64_t* b, unsigned parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(su32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mb_try_cluster(uint64_t* b, unsigned parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(su32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(su32(bar)) : "memory");
}
__device__ __forceinline__ unsigned mapa(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_remote16(unsigned addr, const uint4& v) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void remote_arrive(unsigned addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CL_WARPS * 32) : "memory"); }
__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// How a rank's units of one product are dealt out to the eight consumer warps: `ksplit` warps share a unit (each takes
// ksteps / ksplit consecutive k32 blocks of it), 8 / ksplit units run at a time (a round), and a round is cut along
// K into `chunks` ring stages of `ks` blocks per warp.  Chosen to make the chain of dependent steps short; the
// same rule packs the stream (engine/cluster.py: choose_split).
struct Split { int ksplit, ks, upr, rounds, chunks; };
__host__ __device__ inline Split choose_split(int n_units, int ksteps, int ks_target) {
    Split best{1, 1, 8, 0, 0};
    long best_cost = -1;
    for (int ksplit = 1; ksplit <= 8; ksplit *= 2) {
        if (ksteps % ksplit) continue;
        const int per = ksteps / ksplit, upr = 8 / ksplit;
        int ks = 1;
        for (int d = 1; d <= ks_target && d <= per; ++d) if (per % d == 0) ks = d;
        const int rounds = (n_units + upr - 1) / upr;
        const long cost = (long)rounds * (per + 2 * (per / ks) + 16);   // blocks; a stage's and a round's fixed cost in blocks
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = Split{ksplit, ks, upr, rounds, per / ks}; }
    }
    return best;
}

// Blocked split of n units over cs ranks.
__device__ __forceinline__ int unit_begin(int n, int cs, int rank) { return (int)((long long)n * rank / cs); }

struct Item { int r, kv, pa, pb, pos, lo; };
// Part `id` of phase 2: (row, kv head, part) and the cache pages [pa, pb) it reads (keys before the new token only).
__device__ __forceinline__ Item item_of(int id, int P, int Hkv, const int* spos, int window) {
    Item it;
    const int part = id % P, rk = id / P;
    it.kv = rk % Hkv; it.r = rk / Hkv;
    it.pos = spos[it.r];
    it.lo = (window > 0 && it.pos - window + 1 > 0) ? it.pos - window + 1 : 0;
    const int first = it.lo / VM_PAGE_TOKENS, end = (it.pos + VM_PAGE_TOKENS - 1) / VM_PAGE_TOKENS;
    const int pages = end > first ? end - first : 0;
    const int per = (pages + P - 1) / P;
    it.pa = first + part * per;
    it.pb = min(end, it.pa + per);
    if (it.pb < it.pa) it.pb = it.pa;
    return it;
}

// What a consumer thread carries through the kernel (passed in and out of the phase functions by value).
struct Walk {
    unsigned slot, par;   // the ring stage that comes next, and the parity of its `full` barrier
    unsigned ph;          // phases finished so far
    unsigned rd;          // joins of warps that shared a unit so far (the join buffer alternates)
    unsigned dead;        // a wait gave up: wait no more
};

// The start of dynamic shared memory: barriers, a copy of the parameters (the phase functions are separate
// functions and read them here), and what the CTA worked out about its own share at the start.
struct ClShared {
    uint64_t full[CL_MAX_STAGES], empty[CL_MAX_STAGES], phasebar[2];
    ClParams p;
    int rank, row0, R, n_items, cs_log;
    int u0[4], n_units[4];           // this rank's units of the four products: q k v, out, gate and up, down
    Split split[4];
};
constexpr int CL_HEADER = 1024;
static_assert(sizeof(ClShared) <= CL_HEADER, "the shared-memory header outgrew its reserve");

extern __shared__ __align__(128) unsigned char cl_smem[];
__device__ __forceinline__ ClShared& shared_header() { return *reinterpret_cast<ClShared*>(cl_smem); }

__device__ __forceinline__ void ring_advance(unsigned& slot, unsigned& par, unsigned n, unsigned S) {
    slot += n;
    while (slot >= S) { slot -= S; par ^= 1u; }
}
__device__ __forceinline__ void wait_full(uint64_t* bar, unsigned parity, Walk& w, int* err) {
    if (w.dead) return;
    for (int i = 0; i < CL_WAIT_LIMIT; ++i) if (mb_try(bar, parity)) return;
    w.dead = 1u;
    atomicExch(err, CL_ERR_WAIT);
}

enum : int { PROD_QKV = 0, PROD_OUT = 1, PROD_GU = 2, PROD_DOWN = 3 };

// ---------------------------------------------------------------------------------------------- producer
// One thread per CTA: keeps the ring full, in the order the consumers read it.
template <int D>
__device__ __noinline__ void cl_producer() {
    ClShared& C = shared_header();
    const ClParams& p = C.p;
    const int S = p.n_stages, CS = p.cs, Hkv = p.Hkv;
    constexpr unsigned PAGE_BYTES = VM_PAGE_TOKENS * D * 2;
    const int* spos = reinterpret_cast<const int*>(cl_smem + p.o_pos);
    const int* stab = reinterpret_cast<const int*>(cl_smem + p.o_tab);
    unsigned char* ring = cl_smem + p.o_ring;
    unsigned slot = 0, par = 0, count = 0;
    bool dead = false;
    auto issue = [&](const void* src, unsigned bytes, const void* src2, unsigned bytes2) {
        if (count >= (unsigned)S && !dead) {              // the slot's previous use must have been read
            bool ok = false;
            for (int i = 0; i < CL_WAIT_LIMIT; ++i) if (mb_try(&C.empty[slot], par ^ 1u)) { ok = true; break; }
            if (!ok) { dead = true; atomicExch(p.err, CL_ERR_WAIT); }
        }
        mb_expect(&C.full[slot], bytes + bytes2);
        const unsigned dst = su32(ring + (size_t)slot * p.stage_bytes);
        bulk_g2s(dst, src, bytes, &C.full[slot]);
        if (bytes2) bulk_g2s(dst + bytes, src2, bytes2, &C.full[slot]);
        ++count;
        ring_advance(slot, par, 1, S);
    };
    auto gemm_stages = [&](const unsigned char*& wp, int which) {
        const Split sp = C.split[which];
        const int n_units = C.n_units[which];
        for (int rd = 0; rd < sp.rounds; ++rd) {
            const unsigned bytes = (unsigned)(min(sp.upr, n_units - rd * sp.upr) * sp.ksplit * sp.ks) * CL_FRAG;
            for (int j = 0; j < sp.chunks; ++j) { issue(wp, bytes, nullptr, 0); wp += bytes; }
        }
    };
    const ClLayer* layers = reinterpret_cast<const ClLayer*>(cl_smem + p.o_layers);
    for (int l = 0; l < p.n_layers; ++l) {
        const ClLayer L = layers[l];
        const unsigned char* wp = L.w + (size_t)C.rank * p.rank_stride;
        issue(wp, p.hid * 4, nullptr, 0); wp += p.hid * 4;                               // norm 1
        gemm_stages(wp, PROD_QKV);
        for (int id = C.rank; id < C.n_items; id += CS) {                                // cached pages
            const Item im = item_of(id, p.P, Hkv, spos, p.window);
            for (int pg = im.pa; pg < im.pb; ++pg) {
                int page = (pg < p.max_blocks) ? stab[im.r * p.max_blocks + pg] : -1;
                if (page < 0 || page >= p.n_pages) { atomicExch(p.err, 3); page = 0; }
                const size_t off = ((size_t)page * Hkv + im.kv) * VM_PAGE_TOKENS * D;
                issue(L.k + off, PAGE_BYTES, L.v + off, PAGE_BYTES);
            }
        }
        gemm_stages(wp, PROD_OUT);
        issue(wp, p.hid * 4, nullptr, 0); wp += p.hid * 4;                               // norm 2
        gemm_stages(wp, PROD_GU);
        gemm_stages(wp, PROD_DOWN);
    }
}

// ---------------------------------------------------------------------------------------------- consumer phases
// End of a phase: this warp's remote stores are done; tell every CTA, then wait for every CTA's warps.
__device__ __forceinline__ Walk cl_phase_end(Walk w) {
    ClShared& C = shared_header();
    const int lane = threadIdx.x & 31;
    __syncwarp();                  // the lanes' remote stores are ordered before the release below
    if (C.p.trace && threadIdx.x == 0) C.p.trace[((size_t)w.ph * gridDim.x + blockIdx.x) * 2] = globaltimer();
    uint64_t* bar = &C.phasebar[w.ph & 1];
    if (lane < C.p.cs) remote_arrive(mapa(su32(bar), (unsigned)lane));
    if (!w.dead) {
        const unsigned parity = (w.ph >> 1) & 1;
        bool ok = false;
        for (int i = 0; i < CL_WAIT_LIMIT; ++i) if (mb_try_cluster(bar, parity)) { ok = true; break; }
        if (!ok) { w.dead = 1u; atomicExch(C.p.err, CL_ERR_WAIT); }
    }
    if (C.p.trace && threadIdx.x == 0) C.p.trace[((size_t)w.ph * gridDim.x + blockIdx.x) * 2 + 1] = globaltimer();
    ++w.ph;
    return w;
}

// x = rmsnorm(h) * weight into xa (the weight comes through the ring as one stage); all warps share every row.
__device__ __forceinline__ Walk cl_norm(Walk w, float eps) {
    ClShared& C = shared_header();
    const ClParams& p = C.p;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, R = C.R, hid = p.hid;
    const float* h = reinterpret_cast<const float*>(cl_smem + p.o_h);
    __nv_bfloat16* xa = reinterpret_cast<__nv_bfloat16*>(cl_smem + p.o_xa);
    float* nred = reinterpret_cast<float*>(cl_smem + p.o_nred);
    for (int r = 0; r < R; ++r) {
        float ss = 0.f;
        for (int k = tid; k < hid; k += CL_WARPS * 32) { const float v = h[r * p.hp + k]; ss += v * v; }
        ss = vm_warp_sum(ss);
        if (lane == 0) nred[warp * 16 + r] = ss;
    }
    consumer_sync();
    wait_full(&C.full[w.slot], w.par, w, p.err);
    const float* nw = reinterpret_cast<const float*>(cl_smem + p.o_ring + (size_t)w.slot * p.stage_bytes);
    for (int r = 0; r < R; ++r) {
        float ss = 0.f;
#pragma unroll
        for (int ww = 0; ww < CL_WARPS; ++ww) ss += nred[ww * 16 + r];
        const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
        for (int k = tid; k < hid; k += CL_WARPS * 32) xa[r * p.xap + k] = __float2bfloat16_rn(h[r * p.hp + k] * inv * nw[k]);
    }
    __syncwarp();
    if (lane == 0) mb_arrive(&C.empty[w.slot], 1);
    ring_advance(w.slot, w.par, 1, p.n_stages);
    consumer_sync();
    return w;
}

// Send this warp's tile in `wst` (rows r < R; `ppr` 16-byte pieces per row, `row_bytes` apart) to every CTA of the
// cluster; piece q of row r goes to shared-memory address dst0 + r * dst_row_bytes + q * dst_piece_bytes there.
__device__ __forceinline__ void send_tile(const unsigned char* wst, int R, int cs_log, int ppr_log, int row_bytes, unsigned dst0,
                                          int dst_row_bytes, int dst_piece_bytes) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    const int n = (R << ppr_log) << cs_log;
    for (int x = lane; x < n; x += 32) {
        const int dest = x & ((1 << cs_log) - 1), pc = x >> cs_log;
        const int r = pc >> ppr_log, q = pc & ((1 << ppr_log) - 1);
        const uint4 v = *reinterpret_cast<const uint4*>(wst + r * row_bytes + q * 16);
        st_remote16(mapa(dst0 + r * dst_row_bytes + q * dst_piece_bytes, (unsigned)dest), v);
    }
    __syncwarp();
}

// One product of a phase: this rank's units of W (16 weight rows each) against the rows in X, and its epilogue.
template <int D, int NB>
__device__ __forceinline__ Walk cl_gemm(Walk w, int layer, const int WHICH) {
    ClShared& C = shared_header();
    const ClParams& p = C.p;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int R = C.R, CS = p.cs, S = p.n_stages, H = p.H, Hkv = p.Hkv;
    constexpr int DH = D / 2;
    const Split sp = C.split[WHICH];
    const int n_units = C.n_units[WHICH], u0 = C.u0[WHICH];
    const int ksteps = (WHICH == PROD_OUT) ? (H * D) / 32 : (WHICH == PROD_DOWN ? p.I / 32 : p.hid / 32);   // k32 blocks
    const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(cl_smem + (WHICH == PROD_DOWN ? p.o_qa : p.o_xa));
    const int xpitch = (WHICH == PROD_DOWN) ? p.qap : p.xap;
    float* h = reinterpret_cast<float*>(cl_smem + p.o_h);
    __nv_bfloat16* qa = reinterpret_cast<__nv_bfloat16*>(cl_smem + p.o_qa);
    unsigned char* wst = cl_smem + p.o_wst + warp * 1024;
    float* red = reinterpret_cast<float*>(cl_smem + p.o_red);
    const unsigned char* ring = cl_smem + p.o_ring;
    const int unit_l = warp / sp.ksplit, slice = warp - unit_l * sp.ksplit;
    const int k_first = slice * (ksteps / sp.ksplit);

    for (int rd = 0; rd < sp.rounds; ++rd) {
        const int units_now = min(sp.upr, n_units - rd * sp.upr);
        const int warps_now = units_now * sp.ksplit;
        const bool active = unit_l < units_now;
        float acc[2][NB][4];
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) acc[c][nb][0] = acc[c][nb][1] = acc[c][nb][2] = acc[c][nb][3] = 0.f;
        if (active) {
            unsigned slot = w.slot, par = w.par;
            for (int j = 0; j < sp.chunks; ++j) {
                wait_full(&C.full[slot], par, w, p.err);
                const unsigned char* a_base = ring + (size_t)slot * p.stage_bytes + (size_t)warp * sp.ks * CL_FRAG + lane * 16;
                const __nv_bfloat16* x_base = X + (size_t)g * xpitch + (size_t)(k_first + j * sp.ks) * 32 + 8 * t4;
                // a k32 block is two mma steps; the weights were packed so that one 16-byte load of a row of X is the B
                // operand of both (engine/cluster.py: _fragments)
                uint4 a[CL_KS_MAX][2], b[CL_KS_MAX][NB];
#pragma unroll
                for (int t = 0; t < CL_KS_MAX; ++t) {
                    if (t < sp.ks) {
                        a[t][0] = *reinterpret_cast<const uint4*>(a_base + t * CL_FRAG);
                        a[t][1] = *reinterpret_cast<const uint4*>(a_base + t * CL_FRAG + CL_FRAG / 2);
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb)
                            b[t][nb] = *reinterpret_cast<const uint4*>(x_base + (size_t)nb * 8 * xpitch + t * 32);
                    }
                }
#pragma unroll
                for (int t = 0; t < CL_KS_MAX; ++t) {
                    if (t < sp.ks) {
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {             // two chains of dependent mma instead of one
                            vm_mma_bf16_16816(acc[0][nb], a[t][0].x, a[t][0].y, a[t][0].z, a[t][0].w, b[t][nb].x, b[t][nb].y);
                            vm_mma_bf16_16816(acc[1][nb], a[t][1].x, a[t][1].y, a[t][1].z, a[t][1].w, b[t][nb].z, b[t][nb].w);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mb_arrive(&C.empty[slot], warp == 0 ? CL_WARPS - warps_now + 1 : 1);
                ring_advance(slot, par, 1, S);
            }
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                acc[0][nb][0] += acc[1][nb][0]; acc[0][nb][1] += acc[1][nb][1];
                acc[0][nb][2] += acc[1][nb][2]; acc[0][nb][3] += acc[1][nb][3];
            }
        }
        ring_advance(w.slot, w.par, sp.chunks, S);
        if (sp.ksplit > 1) {                                          // join the warps that shared a unit, in a fixed order
            float* rbuf = red + (size_t)(w.rd & 1) * CL_WARPS * NB * 128;
            if (active && slice > 0) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
                    *reinterpret_cast<float4*>(rbuf + ((size_t)warp * NB + nb) * 128 + lane * 4) =
                        make_float4(acc[0][nb][0], acc[0][nb][1], acc[0][nb][2], acc[0][nb][3]);
            }
            consumer_sync();
            if (active && slice == 0) {
                for (int sl = 1; sl < sp.ksplit; ++sl) {
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const float4 v = *reinterpret_cast<const float4*>(rbuf + ((size_t)(warp + sl) * NB + nb) * 128 + lane * 4);
                        acc[0][nb][0] += v.x; acc[0][nb][1] += v.y; acc[0][nb][2] += v.z; acc[0][nb][3] += v.w;
                    }
                }
            }
            ++w.rd;
        }
        if (!(active && slice == 0)) continue;
        // ---- epilogue of unit u: acc[0][nb] = {(row g, r), (row g, r+1), (row g+8, r), (row g+8, r+1)}, r = 8 nb + 2 t4
        const int u = u0 + rd * sp.upr + unit_l;
        if (WHICH == PROD_QKV) {            // rotary, cache write, q k v of the new tokens to every CTA
            const float* cs_tab = reinterpret_cast<const float*>(cl_smem + p.o_cs);
            const int* spos = reinterpret_cast<const int*>(cl_smem + p.o_pos);
            const int* stab = reinterpret_cast<const int*>(cl_smem + p.o_tab);
            const int head = u / (D / 16), d0 = (u - head * (D / 16)) * 8;      // columns head*D + d0 + g and + D/2
            __nv_bfloat16* t = reinterpret_cast<__nv_bfloat16*>(wst);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int r = nb * 8 + 2 * t4 + e;
                    if (r < R) {
                        float ya = acc[0][nb][e], yb = acc[0][nb][2 + e];
                        if (head < H + Hkv && p.rot > 0) {
                            const float c = cs_tab[2 * (r * DH + d0 + g)], sn = cs_tab[2 * (r * DH + d0 + g) + 1];
                            const float x1 = ya, x2 = yb;
                            ya = x1 * c - x2 * sn;
                            yb = x2 * c + x1 * sn;
                        }
                        const __nv_bfloat16 va = __float2bfloat16_rn(ya), vb = __float2bfloat16_rn(yb);
                        t[r * 16 + g] = va; t[r * 16 + 8 + g] = vb;
                        if (head >= H) {                                        // the new token's k or v: into its cache page
                            const int pos = spos[r], blk = pos / VM_PAGE_TOKENS;
                            const int page = (blk < p.max_blocks) ? stab[r * p.max_blocks + blk] : -1;
                            if (page < 0 || page >= p.n_pages) { atomicExch(p.err, 2); }
                            else {
                                const bool is_k = head < H + Hkv;
                                const int hk = is_k ? head - H : head - H - Hkv;
                                const ClLayer& L = reinterpret_cast<const ClLayer*>(cl_smem + p.o_layers)[layer];
                                __nv_bfloat16* dst = const_cast<__nv_bfloat16*>(is_k ? L.k : L.v)
                                    + (((size_t)page * Hkv + hk) * VM_PAGE_TOKENS + pos % VM_PAGE_TOKENS) * D + d0 + g;
                                dst[0] = va; dst[DH] = vb;
                            }
                        }
                    }
                }
            }
            send_tile(wst, R, C.cs_log, 1, 32, su32(qa + head * D + d0), p.qap * 2, DH * 2);
        } else if (WHICH == PROD_GU) {      // SwiGLU; act to every CTA
            __nv_bfloat16* t = reinterpret_cast<__nv_bfloat16*>(wst);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int r = nb * 8 + 2 * t4 + e;
                    if (r < R) {
                        const float gate = acc[0][nb][e], up = acc[0][nb][2 + e];
                        const float sig = 1.0f / (1.0f + expf(-gate));
                        t[r * 8 + g] = __float2bfloat16_rn((sig * gate) * up);
                    }
                }
            }
            send_tile(wst, R, C.cs_log, 0, 16, su32(qa + 8 * u), p.qap * 2, 0);
        } else {                            // h[:, 16u .. 16u+16) += acc; the new columns to every CTA
            float* t = reinterpret_cast<float*>(wst);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int r = nb * 8 + 2 * t4 + e;
                    if (r < R) {
                        t[r * 16 + g] = h[r * p.hp + 16 * u + g] + acc[0][nb][e];
                        t[r * 16 + 8 + g] = h[r * p.hp + 16 * u + 8 + g] + acc[0][nb][2 + e];
                    }
                }
            }
            send_tile(wst, R, C.cs_log, 2, 64, su32(h + 16 * u), p.hp * 4, 16);
        }
    }
    return w;
}

// Phase 2: this rank's parts of the attention over the cached keys; every part goes to every CTA.
template <int D>
__device__ __forceinline__ Walk cl_attention(Walk w) {
    ClShared& C = shared_header();
    const ClParams& p = C.p;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int CS = p.cs, S = p.n_stages, Hkv = p.Hkv, G = p.H / p.Hkv, P = p.P;
    constexpr int PW = D + 4;
    const __nv_bfloat16* qa = reinterpret_cast<const __nv_bfloat16*>(cl_smem + p.o_qa);
    float* part = reinterpret_cast<float*>(cl_smem + p.o_part);
    float* res = reinterpret_cast<float*>(cl_smem + p.o_res);
    float* ipart = reinterpret_cast<float*>(cl_smem + p.o_ipart);
    const int* spos = reinterpret_cast<const int*>(cl_smem + p.o_pos);
    const unsigned char* ring = cl_smem + p.o_ring;

    for (int id = C.rank; id < C.n_items; id += CS) {
        const Item im = item_of(id, P, Hkv, spos, p.window);
        const int n_pg = im.pb - im.pa;
        const int h0 = im.kv * G;
        // the queries of the kv head's G heads as the rows of the tile (rows past G are zero)
        unsigned qf[D / 16][4];
        {
            const __nv_bfloat16* qrow = qa + im.r * p.qap + (size_t)(h0 + g) * D + 2 * t4;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                qf[kk][0] = (g < G) ? *reinterpret_cast<const unsigned*>(qrow + kk * 16) : 0u;
                qf[kk][2] = (g < G) ? *reinterpret_cast<const unsigned*>(qrow + kk * 16 + 8) : 0u;
                qf[kk][1] = (g + 8 < G) ? *reinterpret_cast<const unsigned*>(qrow + 8 * D + kk * 16) : 0u;
                qf[kk][3] = (g + 8 < G) ? *reinterpret_cast<const unsigned*>(qrow + 8 * D + kk * 16 + 8) : 0u;
            }
        }
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
        float o[D / 8][4];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
        unsigned slot = w.slot, par = w.par;
        ring_advance(slot, par, warp, S);
        for (int x = warp; x < n_pg; x += CL_WARPS) {
            wait_full(&C.full[slot], par, w, p.err);
            const __nv_bfloat16* ks = reinterpret_cast<const __nv_bfloat16*>(ring + (size_t)slot * p.stage_bytes);
            const __nv_bfloat16* vs = ks + VM_PAGE_TOKENS * D;
            const int key0 = (im.pa + x) * VM_PAGE_TOKENS;
            float s[VM_PAGE_TOKENS / 8][4];
#pragma unroll
            for (int nb = 0; nb < VM_PAGE_TOKENS / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < VM_PAGE_TOKENS / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    vm_ldmatrix_x4(b0, b1, b2, b3, ks + (nb * 8 + (lane & 7) + 8 * (lane >> 4)) * D + kk * 16 + 8 * ((lane >> 3) & 1));
                    vm_mma_bf16_16816(s[nb], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
                    vm_mma_bf16_16816(s[nb + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < VM_PAGE_TOKENS / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + nb * 8 + 2 * t4 + e;
                    const bool ok = (key < im.pos && key >= im.lo);
                    const float va = ok ? s[nb][e] * p.scale_log2 : -INFINITY;
                    const float vb = ok ? s[nb][2 + e] * p.scale_log2 : -INFINITY;
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
            unsigned pa[VM_PAGE_TOKENS / 16][4];
#pragma unroll
            for (int nb = 0; nb < VM_PAGE_TOKENS / 8; ++nb) {
                const float p0 = exp2f(s[nb][0] - use_a), p1 = exp2f(s[nb][1] - use_a);
                const float p2 = exp2f(s[nb][2] - use_b), p3 = exp2f(s[nb][3] - use_b);
                sum_a += p0 + p1; sum_b += p2 + p3;
                pa[nb >> 1][(nb & 1) * 2 + 0] = vm_pack_bf16(p0, p1);
                pa[nb >> 1][(nb & 1) * 2 + 1] = vm_pack_bf16(p2, p3);
            }
            l_a = l_a * al_a + sum_a; l_b = l_b * al_b + sum_b;
            m_a = mn_a; m_b = mn_b;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
#pragma unroll
            for (int kk = 0; kk < VM_PAGE_TOKENS / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < D / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    vm_ldmatrix_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * D + nb * 8 + 8 * (lane >> 4));
                    vm_mma_bf16_16816(o[nb], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    vm_mma_bf16_16816(o[nb + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
            __syncwarp();
            if (lane == 0) mb_arrive(&C.empty[slot], CL_WARPS);      // the page had one reader
            ring_advance(slot, par, CL_WARPS, S);
        }
        ring_advance(w.slot, w.par, n_pg, S);
        // this warp's rows (sums, max, denominator) -> res; the quad's denominators are joined first
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        {
            float* ra = res + ((size_t)warp * G + g) * (D + 2);
            float* rb = res + ((size_t)warp * G + g + 8) * (D + 2);
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                const int d = i * 8 + 2 * t4;
                if (g < G) { ra[d] = o[i][0]; ra[d + 1] = o[i][1]; }
                if (g + 8 < G) { rb[d] = o[i][2]; rb[d + 1] = o[i][3]; }
            }
            if (t4 == 0) {
                if (g < G) { ra[D] = m_a; ra[D + 1] = l_a; }
                if (g + 8 < G) { rb[D] = m_b; rb[D + 1] = l_b; }
            }
        }
        consumer_sync();
        for (int i = tid; i < G * D; i += CL_WARPS * 32) {          // join the warps
            const int r = i / D, d = i - r * D;
            float M = -INFINITY;
#pragma unroll
            for (int ww = 0; ww < CL_WARPS; ++ww) M = fmaxf(M, res[((size_t)ww * G + r) * (D + 2) + D]);
            float acc = 0.f, Lsum = 0.f;
#pragma unroll
            for (int ww = 0; ww < CL_WARPS; ++ww) {
                const float* rr = res + ((size_t)ww * G + r) * (D + 2);
                const float f = (rr[D] == -INFINITY) ? 0.f : exp2f(rr[D] - M);
                acc += f * rr[d]; Lsum += f * rr[D + 1];
            }
            ipart[r * PW + d] = acc;
            if (d == 0) { ipart[r * PW + D] = M; ipart[r * PW + D + 1] = Lsum; ipart[r * PW + D + 2] = 0.f; ipart[r * PW + D + 3] = 0.f; }
        }
        consumer_sync();
        {                                                            // the part to every CTA
            constexpr int PCS = PW / 4;                              // 16-byte pieces per head
            const int n = G * PCS * CS;
            const unsigned dst0 = su32(part + (size_t)id * G * PW);
            for (int x = tid; x < n; x += CL_WARPS * 32) {
                const int dest = x & (CS - 1), pc = x >> C.cs_log;
                const uint4 v = *reinterpret_cast<const uint4*>(ipart + pc * 4);
                st_remote16(mapa(dst0 + pc * 16, (unsigned)dest), v);
            }
        }
        consumer_sync();                                             // res and ipart may be reused
    }
    return w;
}

// Start of phase 3: every CTA joins the parts of every (row, head) and the new token's own key into the attention rows.
template <int D>
__device__ __forceinline__ void cl_join() {
    ClShared& C = shared_header();
    const ClParams& p = C.p;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int R = C.R, H = p.H, Hkv = p.Hkv, G = H / Hkv, P = p.P;
    constexpr int PW = D + 4;
    const __nv_bfloat16* qa = reinterpret_cast<const __nv_bfloat16*>(cl_smem + p.o_qa);
    __nv_bfloat16* xa = reinterpret_cast<__nv_bfloat16*>(cl_smem + p.o_xa);
    const float* part = reinterpret_cast<const float*>(cl_smem + p.o_part);
    float* snew = reinterpret_cast<float*>(cl_smem + p.o_snew);
    for (int i = warp; i < R * H; i += CL_WARPS) {                   // the new token's own key: q . k_new
        const int r = i / H, hh = i - r * H, kv = hh / G;
        const __nv_bfloat16* qv = qa + r * p.qap + (size_t)hh * D;
        const __nv_bfloat16* kn = qa + r * p.qap + (size_t)(H + kv) * D;
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) dot += __bfloat162float(qv[d]) * __bfloat162float(kn[d]);
        dot = vm_warp_sum(dot);
        if (lane == 0) snew[i] = dot * p.scale_log2;
    }
    consumer_sync();
    const int d = tid % D;
    for (int r = 0; r < R; ++r) {
        for (int hh = tid / D; hh < H; hh += CL_WARPS * 32 / D) {
            const int kv = hh / G, hg = hh - kv * G;
            const float sn = snew[r * H + hh];
            const float* pp = part + ((size_t)(r * Hkv + kv) * P * G + hg) * PW;      // part 0; parts are G*PW apart
            float M = sn;
            for (int q = 0; q < P; ++q) M = fmaxf(M, pp[(size_t)q * G * PW + D]);
            const float fn = exp2f(sn - M);
            float acc = fn * __bfloat162float(qa[r * p.qap + (size_t)(H + Hkv + kv) * D + d]);
            float Lsum = fn;
            for (int q = 0; q < P; ++q) {
                const float* pq = pp + (size_t)q * G * PW;
                const float f = (pq[D] == -INFINITY) ? 0.f : exp2f(pq[D] - M);
                acc += f * pq[d]; Lsum += f * pq[D + 1];
            }
            xa[r * p.xap + hh * D + d] = __float2bfloat16_rn(acc / Lsum);
        }
    }
    consumer_sync();
}

// One layer for the consumer warps.  A function of its own (not inlined into the loop over the layers), so that the
// compiler keeps each phase's addresses and constants only while the phase runs.
template <int D, int NB>
__device__ __noinline__ Walk cl_layer(Walk w, int l) {
    const ClLayer* layers = reinterpret_cast<const ClLayer*>(cl_smem + shared_header().p.o_layers);
    // the four products share one copy of the code (a loop that is not unrolled): q k v, out, gate and up, down
#pragma unroll 1
    for (int which = PROD_QKV; which <= PROD_DOWN; ++which) {
        if (which == PROD_QKV || which == PROD_GU)        // phases 1 and 4 begin with a norm
            w = cl_norm(w, which == PROD_QKV ? layers[l].eps1 : layers[l].eps2);
        if (which == PROD_OUT) cl_join<D>();              // phase 3 begins by joining the attention parts
        w = cl_gemm<D, NB>(w, l, which);
        w = cl_phase_end(w);
        if (which == PROD_QKV) {                          // phase 2: attention over the cached keys
            w = cl_attention<D>(w);
            w = cl_phase_end(w);
        }
    }
    return w;
}

// ---------------------------------------------------------------------------------------------- the kernel
template <int D, int NB>
__global__ void __launch_bounds__(CL_THREADS, 1) decode_cluster_kernel(const ClParams p) {
    ClShared& C = shared_header();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned rank, cid;
    asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm("mov.u32 %0, %%clusterid.x;" : "=r"(cid));
    const int CS = p.cs, S = p.n_stages, hid = p.hid;
    const int row0 = (int)cid * p.rpc;
    const int R = min(p.rpc, p.B - row0);
    constexpr int DH = D / 2;
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mb_init(&C.full[s], 1); mb_init(&C.empty[s], CL_WARPS); }
        mb_init(&C.phasebar[0], CS * CL_WARPS);
        mb_init(&C.phasebar[1], CS * CL_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        C.p = p;
        C.rank = (int)rank; C.row0 = row0; C.R = R; C.n_items = R * p.Hkv * p.P;
        C.cs_log = 31 - __clz(CS);
        const int n[4] = {(p.H + 2 * p.Hkv) * D / 16, hid / 16, p.I / 8, hid / 16};
        const int ksteps[4] = {hid / 32, p.H * D / 32, hid / 32, p.I / 32};      // k32 blocks
        for (int i = 0; i < 4; ++i) {
            C.u0[i] = unit_begin(n[i], CS, rank);
            C.n_units[i] = unit_begin(n[i], CS, rank + 1) - C.u0[i];
            C.split[i] = choose_split(C.n_units[i], ksteps[i], p.ks_target);
        }
    }
    int* spos = reinterpret_cast<int*>(cl_smem + p.o_pos);
    int* stab = reinterpret_cast<int*>(cl_smem + p.o_tab);
    for (int i = tid; i < p.n_layers * (int)(sizeof(ClLayer) / 4); i += CL_THREADS)
        reinterpret_cast<unsigned*>(cl_smem + p.o_layers)[i] = reinterpret_cast<const unsigned*>(p.layers)[i];
    for (int i = tid; i < R; i += CL_THREADS) spos[i] = p.positions[row0 + i];
    for (int i = tid; i < R * p.max_blocks; i += CL_THREADS)
        stab[i] = p.table[(size_t)(row0 + i / p.max_blocks) * p.max_blocks + i % p.max_blocks];
    __syncthreads();
    cluster_sync_all();          // every CTA's barriers exist before anyone arrives on them

    if (warp == CL_WARPS) {
        if (lane == 0) cl_producer<D>();
        __syncwarp();
    } else {
        float* h = reinterpret_cast<float*>(cl_smem + p.o_h);
        // cos/sin of the rows' positions; embedding rows into h
        if (p.rot > 0) {
            float* cs_tab = reinterpret_cast<float*>(cl_smem + p.o_cs);                 // [rows][D/2][cos, sin]
            for (int i = tid; i < R * DH; i += CL_WARPS * 32) {
                const int r = i / DH, j = i - r * DH;
                float sn, c;
                sincosf((float)spos[r] * p.inv_freq[j], &sn, &c);
                cs_tab[2 * i] = c; cs_tab[2 * i + 1] = sn;
            }
        }
        for (int i = tid; i < R * hid; i += CL_WARPS * 32) {
            const int r = i / hid, k = i - r * hid;
            int tok = p.tokens[row0 + r];
            if (tok < 0 || tok >= p.V) { atomicExch(p.err, 1); tok = 0; }
            h[r * p.hp + k] = p.embed_f32 ? static_cast<const float*>(p.embed)[(size_t)tok * hid + k]
                                          : __bfloat162float(static_cast<const __nv_bfloat16*>(p.embed)[(size_t)tok * hid + k]);
        }
        consumer_sync();
        Walk w{0u, 0u, 0u, 0u, 0u};
        for (int l = 0; l < p.n_layers; ++l) w = cl_layer<D, NB>(w, l);
        // the rows' residual stream for the final norm and the head: each rank writes its share of the columns
        {
            const int c0 = unit_begin(hid, CS, rank), c1 = unit_begin(hid, CS, rank + 1), wdt = c1 - c0;
            for (int i = tid; i < R * wdt; i += CL_WARPS * 32) {
                const int r = i / wdt, c = c0 + i - r * wdt;
                p.h_out[(size_t)(row0 + r) * hid + c] = h[r * p.hp + c];
            }
        }
    }
    cluster_sync_all();          // nobody leaves while a peer may still write into its shared memory
}

// ---------------------------------------------------------------------------------------------- host side
inline int round_up(int x, int a) { return (x + a - 1) / a * a; }

// Shared-memory layout for `rows` rows per cluster; returns the total, or -1 if fewer than three ring stages fit.
int cluster_layout(ClParams& p, int rows) {
    const int RB = rows <= 8 ? 8 : 16;
    const int G = p.H / p.Hkv, QW = (p.H + 2 * p.Hkv) * p.D;
    p.hp = p.hid + 4;
    auto pitch = [](int k) { return k + ((64 - (k * 2) % 128 + 128) % 128) / 2; };    // bytes == 64 (mod 128): the 16-byte
    p.xap = pitch(p.hid > p.H * p.D ? p.hid : p.H * p.D);                            // loads of eight rows miss each other's banks
    p.qap = pitch(QW > p.I ? QW : p.I);
    int o = CL_HEADER;
    p.o_h = o; o += round_up(RB * p.hp * 4, 128);
    p.o_xa = o; o += round_up(RB * p.xap * 2, 128);
    p.o_qa = o; o += round_up(RB * p.qap * 2, 128);
    p.o_part = o; o += round_up(rows * p.Hkv * p.P * G * (p.D + 4) * 4, 128);
    p.o_res = o; o += round_up(CL_WARPS * G * (p.D + 2) * 4, 128);
    p.o_ipart = o; o += round_up(G * (p.D + 4) * 4, 128);
    p.o_wst = o; o += CL_WARPS * 1024;
    p.o_cs = o; o += round_up(RB * p.D * 4, 128);
    p.o_pos = o; o += round_up(RB * 4, 128);
    p.o_tab = o; o += round_up(RB * p.max_blocks * 4, 128);
    p.o_snew = o; o += round_up(RB * p.H * 4, 128);
    p.o_red = o; o += 2 * CL_WARPS * (RB / 8) * 128 * 4;
    p.o_nred = o; o += CL_WARPS * 16 * 4;
    p.o_layers = o; o += round_up(p.n_layers * (int)sizeof(ClLayer), 128);
    p.o_ring = o;
    int stage = CL_WARPS * p.ks_target * CL_FRAG;
    if (2 * VM_PAGE_TOKENS * p.D * 2 > stage) stage = 2 * VM_PAGE_TOKENS * p.D * 2;
    if (p.hid * 4 > stage) stage = p.hid * 4;
    p.stage_bytes = round_up(stage, 128);
    int n = (CL_SMEM_LIMIT - o) / p.stage_bytes;
    if (n > CL_MAX_STAGES) n = CL_MAX_STAGES;
    p.n_stages = n;
    if (n < 3) return -1;
    return o + n * p.stage_bytes;
}

bool cluster_sizes_ok(const ClParams& p) {
    if (p.B <= 0 || p.rpc < 1 || p.rpc > 16) return false;
    if (!(p.cs == 1 || p.cs == 2 || p.cs == 4 || p.cs == 8 || p.cs == 16)) return false;
    if (!(p.D == 16 || p.D == 32 || p.D == 64 || p.D == 128)) return false;
    if (p.hid % 32 || (p.H * p.D) % 32 || p.I % 32 || p.H % p.Hkv || p.H / p.Hkv > 16) return false;
    if (!(p.rot == 0 || p.rot == p.D)) return false;
    if (p.ks_target < 1 || p.ks_target > CL_KS_MAX) return false;
    if (p.P < 1) return false;
    return true;
}

template <int D, int NB>
int cluster_launch(const ClParams& p, int smem, cudaStream_t stream) {
    static int configured = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_cluster_kernel<D, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, CL_SMEM_LIMIT);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(decode_cluster_kernel<D, NB>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured = 1;
    }
    const int clusters = (p.B + p.rpc - 1) / p.rpc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * p.cs); cfg.blockDim = dim3(CL_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_cluster_kernel<D, NB>, p);
    if (e != cudaSuccess) return (int)e;
    return vm_launch_status();
}

}  // namespace

VM_API int vm_decode_cluster_layer_bytes() { return (int)sizeof(ClLayer); }

// Ring stages that fit for these sizes (at least 3 means the kernel takes them), or -1.
VM_API int vm_decode_cluster_fit(int rows, int cs, int n_layers, int hid, int H, int Hkv, int D, int I, int max_blocks, int ks_target,
                                 int P) {
    ClParams p{};
    p.B = rows; p.rpc = rows; p.cs = cs; p.n_layers = n_layers; p.hid = hid; p.H = H; p.Hkv = Hkv; p.D = D; p.I = I; p.max_blocks = max_blocks;
    p.ks_target = ks_target; p.P = P; p.rot = 0;
    if (!cluster_sizes_ok(p)) return -1;
    if (cluster_layout(p, rows) < 0) return -1;
    return p.n_stages;
}

// Embedding and every layer of one decode step (one new token per sequence) for B sequences, `rpc` of them per
// cluster of `cs` CTAs; the rows' residual stream goes to h_out [B, hid] (float32) for the final norm and the head.
// `layers`: device array of n_layers ClLayer records.  The weight streams must have been packed for this `cs` and
// this ks_target (engine/cluster.py).  `trace` (optional, [5 * n_layers][CTAs][2] of 64 bits) receives every CTA's arrival at and
// release from each phase barrier in nanoseconds.
VM_API int vm_decode_cluster(const void* layers, int n_layers, int B, int rpc, int cs, int hid, int H, int Hkv, int D, int I,
                             int V, float scale, int window, const float* inv_freq, int rot_dim, const int* tokens,
                             const int* positions, const int* block_table, int max_blocks, int n_pages, const void* embed,
                             int embed_dtype, float* h_out, long long rank_stride, int ks_target, int P,
                             int* err, unsigned long long* trace, cudaStream_t stream) {
    if (B <= 0) return 0;
    ClParams p{};
    p.trace = trace;
    p.layers = static_cast<const ClLayer*>(layers); p.n_layers = n_layers;
    p.B = B; p.rpc = rpc; p.cs = cs; p.hid = hid; p.H = H; p.Hkv = Hkv; p.D = D; p.I = I; p.V = V;
    p.scale_log2 = scale * 1.4426950408889634f; p.window = window; p.inv_freq = inv_freq; p.rot = rot_dim;
    p.tokens = tokens; p.positions = positions; p.table = block_table; p.max_blocks = max_blocks; p.n_pages = n_pages;
    p.embed = embed; p.embed_f32 = (embed_dtype == VM_F32); p.h_out = h_out; p.err = err; p.rank_stride = rank_stride;
    p.ks_target = ks_target; p.P = P;
    if (!cluster_sizes_ok(p) || (rot_dim > 0 && inv_freq == nullptr) || err == nullptr) return VM_ERR_UNSUPPORTED;
    const int smem = cluster_layout(p, rpc);
    if (smem < 0) return VM_ERR_UNSUPPORTED;
    const bool two = rpc > 8;
#define VM_CL_CASE(DD) case DD: return two ? cluster_launch<DD, 2>(p, smem, stream) : cluster_launch<DD, 1>(p, smem, stream);
    switch (D) { VM_CL_CASE(16) VM_CL_CASE(32) VM_CL_CASE(64) VM_CL_CASE(128) }
#undef VM_CL_CASE
    return VM_ERR_UNSUPPORTED;
}
