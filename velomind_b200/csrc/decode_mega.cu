// One decode step in ONE persistent kernel (bfloat16, at most 16 sequences, one new token each).
//
// A decode step of a small model is a chain of tiny dependent kernels: per layer norm + qkv + rotary + cache
// write, attention, out + residual, norm + gate/up + SwiGLU, down + residual; each costs a launch gap and its own
// chain of memory latencies, far more than the bytes it streams.  Here one CTA per SM stays resident for the
// whole step and walks through the same phases, separated by grid-wide barriers; a phase's work items (the CTAs of
// the stand-alone kernels) are dealt out round-robin.  The phases are the device bodies of skinny_gemm.cu and
// attention_decode.cu, so the arithmetic is that of the stand-alone kernels.
//
// Data that one SM writes and another reads in a later phase goes through L2 (cp.async.cg / ld.global.cg), since
// L1 is not coherent between SMs within a kernel.
//
// The grid barrier is a counter in global memory: arrive with a release, poll with an acquire.  The kernel is
// launched cooperatively (all CTAs resident) and every poll loop is bounded; when a wait gives up the CTA raises
// error word 5 and all later barriers fall through, so the kernel always ends.
#include "skinny_body.cuh"
#include "attn_decode_body.cuh"

namespace {

using namespace vmsk;
using namespace vmad;

constexpr int MEGA_WARPS = SK_WARPS;             // 8 warps = 256 threads, as the weight-streaming bodies expect
constexpr int MEGA_THREADS = MEGA_WARPS * 32;
constexpr unsigned MEGA_POLL_LIMIT = 1u << 22;

struct MegaLayer {
    const __nv_bfloat16* wqkv; const __nv_bfloat16* wo; const __nv_bfloat16* wgu; const __nv_bfloat16* wd;
    const float* norm1; const float* norm2;
    __nv_bfloat16* kpages; __nv_bfloat16* vpages;
    float eps1, eps2;
};

struct MegaParams {
    const MegaLayer* layers; int n_layers;
    int B, hid, H, Hkv, D, I, V;
    float scale; int window; const float* inv_freq; int rot_dim;
    const int* tokens; const int* positions; const int* seq_of_token; const int* block_table; int max_blocks, n_pages;
    const void* embed; int embed_dtype;
    float* h; __nv_bfloat16* q; __nv_bfloat16* att; __nv_bfloat16* act; __nv_bfloat16* xf; float* logits;
    const float* final_norm; float final_eps; const __nv_bfloat16* head;
    float* partial; int* counters; int n_splits;
    unsigned* barrier; int* err;
    unsigned long long* trace; int trace_phases;   // optional: per phase and CTA, the time of arrival at and departure from the barrier
};

// Ask L2 for rows [row0, row0 + rows) of a K-wide bf16 matrix (what this CTA will stream in a later phase), so that the
// loads after the next barrier find them there instead of in DRAM.
__device__ __forceinline__ void prefetch_rows_l2(const __nv_bfloat16* W, int K, int row0, int rows) {
    const char* base = reinterpret_cast<const char*>(W + (size_t)row0 * K);
    const int lines = (rows * K * 2 + 127) / 128;
    for (int i = threadIdx.x; i < lines; i += blockDim.x)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (size_t)i * 128));
}

// the weight rows of this CTA's items of a plain or paired product: item `it` covers rows rowA(it).. and rowB(it)..
__device__ __forceinline__ void prefetch_items(const __nv_bfloat16* W, int K, int items, int rows_per_item, int second_offset) {
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        prefetch_rows_l2(W, K, it * rows_per_item, rows_per_item);
        if (second_offset > 0) prefetch_rows_l2(W, K, second_offset + it * rows_per_item, rows_per_item);
    }
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs arrive; nobody passes before all have.  `target` counts arrivals so far (the counter is zero at launch).
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void grid_barrier(const MegaParams& p, unsigned& target) {
    const unsigned phase = target / gridDim.x;
    target += gridDim.x;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (p.trace && (int)phase < p.trace_phases) p.trace[((size_t)phase * gridDim.x + blockIdx.x) * 2] = global_ns();
        __threadfence();
        atomicAdd(p.barrier, 1u);
        if (*reinterpret_cast<volatile int*>(p.err) != 5) {
            unsigned polls = 0;
            while (ld_acquire(p.barrier) < target) {
                if (++polls > MEGA_POLL_LIMIT) { atomicExch(p.err, 5); break; }
            }
        }
        __threadfence();
        if (p.trace && (int)phase < p.trace_phases) p.trace[((size_t)phase * gridDim.x + blockIdx.x) * 2 + 1] = global_ns();
    }
    __syncthreads();
}

// The parameter block of a phase lives in shared memory and is written by one thread: 256 threads building it on their
// own stacks cost more local-memory traffic than the phase's weights.
__device__ __forceinline__ void skinny_base(SkinnyParams& s, const MegaParams& p, int K) {
    s = SkinnyParams{};
    s.M = p.B; s.K = K;
    s.kc = skinny_chunk(K, 16);
    s.row_bytes = skinny_pitch(s.kc);
    s.err = p.err;
}

// Each phase is a function of its own (not inlined), so that the register allocation of one phase does not have to
// make room for the others.
__device__ __noinline__ void phase_skinny(const SkinnyParams& s, int items, unsigned char* smem) {
    for (int it = blockIdx.x; it < items; it += gridDim.x) skinny_body<1, false>(s, it, smem);
}
__device__ __noinline__ void phase_head(const SkinnyParams& s, int items, unsigned char* smem) {
    for (int it = blockIdx.x; it < items; it += gridDim.x) skinny_wide_body<1, false>(s, it, smem);
}
template <int D>
__device__ __noinline__ void phase_attention(const MegaParams& p, const MegaLayer& L, int groups, unsigned char* smem) {
    const int items = p.n_splits * groups * p.B;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int split = it % p.n_splits, rest = it / p.n_splits;
        const int gy = rest % groups, b = rest / groups;
        attn_decode_body<D, MEGA_WARPS, false>(p.q, p.H * p.D, L.kpages, L.vpages, p.block_table, p.max_blocks, p.positions,
                                               p.att, p.partial, p.counters, p.H, p.Hkv, p.scale * 1.4426950408889634f,
                                               p.window, p.n_pages, p.err, split, p.n_splits, gy, groups, b, smem);
    }
}

template <int D>
__global__ void __launch_bounds__(MEGA_THREADS)
decode_mega_kernel(const MegaParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ SkinnyParams s;
    unsigned target = 0;
    const int tid = threadIdx.x;

    // ---- phase 0: embedding rows into the float32 residual stream
    for (int b = blockIdx.x; b < p.B; b += gridDim.x) {
        const int id = p.tokens[b];
        const bool ok = id >= 0 && id < p.V;
        if (!ok && tid == 0) atomicExch(p.err, 1);
        for (int i = tid; i < p.hid; i += MEGA_THREADS) {
            float v = 0.f;
            if (ok) v = (p.embed_dtype == VM_F32) ? static_cast<const float*>(p.embed)[(size_t)id * p.hid + i]
                                                  : __bfloat162float(static_cast<const __nv_bfloat16*>(p.embed)[(size_t)id * p.hid + i]);
            p.h[(size_t)b * p.hid + i] = v;
        }
    }
    grid_barrier(p, target);

    const int G = p.H / p.Hkv;
    const int groups = p.Hkv * ((G + DEC_ROWS - 1) / DEC_ROWS);
    for (int l = 0; l < p.n_layers; ++l) {
        const MegaLayer L = p.layers[l];
        // ---- norm + qkv + rotary + cache write
        {
            if (tid == 0) {
            skinny_base(s, p, p.hid);
            s.A = p.h; s.pro = PRO_RMSNORM; s.norm_w = L.norm1; s.eps = L.eps1; s.W = L.wqkv; s.N = (p.H + 2 * p.Hkv) * p.D;
            s.out = p.q; s.out_stride = p.H * p.D; s.epi = EPI_ROPE_KV; s.tiles = 2;
            s.positions = p.positions; s.seq_of_token = p.seq_of_token; s.block_table = p.block_table; s.max_blocks = p.max_blocks;
            s.inv_freq = p.inv_freq; s.rot_dim = p.rot_dim; s.kpages = L.kpages; s.vpages = L.vpages;
            s.H = p.H; s.Hkv = p.Hkv; s.D = p.D; s.n_pages = p.n_pages;
            }
            __syncthreads();
            prefetch_items(L.wo, p.H * p.D, p.hid / 8, 8, 0);                 // the next phases' weights, into L2 meanwhile
            phase_skinny(s, (p.H + 2 * p.Hkv) * (p.D / 16), smem);
        }
        grid_barrier(p, target);
        // ---- attention over the cache (split over the keys; the last CTA of a head group merges)
        prefetch_items(L.wgu, p.hid, p.I / 8, 8, p.I);
        phase_attention<D>(p, L, groups, smem);
        grid_barrier(p, target);
        // ---- out projection + residual
        {
            if (tid == 0) {
            skinny_base(s, p, p.H * p.D);
            s.A = p.att; s.pro = PRO_NONE; s.W = L.wo; s.N = p.hid; s.h = p.h; s.epi = EPI_RESIDUAL; s.tiles = 1;
            }
            __syncthreads();
            prefetch_items(L.wd, p.I, p.hid / 8, 8, 0);
            phase_skinny(s, p.hid / 8, smem);
        }
        grid_barrier(p, target);
        // ---- norm + gate/up + SwiGLU
        {
            if (tid == 0) {
            skinny_base(s, p, p.hid);
            s.A = p.h; s.pro = PRO_RMSNORM; s.norm_w = L.norm2; s.eps = L.eps2; s.W = L.wgu; s.N = 2 * p.I;
            s.out = p.act; s.out_stride = p.I; s.I = p.I; s.epi = EPI_SWIGLU; s.tiles = 2;
            }
            __syncthreads();
            if (l + 1 < p.n_layers) {                                          // next layer's qkv rows, an equal share per CTA
                const int rows_total = (p.H + 2 * p.Hkv) * p.D;
                const int share = (rows_total + gridDim.x - 1) / gridDim.x;
                const int r0 = blockIdx.x * share;
                if (r0 < rows_total) prefetch_rows_l2(p.layers[l + 1].wqkv, p.hid, r0, min(share, rows_total - r0));
            }
            phase_skinny(s, p.I / 8, smem);
        }
        grid_barrier(p, target);
        // ---- down projection + residual
        {
            if (tid == 0) {
            skinny_base(s, p, p.I);
            s.A = p.act; s.pro = PRO_NONE; s.W = L.wd; s.N = p.hid; s.h = p.h; s.epi = EPI_RESIDUAL; s.tiles = 1;
            }
            __syncthreads();
            phase_skinny(s, p.hid / 8, smem);
        }
        grid_barrier(p, target);
    }
    // ---- final norm of every row (one warp per row), as bf16 for the head
    {
        const int warp = tid >> 5, lane = tid & 31;
        for (int r = blockIdx.x * MEGA_WARPS + warp; r < p.B; r += gridDim.x * MEGA_WARPS) {
            const float* row = p.h + (size_t)r * p.hid;
            float ss = 0.f;
            for (int i0 = lane; i0 < p.hid; i0 += 32 * 8) {              // eight loads in flight per lane
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) { const int i = i0 + 32 * u; v[u] = (i < p.hid) ? __ldcg(row + i) : 0.f; }
#pragma unroll
                for (int u = 0; u < 8; ++u) ss += v[u] * v[u];
            }
            ss = vm_warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)p.hid + p.final_eps);
            for (int i0 = lane; i0 < p.hid; i0 += 32 * 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) { const int i = i0 + 32 * u; v[u] = (i < p.hid) ? __ldcg(row + i) : 0.f; }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + 32 * u;
                    if (i < p.hid) p.xf[(size_t)r * p.hid + i] = __float2bfloat16_rn(v[u] * inv * p.final_norm[i]);
                }
            }
        }
    }
    grid_barrier(p, target);
    // ---- head: float32 logits
    {
        if (tid == 0) {
        skinny_base(s, p, p.hid);
        s.A = p.xf; s.pro = PRO_NONE; s.W = p.head; s.N = p.V; s.out = p.logits; s.out_stride = p.V; s.epi = EPI_STORE_F32;
        s.row_bytes = skinny_pitch(p.hid);
        }
        __syncthreads();
        phase_head(s, (p.V / 8 + SK_WARPS - 1) / SK_WARPS, smem);
    }
}

template <int D>
int mega_launch(const MegaParams& p, cudaStream_t stream) {
    size_t smem = attn_decode_smem_bytes<D, MEGA_WARPS>();
    const size_t sk = skinny_smem_bytes(p.hid > p.I ? p.hid : p.I, 16);
    if (sk > smem) smem = sk;
    const size_t sk2 = skinny_smem_bytes(p.H * p.D, 16);
    if (sk2 > smem) smem = sk2;
    if (smem > 220 * 1024) return VM_ERR_UNSUPPORTED;
    static bool configured = false;
    static int grid = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, sms = 0, occ = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, decode_mega_kernel<D>, MEGA_THREADS, smem);
        if (e != cudaSuccess || occ < 1) return VM_ERR_UNSUPPORTED;
        grid = sms;                                   // one CTA per SM; all of them resident (cooperative launch)
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(MEGA_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_mega_kernel<D>, p);
    if (e != cudaSuccess) return (int)e;
    return vm_launch_status();
}

}  // namespace

// sizeof(MegaLayer) for the host to lay the per-layer table out
VM_API int vm_decode_mega_layer_bytes() { return (int)sizeof(MegaLayer); }

// One decode step for B <= 16 sequences.  `layers`: device array of n_layers records {wqkv, wo, wgu, wd, norm1, norm2,
// kpages, vpages (pointers), eps1, eps2 (floats)}.  `barrier` must be zero at launch; `counters` zero (left zero).
VM_API int vm_decode_mega(const void* layers, int n_layers, int B, int hid, int H, int Hkv, int D, int I, int V, float scale,
                          int window, const float* inv_freq, int rot_dim, const int* tokens, const int* positions,
                          const int* seq_of_token, const int* block_table, int max_blocks, int n_pages, const void* embed,
                          int embed_dtype, float* h, void* q, void* att, void* act, void* xf, float* logits,
                          const float* final_norm, float final_eps, const void* head, float* partial, int* counters,
                          int n_splits, unsigned* barrier, int* err, unsigned long long* trace, int trace_phases,
                          cudaStream_t stream) {
    if (B <= 0) return 0;
    if (B > 16 || hid % 32 || I % 32 || (H * D) % 32 || D % 16 || hid % 8 || I % 8 || V % 8 || H % Hkv ||
        !(rot_dim == 0 || rot_dim == D) || n_splits < 1 || n_splits > MAX_SPLITS)
        return VM_ERR_UNSUPPORTED;
    MegaParams p{};
    p.layers = static_cast<const MegaLayer*>(layers); p.n_layers = n_layers;
    p.B = B; p.hid = hid; p.H = H; p.Hkv = Hkv; p.D = D; p.I = I; p.V = V; p.scale = scale; p.window = window;
    p.inv_freq = inv_freq; p.rot_dim = rot_dim; p.tokens = tokens; p.positions = positions; p.seq_of_token = seq_of_token;
    p.block_table = block_table; p.max_blocks = max_blocks; p.n_pages = n_pages; p.embed = embed; p.embed_dtype = embed_dtype;
    p.h = h; p.q = (__nv_bfloat16*)q; p.att = (__nv_bfloat16*)att; p.act = (__nv_bfloat16*)act; p.xf = (__nv_bfloat16*)xf;
    p.logits = logits; p.final_norm = final_norm; p.final_eps = final_eps; p.head = (const __nv_bfloat16*)head;
    p.partial = partial; p.counters = counters; p.n_splits = n_splits; p.barrier = barrier; p.err = err; p.trace = trace; p.trace_phases = trace_phases;
    switch (D) {
        case 16: return mega_launch<16>(p, stream);
        case 32: return mega_launch<32>(p, stream);
        case 48: return mega_launch<48>(p, stream);
        case 64: return mega_launch<64>(p, stream);
        default: return VM_ERR_UNSUPPORTED;
    }
}
