// Decode attention for bfloat16: every sequence of the batch brings ONE new token; its query heads read
// the whole cache of the sequence.  The work is bandwidth- and latency-bound, so the keys of a sequence
// are split over several CTAs (split-KV) and the partial results are merged by the last CTA to finish.
//
// Arithmetic as in attention_generic.cu (reference: examples/common/llama/llama_graph.cpp:97-103 and the
// online form of src/cpu/ops/fused_attention.cpp:84-135); the G = H / Hkv query heads that share a kv
// head (src/cpu/ops/repeat_kv.cpp:51-61) are served by one CTA, so each key and value is read once.
//
// grid = (n_splits, Hkv * ceil(G / GM), B), 128 threads.  A CTA's key range is a whole number of cache
// pages, computed on the device from the sequence's length: the launch shape does not depend on the
// lengths, so the launch can sit in a CUDA graph.  Scratch (global memory beyond inputs and outputs):
// float partials [B, H, n_splits, D + 2] and one int counter per (B, kv-head group), which must be zero
// before the first launch and is left zero by every launch.
#include "common.cuh"

namespace {

constexpr int DEC_WARPS = 4;

__device__ __forceinline__ void dec_cp_async16(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem));
}

// One CTA iteration covers UNIT_PAGES cache pages (128 keys): all of their keys and values are fetched
// into shared memory at once (every thread has several 16-byte copies in flight), then each warp works
// on its own 32 keys.
constexpr int UNIT_PAGES = 2;
constexpr int UNIT_KEYS = UNIT_PAGES * VM_PAGE_TOKENS;
static_assert(UNIT_KEYS == DEC_WARPS * 32, "one 32-key chunk per warp");

template <int GM, int EPL>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                   const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                   int* __restrict__ counters, int H, int Hkv, int D, float scale, int window, int n_pages,
                   int* __restrict__ err) {
    // shared: q [GM][D] float | per-warp results [DEC_WARPS][GM][D+2] float | K [128][D+8] bf16 | V [128][D+8] bf16
    extern __shared__ __align__(16) float sm[];
    const int split = blockIdx.x, n_splits = gridDim.x;
    const int G = H / Hkv;
    const int groups_per_kv = (G + GM - 1) / GM;
    const int hk = blockIdx.y / groups_per_kv, gg = blockIdx.y - hk * groups_per_kv;
    const int b = blockIdx.z;
    const int h0 = hk * G + gg * GM;                       // first query head of this CTA
    const int ng = min(GM, G - gg * GM);                   // query heads of this CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[b];                          // one token per sequence: token index == sequence index
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_page = lo / VM_PAGE_TOKENS, last_page = pos / VM_PAGE_TOKENS;
    const int units = (last_page - first_page) / UNIT_PAGES + 1;
    const int per_split = (units + n_splits - 1) / n_splits;
    const int unit_a = split * per_split, unit_b = min(units, unit_a + per_split);
    const int DP = D + 8;                                  // padded row: an odd number of 16-byte units
    float* qs = sm;
    float* res = sm + GM * D;
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(res + DEC_WARPS * GM * (D + 2));
    __nv_bfloat16* sV = sK + UNIT_KEYS * DP;
    for (int i = threadIdx.x; i < ng * D; i += blockDim.x) {
        const int g = i / D, d = i - g * D;
        qs[g * D + d] = __bfloat162float(q[(size_t)b * q_row_stride + (size_t)(h0 + g) * D + d]) * scale;
    }

    float m[GM], l[GM], acc[GM][EPL];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[g][i] = 0.f;
    }
    const size_t page_stride = (size_t)Hkv * VM_PAGE_TOKENS * D;
    const int* table = block_table + (size_t)b * max_blocks;
    const int CH = D / 8;                                  // 16-byte chunks per row
    for (int unit = unit_a; unit < unit_b; ++unit) {
        const int blk0 = first_page + unit * UNIT_PAGES;
        __syncthreads();                                   // the previous unit's tiles (and qs, the first time) are settled
        for (int pg = 0; pg < UNIT_PAGES; ++pg) {
            const int blk = blk0 + pg;
            if (blk > last_page) break;
            const int page = (blk < max_blocks) ? table[blk] : -1;
            if (page < 0 || page >= n_pages) { if (threadIdx.x == 0 && err) atomicExch(err, 3); continue; }
            const __nv_bfloat16* kg = kpages + (size_t)page * page_stride + (size_t)hk * VM_PAGE_TOKENS * D;
            const __nv_bfloat16* vg = vpages + (size_t)page * page_stride + (size_t)hk * VM_PAGE_TOKENS * D;
            for (int c = threadIdx.x; c < VM_PAGE_TOKENS * CH; c += blockDim.x) {
                const int r = c / CH, ch = c - r * CH;
                dec_cp_async16(sK + (size_t)(pg * VM_PAGE_TOKENS + r) * DP + ch * 8, kg + (size_t)r * D + ch * 8);
                dec_cp_async16(sV + (size_t)(pg * VM_PAGE_TOKENS + r) * DP + ch * 8, vg + (size_t)r * D + ch * 8);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();
        const int base = blk0 * VM_PAGE_TOKENS + warp * 32;
        if (base > pos || base + 31 < lo) continue;         // warp-uniform: none of this warp's keys is visible
        {
            const int blk = base / VM_PAGE_TOKENS;
            const int page = (blk < max_blocks) ? table[blk] : -1;
            if (page < 0 || page >= n_pages) continue;      // reported above; its tile was not loaded
        }
        const int j = base + lane;
        const bool valid = (j >= lo && j <= pos);
        float s[GM];
#pragma unroll
        for (int g = 0; g < GM; ++g) s[g] = 0.f;
        if (valid) {
            const uint4* krow = reinterpret_cast<const uint4*>(sK + (size_t)(warp * 32 + lane) * DP);
            for (int ch = 0; ch < CH; ++ch) {
                const uint4 kv = krow[ch];
                const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 kf = __bfloat1622float2(k2[e]);
#pragma unroll
                    for (int g = 0; g < GM; ++g) {
                        if (g < ng) {
                            s[g] = fmaf(qs[g * D + ch * 8 + 2 * e], kf.x, s[g]);
                            s[g] = fmaf(qs[g * D + ch * 8 + 2 * e + 1], kf.y, s[g]);
                        }
                    }
                }
            }
        }
        float p[GM];
#pragma unroll
        for (int g = 0; g < GM; ++g) {
            const float sv = valid ? s[g] : -INFINITY;
            const float mn = fmaxf(m[g], vm_warp_max(sv));           // the chunk holds at least one visible key
            p[g] = valid ? expf(sv - mn) : 0.f;
            const float alpha = expf(m[g] - mn);
            l[g] = l[g] * alpha + vm_warp_sum(p[g]);
#pragma unroll
            for (int i = 0; i < EPL; ++i) acc[g][i] *= alpha;
            m[g] = mn;
        }
        const int cnt = min(32, pos - base + 1);
        const int first = max(0, lo - base);
        for (int jj = first; jj < cnt; ++jj) {
            const __nv_bfloat16* vrow = sV + (size_t)(warp * 32 + jj) * DP;
            float vv[EPL];
#pragma unroll
            for (int i = 0; i < EPL; ++i) { const int d = lane + 32 * i; vv[i] = (d < D) ? __bfloat162float(vrow[d]) : 0.f; }
#pragma unroll
            for (int g = 0; g < GM; ++g) {
                const float pj = __shfl_sync(0xffffffffu, p[g], jj);
#pragma unroll
                for (int i = 0; i < EPL; ++i) acc[g][i] = fmaf(pj, vv[i], acc[g][i]);
            }
        }
    }
    __syncthreads();
    // ---- join the CTA's warps
    const int RW = D + 2;
#pragma unroll
    for (int g = 0; g < GM; ++g) {
        if (g < ng) {
            float* r = res + ((size_t)warp * GM + g) * RW;
#pragma unroll
            for (int i = 0; i < EPL; ++i) { const int d = lane + 32 * i; if (d < D) r[d] = acc[g][i]; }
            if (lane == 0) { r[D] = m[g]; r[D + 1] = l[g]; }
        }
    }
    __syncthreads();
    // partial[b, h, split, :] = (o[D], m, l), merged over the warps
    for (int i = threadIdx.x; i < ng * D; i += blockDim.x) {
        const int g = i / D, d = i - g * D;
        float M = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, res[((size_t)w * GM + g) * RW + D]);
        float o = 0.f, L = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* r = res + ((size_t)w * GM + g) * RW;
            const float f = (r[D] == -INFINITY) ? 0.f : expf(r[D] - M);
            o += f * r[d]; L += f * r[D + 1];
        }
        float* dst = partial + (((size_t)b * H + (h0 + g)) * n_splits + split) * RW;
        dst[d] = o;
        if (d == 0) { dst[D] = M; dst[D + 1] = L; }
    }
    // ---- the last CTA of this (sequence, head group) merges the splits
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int old = atomicAdd(&counters[(size_t)b * gridDim.y + blockIdx.y], 1);
        is_last = (old == n_splits - 1);
        if (is_last) counters[(size_t)b * gridDim.y + blockIdx.y] = 0;     // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < ng * D; i += blockDim.x) {
        const int g = i / D, d = i - g * D;
        const float* src = partial + ((size_t)b * H + (h0 + g)) * n_splits * RW;
        float M = -INFINITY;
        for (int s2 = 0; s2 < n_splits; ++s2) M = fmaxf(M, __ldcg(src + (size_t)s2 * RW + D));
        float o = 0.f, L = 0.f;
        for (int s2 = 0; s2 < n_splits; ++s2) {
            const float ms = __ldcg(src + (size_t)s2 * RW + D);
            const float f = (ms == -INFINITY) ? 0.f : expf(ms - M);
            o += f * __ldcg(src + (size_t)s2 * RW + d);
            L += f * __ldcg(src + (size_t)s2 * RW + D + 1);
        }
        out[((size_t)b * H + (h0 + g)) * D + d] = __float2bfloat16_rn(o / L);
    }
}

template <int GM>
int launch_decode(int epl, dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16* q, int q_row_stride,
                  const __nv_bfloat16* kpages, const __nv_bfloat16* vpages, const int* block_table, int max_blocks,
                  const int* positions, __nv_bfloat16* out, float* partial, int* counters, int H, int Hkv, int D,
                  float scale, int window, int n_pages, int* err) {
#define VM_DEC_CASE(E)                                                                                               \
    case E:                                                                                                          \
        if (smem > 48 * 1024) {                                                                                      \
            static bool configured = false;                                                                          \
            if (!configured) {                                                                                       \
                cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<GM, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
                if (e != cudaSuccess) return (int)e;                                                                 \
                configured = true;                                                                                   \
            }                                                                                                        \
        }                                                                                                            \
        attn_decode_kernel<GM, E><<<grid, DEC_WARPS * 32, smem, stream>>>(q, q_row_stride, kpages, vpages, block_table, \
            max_blocks, positions, out, partial, counters, H, Hkv, D, scale, window, n_pages, err);                   \
        break;
    switch (epl) {
        VM_DEC_CASE(1) VM_DEC_CASE(2) VM_DEC_CASE(3) VM_DEC_CASE(4)
        default: return VM_ERR_UNSUPPORTED;
    }
#undef VM_DEC_CASE
    return vm_launch_status();
}

}  // namespace

// Bytes of float scratch the kernel needs for a batch of B sequences.
VM_API long long vm_attention_decode_scratch_floats(int B, int H, int D, int n_splits) {
    return (long long)B * H * n_splits * (D + 2);
}

// q: [B, H, D] rows with stride q_row_stride; out: [B, H*D].  counters: at least B * Hkv * ceil(G/GM) ints, zero.
VM_API int vm_attention_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                    const int* block_table, int max_blocks, const int* positions, void* out,
                                    float* partial, int* counters, int B, int H, int Hkv, int D, int n_splits,
                                    float scale, int window, int n_pages, int* err, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || D % 8 != 0 || D > 128 || n_splits < 1 || (q_row_stride % 8) != 0)
        return VM_ERR_UNSUPPORTED;
    const int G = H / Hkv;
    const int GM = G <= 1 ? 1 : (G <= 2 ? 2 : (G <= 4 ? 4 : 8));
    const int groups = (G + GM - 1) / GM;
    dim3 grid(n_splits, Hkv * groups, B);
    const size_t smem = ((size_t)GM * D + (size_t)DEC_WARPS * GM * (D + 2)) * sizeof(float)
                        + 2 * (size_t)UNIT_KEYS * (D + 8) * sizeof(__nv_bfloat16);
    const int epl = (D + 31) / 32;
    const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)kpages, *vv = (const __nv_bfloat16*)vpages;
    switch (GM) {
        case 1: return launch_decode<1>(epl, grid, smem, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, (__nv_bfloat16*)out, partial, counters, H, Hkv, D, scale, window, n_pages, err);
        case 2: return launch_decode<2>(epl, grid, smem, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, (__nv_bfloat16*)out, partial, counters, H, Hkv, D, scale, window, n_pages, err);
        case 4: return launch_decode<4>(epl, grid, smem, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, (__nv_bfloat16*)out, partial, counters, H, Hkv, D, scale, window, n_pages, err);
        default: return launch_decode<8>(epl, grid, smem, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, (__nv_bfloat16*)out, partial, counters, H, Hkv, D, scale, window, n_pages, err);
    }
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (declared and explained in velomind_no_alloc.h).
#include "velomind_no_alloc.h"

namespace {

// The scratch of the no-alloc entry point.  In HOST code this name is only a handle for the symbol: it is
// not a device address and must never be passed to a kernel; the address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char vm_no_alloc_scratch[VM_NO_ALLOC_SCRATCH_BYTES];

constexpr int NO_ALLOC_MAX_DEVICES = 64;
unsigned char* no_alloc_base[NO_ALLOC_MAX_DEVICES] = {};     // per device, looked up on the first call there

long long no_alloc_counter_bytes(int B, int H) { return (((long long)B * H * 4) + 255) / 256 * 256; }

}  // namespace

VM_API long long vm_attention_decode_no_alloc_bytes(int B, int H, int D, int n_splits) {
    return no_alloc_counter_bytes(B, H) + 4ll * B * H * n_splits * (D + 2);
}

VM_API int vm_attention_decode_bf16_no_alloc(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                             const int* block_table, int max_blocks, const int* positions, void* out,
                                             int B, int H, int Hkv, int D, int n_splits, float scale, int window,
                                             int n_pages, int* err, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || D <= 0 || n_splits < 1) return VM_ERR_BAD_ARG;
    if (vm_attention_decode_no_alloc_bytes(B, H, D, n_splits) > VM_NO_ALLOC_SCRATCH_BYTES) return VM_NO_ALLOC_TOO_LARGE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NO_ALLOC_MAX_DEVICES) return VM_ERR_UNSUPPORTED;
    if (no_alloc_base[dev] == nullptr) {
        // once per device, with that device current: the symbol's address ON THIS DEVICE
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, vm_no_alloc_scratch);
        if (e != cudaSuccess) return (int)e;
        no_alloc_base[dev] = static_cast<unsigned char*>(p);
    }
    unsigned char* base = no_alloc_base[dev];
    int* counters = reinterpret_cast<int*>(base);
    float* partial = reinterpret_cast<float*>(base + no_alloc_counter_bytes(B, H));
    // the array keeps the last call's contents: the counters must start at zero
    e = cudaMemsetAsync(counters, 0, (size_t)no_alloc_counter_bytes(B, H), stream);
    if (e != cudaSuccess) return (int)e;
    return vm_attention_decode_bf16(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, out, partial,
                                    counters, B, H, Hkv, D, n_splits, scale, window, n_pages, err, stream);
}
