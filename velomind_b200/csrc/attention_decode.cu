// Decode attention for bfloat16: every sequence of the batch brings ONE new token; its query heads read
// the whole cache of the sequence.  The work is bandwidth- and latency-bound, so the keys of a sequence
// are split over several CTAs (split-KV) and the partial results are merged by the last CTA to finish.
//
// Arithmetic as in attention_generic.cu (reference: examples/common/llama/llama_graph.cpp:97-103 and the
// online form of src/cpu/ops/fused_attention.cpp:84-135); the G = H / Hkv query heads that share a kv
// head (src/cpu/ops/repeat_kv.cpp:51-61) are served by one CTA, so each key and value is read once.
//
// grid = (n_splits, Hkv * ceil(G / 16), B), 128 threads; or, with one split and no more CTAs than SMs, 320 threads
// (ten warps, a cache page each: a sequence of up to 640 tokens is one round, and no partial result leaves the CTA).  A CTA's key range is a whole number of cache
// pages, computed on the device from the sequence's length: the launch shape does not depend on the
// lengths, so the launch can sit in a CUDA graph.  Head sizes 16, 32, ..., 128.  Scratch (global memory beyond inputs and outputs):
// float partials [B, H, n_splits, D + 2] and one int counter per (B, kv-head group), which must be zero
// before the first launch and is left zero by every launch.
#include "attn_decode_body.cuh"

namespace {

constexpr int DEC_WARPS = 4;
constexpr int DEC_WARPS_WIDE = 10;
using namespace vmad;

template <int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                   const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                   int* __restrict__ counters, int H, int Hkv, float scale_log2, int window, int n_pages,
                   int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    attn_decode_body<D, WARPS, true>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, out, partial,
                                         counters, H, Hkv, scale_log2, window, n_pages, err, blockIdx.x, gridDim.x, blockIdx.y,
                                         gridDim.y, blockIdx.z, smem_raw);
}

template <int D, int WARPS>
int launch_decode(dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, int q_row_stride, const __nv_bfloat16* kpages,
                  const __nv_bfloat16* vpages, const int* block_table, int max_blocks, const int* positions,
                  __nv_bfloat16* out, float* partial, int* counters, int H, int Hkv, float scale, int window, int n_pages,
                  int* err) {
    const size_t smem = attn_decode_smem_bytes<D, WARPS>();
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    vm_launch_pdl(attn_decode_kernel<D, WARPS>, grid, dim3(WARPS * 32), smem, stream, q, q_row_stride, kpages, vpages, block_table,
                  max_blocks, positions, out, partial, counters, H, Hkv, scale * 1.4426950408889634f, window, n_pages, err);
    return vm_launch_status();
}

}  // namespace

// Bytes of float scratch the kernel needs for a batch of B sequences.
VM_API long long vm_attention_decode_scratch_floats(int B, int H, int D, int n_splits) {
    return (long long)B * H * n_splits * (D + 2);
}

// q: [B, H, D] rows with stride q_row_stride; out: [B, H*D].  counters: at least B * Hkv * ceil(G/16) ints, zero.
VM_API int vm_attention_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                    const int* block_table, int max_blocks, const int* positions, void* out,
                                    float* partial, int* counters, int B, int H, int Hkv, int D, int n_splits,
                                    float scale, int window, int n_pages, int* err, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || n_splits < 1 || n_splits > MAX_SPLITS || (q_row_stride % 8) != 0)
        return VM_ERR_UNSUPPORTED;
    const int G = H / Hkv;
    dim3 grid(n_splits, Hkv * ((G + DEC_ROWS - 1) / DEC_ROWS), B);
    const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)kpages, *vv = (const __nv_bfloat16*)vpages;
    // one split and a CTA per SM at most: ten warps per CTA, if their pages fit into shared memory
    const bool wide = n_splits == 1 && (long long)grid.y * grid.z <= vm_sm_count();
#define VM_DEC_CASE(DD)                                                                                                \
    case DD:                                                                                                           \
        if (wide && attn_decode_smem_bytes<DD, DEC_WARPS_WIDE>() <= 227 * 1024)                                        \
            return launch_decode<DD, DEC_WARPS_WIDE>(grid, stream, qq, q_row_stride, kk, vv, block_table, max_blocks,  \
                                                     positions, (__nv_bfloat16*)out, partial, counters, H, Hkv, scale, \
                                                     window, n_pages, err);                                            \
        return launch_decode<DD, DEC_WARPS>(grid, stream, qq, q_row_stride, kk, vv, block_table, max_blocks, positions, \
                                            (__nv_bfloat16*)out, partial, counters, H, Hkv, scale, window, n_pages, err);
    switch (D) {
        VM_DEC_CASE(16) VM_DEC_CASE(32) VM_DEC_CASE(48) VM_DEC_CASE(64)
        VM_DEC_CASE(80) VM_DEC_CASE(96) VM_DEC_CASE(112) VM_DEC_CASE(128)
        default: return VM_ERR_UNSUPPORTED;
    }
#undef VM_DEC_CASE
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

namespace {
// The array's address on the current device: looked up once per device, with that device current.  (No lock: two host
// threads that both make a device's first call look the same address up and store the same value.)
int no_alloc_address(unsigned char** base) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NO_ALLOC_MAX_DEVICES) return VM_ERR_UNSUPPORTED;
    if (no_alloc_base[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, vm_no_alloc_scratch);
        if (e != cudaSuccess) return (int)e;
        no_alloc_base[dev] = static_cast<unsigned char*>(p);
    }
    *base = no_alloc_base[dev];
    return 0;
}
}  // namespace

VM_API void* vm_attention_decode_no_alloc_scratch(void) {
    unsigned char* base = nullptr;
    return no_alloc_address(&base) == 0 ? base : nullptr;
}

VM_API int vm_attention_decode_bf16_no_alloc(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                             const int* block_table, int max_blocks, const int* positions, void* out,
                                             int B, int H, int Hkv, int D, int n_splits, float scale, int window,
                                             int n_pages, int* err, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || D <= 0 || n_splits < 1) return VM_ERR_BAD_ARG;
    // everything the kernel's own launcher would refuse is refused here, before anything is put on the stream
    if (Hkv <= 0 || H % Hkv != 0 || n_splits > MAX_SPLITS || (q_row_stride % 8) != 0 || D % 16 != 0 || D > 128)
        return VM_ERR_UNSUPPORTED;
    if (vm_attention_decode_no_alloc_bytes(B, H, D, n_splits) > VM_NO_ALLOC_SCRATCH_BYTES) return VM_NO_ALLOC_TOO_LARGE;
    unsigned char* base = nullptr;
    const int looked_up = no_alloc_address(&base);
    if (looked_up != 0) return looked_up;
    int* counters = reinterpret_cast<int*>(base);
    float* partial = reinterpret_cast<float*>(base + no_alloc_counter_bytes(B, H));
    // the array keeps the last call's contents: the counters must start at zero
    const cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)no_alloc_counter_bytes(B, H), stream);
    if (e != cudaSuccess) return (int)e;
    return vm_attention_decode_bf16(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, out, partial,
                                    counters, B, H, Hkv, D, n_splits, scale, window, n_pages, err, stream);
}
