// Shared device helpers for the velomind_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// The launchers' declarations, dtype and status codes, the page size and the rotary pairings: one header shared
// with the host library, so that a launcher's definition here is checked against what its callers see.
#include "../include/velomind_b200/kernels.h"

#define VM_API extern "C" __attribute__((visibility("default")))

__device__ __forceinline__ float vm_to_float(float x) { return x; }
__device__ __forceinline__ float vm_to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T vm_from_float(float x);
template <> __device__ __forceinline__ float vm_from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 vm_from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float vm_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float vm_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `red` is a __shared__ float[32]. Every thread gets the result.
__device__ __forceinline__ float vm_block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = vm_warp_sum(v);
    __syncthreads();                 // protect `red` against the previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (lane < nw) ? red[lane] : 0.f;
    return vm_warp_sum(t);
}

// ---- programmatic dependent launch: a kernel launched through vm_launch_pdl may begin (and fetch data that
// no earlier kernel writes, i.e. weights) while its predecessor in the stream is still running; it must call
// vm_pdl_wait() before it reads anything an earlier kernel wrote and before its first global write.
// vm_pdl_launch_dependents() lets the successor start its own preamble.  Without the launch attribute both
// are no-ops.
// One kernel reads more than constants in its preamble: the decode attention fetches positions, the block table
// and the cache rows of EARLIER tokens there.  The rule that makes this sound: the kernel launched directly
// before it (the one that writes the new token's key and value) calls vm_pdl_launch_dependents() only AFTER its
// own vm_pdl_wait(), so when the attention's preamble runs, everything older than that kernel is complete and
// visible; what that kernel itself writes (the new row, the queries) is read after the attention's wait.
// Kernels launched without the attribute (and library kernels) never release their successor early.
__device__ __forceinline__ void vm_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void vm_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int vm_pdl_enabled;      // defined in elementwise.cu; switched by vm_set_pdl()

template <typename... KArgs, typename... Args>
static inline cudaError_t vm_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vm_pdl_enabled ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Streaming multiprocessors of the current device (asked once per device; 0 if the runtime cannot tell).
static inline int vm_sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) cached[dev] = n;
    }
    return cached[dev];
}

static inline int vm_launch_status() {
    cudaError_t e = cudaGetLastError();
    return static_cast<int>(e);
}
