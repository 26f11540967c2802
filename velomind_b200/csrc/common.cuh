// Shared device helpers for the velomind_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VM_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with kernels/ops.py
enum : int { VM_F32 = 0, VM_BF16 = 1 };

// Status codes returned by launchers: 0 ok, >0 a cudaError_t, <0 one of these.
enum : int { VM_ERR_UNSUPPORTED = -1, VM_ERR_BAD_ARG = -2 };

constexpr int VM_PAGE_TOKENS = 64;

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

static inline int vm_launch_status() {
    cudaError_t e = cudaGetLastError();
    return static_cast<int>(e);
}
