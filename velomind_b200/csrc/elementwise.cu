// Embedding gather, fused residual-add + RMSNorm, residual add, SwiGLU.
//
// The residual stream is float32 in both compute modes; norms and the residual sum are computed in
// float32.  T is the activation type (float or bf16).
#include "common.cuh"

int vm_pdl_enabled = 1;
VM_API void vm_set_pdl(int on) { vm_pdl_enabled = on ? 1 : 0; }

// ---------------------------------------------------------------- embedding: out[t,:] = table[tokens[t],:]
// Reference: src/cpu/ops/embedding.cpp:27-32.  Ids are validated on the host before the launch; the
// kernel still refuses an id outside the table (writes zeros and raises the error word).
template <typename W>
__global__ void embed_gather_kernel(const W* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ out, int T, int hid, int vocab, int* __restrict__ err) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t];
    const bool ok = (id >= 0 && id < vocab);
    if (!ok && threadIdx.x == 0 && err) atomicExch(err, 1);
    const W* row = table + (size_t)(ok ? id : 0) * hid;
    for (int i = threadIdx.x; i < hid; i += blockDim.x)
        out[(size_t)t * hid + i] = ok ? vm_to_float(row[i]) : 0.f;
}

VM_API int vm_embed_gather(const void* table, int table_dtype, const int* tokens, float* out, int T, int hid,
                           int vocab, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = hid >= 512 ? 256 : 128;
    if (table_dtype == VM_F32)
        vm_launch_pdl(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, tokens, out, T, hid, vocab, err);
    else if (table_dtype == VM_BF16)
        vm_launch_pdl(embed_gather_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table, tokens, out, T, hid, vocab, err);
    else
        return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// ---------------------------------------------------------------- h (+= delta); out = rmsnorm(h) * w
// Reference: src/cpu/ops/rmsnorm.cpp:42-59: inv = 1/sqrt(mean(x^2) + eps); y = x * inv * w.
// One block per output row.  rows == nullptr: output row r reads residual row r and the sum is written
// back to h.  rows != nullptr: output row r reads residual row rows[r]; h is left untouched (the caller
// has no further use for it).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta, const float* __restrict__ w,
                                   T* __restrict__ out, const int* __restrict__ rows, int hid, float eps) {
    extern __shared__ float row[];          // hid floats
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * hid;
    const T* drow = delta ? delta + (size_t)src * hid : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        float v = hrow[i];
        if (drow) v += vm_to_float(drow[i]);
        row[i] = v;
        ss += v * v;
    }
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        const float v = row[i];
        if (drow && !rows) hrow[i] = v;
        out[(size_t)r * hid + i] = vm_from_float<T>(v * inv * w[i]);
    }
}

// The same for bfloat16 activations and hid % 4 == 0, four values per load and store; one WARP per output row (no
// block-wide barrier), the row's sums kept in the warp's shared memory between the two passes.
constexpr int NORM_VEC_WARPS = 4;
__global__ void __launch_bounds__(NORM_VEC_WARPS * 32)
add_rmsnorm_bf16_vec_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ delta, const float* __restrict__ w,
                            __nv_bfloat16* __restrict__ out, const int* __restrict__ rows, int n_out, int hid, float eps) {
    extern __shared__ __align__(16) float vrow[];        // [warps][hid]
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * NORM_VEC_WARPS + warp;
    if (r >= n_out) return;
    const int src = rows ? rows[r] : r;
    float4* hrow = reinterpret_cast<float4*>(h + (size_t)src * hid);
    const uint2* drow = delta ? reinterpret_cast<const uint2*>(delta + (size_t)src * hid) : nullptr;
    float4* mine = reinterpret_cast<float4*>(vrow + (size_t)warp * hid);
    const int n4 = hid >> 2;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    uint2* orow = reinterpret_cast<uint2*>(out + (size_t)r * hid);
    constexpr int NV = 8;                                // rows of up to 1,024 values: a lane's share stays in registers
    if (n4 <= 32 * NV) {
        // all loads of the row first (they do not depend on one another), then the arithmetic: one memory latency
        float4 v[NV];
        uint2 d[NV];
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int i = lane + 32 * u;
            if (i < n4) { v[u] = hrow[i]; if (drow) d[u] = drow[i]; }
        }
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int i = lane + 32 * u;
            if (i < n4) {
                if (drow) {
                    const __nv_bfloat162 d01 = *reinterpret_cast<const __nv_bfloat162*>(&d[u].x), d23 = *reinterpret_cast<const __nv_bfloat162*>(&d[u].y);
                    v[u].x += __low2float(d01); v[u].y += __high2float(d01); v[u].z += __low2float(d23); v[u].w += __high2float(d23);
                    if (!rows) hrow[i] = v[u];
                }
                ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
            }
        }
        ss = vm_warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int i = lane + 32 * u;
            if (i < n4) {
                const float4 ww = w4[i];
                const __nv_bfloat162 o01 = __floats2bfloat162_rn(v[u].x * inv * ww.x, v[u].y * inv * ww.y);
                const __nv_bfloat162 o23 = __floats2bfloat162_rn(v[u].z * inv * ww.z, v[u].w * inv * ww.w);
                uint2 o;
                o.x = *reinterpret_cast<const unsigned*>(&o01); o.y = *reinterpret_cast<const unsigned*>(&o23);
                orow[i] = o;
            }
        }
        return;
    }
    float ss = 0.f;
    for (int i = lane; i < n4; i += 32) {
        float4 v = hrow[i];
        if (drow) {
            const uint2 d = drow[i];
            const __nv_bfloat162 d01 = *reinterpret_cast<const __nv_bfloat162*>(&d.x), d23 = *reinterpret_cast<const __nv_bfloat162*>(&d.y);
            v.x += __low2float(d01); v.y += __high2float(d01); v.z += __low2float(d23); v.w += __high2float(d23);
            if (!rows) hrow[i] = v;
        }
        mine[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = vm_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    for (int i = lane; i < n4; i += 32) {
        const float4 v = mine[i], ww = w4[i];
        const __nv_bfloat162 o01 = __floats2bfloat162_rn(v.x * inv * ww.x, v.y * inv * ww.y);
        const __nv_bfloat162 o23 = __floats2bfloat162_rn(v.z * inv * ww.z, v.w * inv * ww.w);
        uint2 o;
        o.x = *reinterpret_cast<const unsigned*>(&o01); o.y = *reinterpret_cast<const unsigned*>(&o23);
        orow[i] = o;
    }
}

VM_API int vm_add_rmsnorm(float* h, const void* delta, const float* w, void* out, const int* rows, int n_out,
                          int hid, float eps, int act_dtype, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    const int threads = hid >= 1024 ? 256 : 128;
    const size_t smem = (size_t)hid * sizeof(float);
    if (smem > 200 * 1024) return VM_ERR_UNSUPPORTED;
    if (act_dtype == VM_BF16 && hid % 4 == 0 && smem * NORM_VEC_WARPS <= 48 * 1024 && n_out >= 64 &&
        ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 &&
        ((reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(out)) & 7) == 0) {
        vm_launch_pdl(add_rmsnorm_bf16_vec_kernel, dim3((n_out + NORM_VEC_WARPS - 1) / NORM_VEC_WARPS), dim3(NORM_VEC_WARPS * 32),
                      smem * NORM_VEC_WARPS, stream, h, (const __nv_bfloat16*)delta, w, (__nv_bfloat16*)out, rows, n_out, hid, eps);
        return vm_launch_status();
    }
    if (act_dtype == VM_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        vm_launch_pdl(add_rmsnorm_kernel<float>, dim3(n_out), dim3(threads), smem, stream, h, (const float*)delta, w, (float*)out, rows, hid, eps);
    } else if (act_dtype == VM_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        vm_launch_pdl(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_out), dim3(threads), smem, stream, h, (const __nv_bfloat16*)delta, w, (__nv_bfloat16*)out, rows, hid, eps);
    } else {
        return VM_ERR_UNSUPPORTED;
    }
    return vm_launch_status();
}

// ---------------------------------------------------------------- h += delta
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ h, const T* __restrict__ delta, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        h[i] += vm_to_float(delta[i]);
}

VM_API int vm_residual_add(float* h, const void* delta, long long n, int act_dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 8 ? (n + threads - 1) / threads : 148 * 8);
    if (act_dtype == VM_F32) residual_add_kernel<float><<<blocks, threads, 0, stream>>>(h, (const float*)delta, (size_t)n);
    else if (act_dtype == VM_BF16) residual_add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(h, (const __nv_bfloat16*)delta, (size_t)n);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// ---------------------------------------------------------------- out[t,i] = silu(gu[t,i]) * gu[t,I+i]
// Reference: examples/common/llama/llama_graph.cpp:22-28, src/cpu/ops/sigmoid.cpp:23-26:
// (1/(1+exp(-g)) * g) * u, in float32.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int T_, int I) {
    const size_t n = (size_t)T_ * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = vm_to_float(gu[t * 2 * I + i]);
        const float u = vm_to_float(gu[t * 2 * I + I + i]);
        const float sig = 1.0f / (1.0f + expf(-g));
        out[idx] = vm_from_float<T>((sig * g) * u);
    }
}

// bfloat16, I % 8 == 0: eight values per load and store
__global__ void swiglu_bf16_vec_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out, size_t n8, int I8) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n8; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I8;
        const int i = (int)(idx - t * I8);
        const uint4 g4 = gu[t * 2 * I8 + i], u4 = gu[t * 2 * I8 + I8 + i];
        const unsigned gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
        unsigned ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gw[k]), u2 = *reinterpret_cast<const __nv_bfloat162*>(&uw[k]);
            const float ga = __low2float(g2), gb = __high2float(g2);
            // (float32 throughout; the hardware exponential and reciprocal are exact to a few units in the last place,
            //  far inside what the bfloat16 result keeps)
            const float sa = __frcp_rn(1.0f + __expf(-ga)), sb = __frcp_rn(1.0f + __expf(-gb));
            const __nv_bfloat162 o2 = __floats2bfloat162_rn((sa * ga) * __low2float(u2), (sb * gb) * __high2float(u2));
            ow[k] = *reinterpret_cast<const unsigned*>(&o2);
        }
        out[idx] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

VM_API int vm_swiglu(const void* gate_up, void* out, int T, int I, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (act_dtype == VM_BF16 && I % 8 == 0 && ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const size_t n8 = (size_t)T * (I / 8);
        const size_t want8 = (n8 + 255) / 256;
        swiglu_bf16_vec_kernel<<<(int)(want8 < 148 * 16 ? want8 : 148 * 16), 256, 0, stream>>>((const uint4*)gate_up, (uint4*)out, n8, I / 8);
        return vm_launch_status();
    }
    const size_t n = (size_t)T * I;
    const int threads = 256;
    const size_t want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (act_dtype == VM_F32) swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, T, I);
    else if (act_dtype == VM_BF16) swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, T, I);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// ---------------------------------------------------------------- dtype conversion (mixed-precision edges)
template <typename A, typename B>
__global__ void convert_kernel(const A* __restrict__ in, B* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = vm_from_float<B>(vm_to_float(in[i]));
}

VM_API int vm_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const size_t want = ((size_t)n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (in_dtype == VM_F32 && out_dtype == VM_BF16) convert_kernel<float, __nv_bfloat16><<<blocks, threads, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, (size_t)n);
    else if (in_dtype == VM_BF16 && out_dtype == VM_F32) convert_kernel<__nv_bfloat16, float><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, (size_t)n);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
