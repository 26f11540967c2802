// Attention over the paged cache, any head size / head count / group size, float32 or bf16 storage,
// float32 arithmetic.  One warp per (token, query head); this is the kernel of the true 32-bit path
// and the fallback for shapes the tensor-core kernels refuse.
//
// Reference arithmetic: examples/common/llama/llama_graph.cpp:97-103 (scores = q k^T, softmax over the
// keys a query may see, times v) in the online form of src/cpu/ops/fused_attention.cpp:84-135.  The
// reference folds 1/sqrt(D) into Wq at load (examples/smollm2/model_loader.cpp:277); here `scale`
// multiplies the query.  Query head h reads kv head h / (H / Hkv) (src/cpu/ops/repeat_kv.cpp:51-61).
//
// A query at position p sees keys at positions max(0, p - window + 1) .. p (window == 0: all).  Keys
// are walked in chunks of 32 that start at absolute multiples of 32, one key per lane, and each
// dot product is summed in index order by one lane: the result for a position does not depend on how
// the tokens were cut into steps or what else is in the batch.
#include "common.cuh"

constexpr int ATT_WARPS = 4;

template <typename T, int EPL>
__global__ void attn_generic_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ kpages,
                                    const T* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    T* __restrict__ out, int n_tokens, int H, int Hkv, int D, float scale, int window,
                                    int n_pages, int* __restrict__ err) {
    extern __shared__ float qs_all[];                       // ATT_WARPS x D
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * ATT_WARPS + warp;
    if (w >= (long long)n_tokens * H) return;
    const int t = (int)(w / H), h = (int)(w - (long long)t * H);
    const int hk = h / (H / Hkv);
    const int pos = positions[t], seq = seq_of_token[t];
    float* qs = qs_all + warp * D;
    const T* qrow = q + (size_t)t * q_row_stride + (size_t)h * D;
    for (int d = lane; d < D; d += 32) qs[d] = vm_to_float(qrow[d]) * scale;
    __syncwarp();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const size_t page_stride = (size_t)Hkv * VM_PAGE_TOKENS * D;
    float m = -INFINITY, l = 0.f;
    float acc[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[i] = 0.f;

    for (int base = (lo / 32) * 32; base <= pos; base += 32) {
        const int blk = base / VM_PAGE_TOKENS;
        const int page = (blk < max_blocks) ? block_table[(size_t)seq * max_blocks + blk] : -1;
        if (page < 0 || page >= n_pages) {                 // a page the step needs is not there: report, skip
            if (lane == 0 && err) atomicExch(err, 3);
            continue;
        }
        const size_t tile = (size_t)page * page_stride + ((size_t)hk * VM_PAGE_TOKENS + (base % VM_PAGE_TOKENS)) * D;
        const int j = base + lane;
        const bool valid = (j >= lo && j <= pos);
        float s = -INFINITY;
        if (valid) {
            const T* krow = kpages + tile + (size_t)lane * D;
            float a = 0.f;
            for (int d = 0; d < D; ++d) a = fmaf(qs[d], vm_to_float(krow[d]), a);
            s = a;
        }
        const float m_new = fmaxf(m, vm_warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);               // m == -inf on the first chunk: alpha = 0
        l = l * alpha + vm_warp_sum(p);
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] *= alpha;
        const int cnt = min(32, pos - base + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vrow = vpages + tile + (size_t)jj * D;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(pj, vm_to_float(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
    T* orow = out + ((size_t)t * H + h) * D;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) orow[d] = vm_from_float<T>(acc[i] * inv);
    }
}

template <typename T>
static int launch_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                          int max_blocks, const int* positions, const int* seq_of_token, void* out, int n_tokens, int H,
                          int Hkv, int D, float scale, int window, int n_pages, int* err, cudaStream_t stream) {
    const long long warps = (long long)n_tokens * H;
    const int blocks = (int)((warps + ATT_WARPS - 1) / ATT_WARPS);
    const size_t smem = (size_t)ATT_WARPS * D * sizeof(float);
    const int epl = (D + 31) / 32;
#define VM_ATT_CASE(E)                                                                                              \
    case E:                                                                                                         \
        attn_generic_kernel<T, E><<<blocks, ATT_WARPS * 32, smem, stream>>>(                                         \
            (const T*)q, q_row_stride, (const T*)kpages, (const T*)vpages, block_table, max_blocks, positions,      \
            seq_of_token, (T*)out, n_tokens, H, Hkv, D, scale, window, n_pages, err);                               \
        break;
    switch (epl) {
        VM_ATT_CASE(1) VM_ATT_CASE(2) VM_ATT_CASE(3) VM_ATT_CASE(4) VM_ATT_CASE(5) VM_ATT_CASE(6) VM_ATT_CASE(7) VM_ATT_CASE(8)
        default: return VM_ERR_UNSUPPORTED;
    }
#undef VM_ATT_CASE
    return vm_launch_status();
}

// q: [n_tokens, H, D] rows with stride q_row_stride elements; out: [n_tokens, H*D] contiguous.
VM_API int vm_attention_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                const int* block_table, int max_blocks, const int* positions, const int* seq_of_token,
                                void* out, int n_tokens, int H, int Hkv, int D, float scale, int window, int n_pages,
                                int act_dtype, int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || D > 256) return VM_ERR_UNSUPPORTED;
    if (act_dtype == VM_F32)
        return launch_generic<float>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, seq_of_token, out,
                                     n_tokens, H, Hkv, D, scale, window, n_pages, err, stream);
    if (act_dtype == VM_BF16)
        return launch_generic<__nv_bfloat16>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, seq_of_token,
                                             out, n_tokens, H, Hkv, D, scale, window, n_pages, err, stream);
    return VM_ERR_UNSUPPORTED;
}
