// Position encoding (half-split rotary pairs) of queries and keys, fused with the write of the new
// keys and values into the paged cache.
//
// Reference: src/cpu/ops/rotary_embedding.cpp:30-44 (pairs (j, j + half): y[j] = a*c - b*s,
// y[j+half] = b*c + a*s) with the angle of examples/common/llama/llama_rope_mask.cpp:17-24
// (float(pos) * inv_freq[j] in float32, then cos/sin).  inv_freq comes from the host as a float32
// table, so a position encoding with other frequencies only changes the table.  Keys are cached after
// rotation (examples/common/llama/llama_graph.cpp:210-215).
//
// qkv is [T, (H + 2*Hkv) * D]: queries, then keys, then values of one token.  Queries are rotated in
// place; keys and values go to page block_table[seq, pos / 64], row pos % 64 of their kv head.
// With kpages == nullptr nothing is cached (the run reads another run's cache).
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                     int max_blocks, const float* __restrict__ inv_freq, int rot_dim,
                                     T* __restrict__ kpages, T* __restrict__ vpages, int H, int Hkv, int D,
                                     int n_pages, int* __restrict__ err) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int blk = pos / VM_PAGE_TOKENS;
    const int page = (blk < max_blocks) ? block_table[(size_t)seq * max_blocks + blk] : -1;
    const bool write_kv = (kpages != nullptr);
    if (write_kv && (page < 0 || page >= n_pages)) {   // the host reserves pages before the step; never write astray
        if (threadIdx.x == 0 && err) atomicExch(err, 2);
        return;
    }
    T* row = qkv + (size_t)t * (H + 2 * Hkv) * D;
    const size_t page_stride = (size_t)Hkv * VM_PAGE_TOKENS * D;
    const int in_page = pos % VM_PAGE_TOKENS;
    const int half = rot_dim / 2;
    const float fpos = (float)pos;

    // rotary pairs of query heads (in place) and key heads (to the cache)
    const int n_pairs = (write_kv ? H + Hkv : H) * half;
    for (int it = threadIdx.x; it < n_pairs; it += blockDim.x) {
        const int head = it / half, j = it - head * half;
        T* x = row + (size_t)head * D;
        const float a = vm_to_float(x[j]), b = vm_to_float(x[j + half]);
        float s, c;
        sincosf(fpos * inv_freq[j], &s, &c);
        const float ya = a * c - b * s;
        const float yb = b * c + a * s;
        if (head < H) {
            x[j] = vm_from_float<T>(ya);
            x[j + half] = vm_from_float<T>(yb);
        } else {
            T* dst = kpages + (size_t)page * page_stride + ((size_t)(head - H) * VM_PAGE_TOKENS + in_page) * D;
            dst[j] = vm_from_float<T>(ya);
            dst[j + half] = vm_from_float<T>(yb);
        }
    }
    if (!write_kv) return;                      // a run that reads another run's cache only rotates its queries
    // key dimensions beyond the rotated part pass through
    const int tail = D - rot_dim;
    for (int it = threadIdx.x; it < Hkv * tail; it += blockDim.x) {
        const int hk = it / tail, d = rot_dim + (it - hk * tail);
        kpages[(size_t)page * page_stride + ((size_t)hk * VM_PAGE_TOKENS + in_page) * D + d] = row[(size_t)(H + hk) * D + d];
    }
    // values
    for (int it = threadIdx.x; it < Hkv * D; it += blockDim.x) {
        const int hk = it / D, d = it - hk * D;
        vpages[(size_t)page * page_stride + ((size_t)hk * VM_PAGE_TOKENS + in_page) * D + d] = row[(size_t)(H + Hkv + hk) * D + d];
    }
}

VM_API int vm_rope_kv_write(void* qkv, const int* positions, const int* seq_of_token, const int* block_table,
                            int max_blocks, const float* inv_freq, int rot_dim, void* kpages, void* vpages,
                            int T, int H, int Hkv, int D, int n_pages, int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot_dim < 0 || rot_dim > D || (rot_dim & 1) || (rot_dim > 0 && inv_freq == nullptr)) return VM_ERR_BAD_ARG;
    const int work = (H + Hkv) * (rot_dim / 2) + Hkv * D;
    const int threads = work >= 512 ? 256 : 128;
    if (act_dtype == VM_F32)
        rope_kv_write_kernel<float><<<T, threads, 0, stream>>>((float*)qkv, positions, seq_of_token, block_table, max_blocks,
            inv_freq, rot_dim, (float*)kpages, (float*)vpages, H, Hkv, D, n_pages, err);
    else if (act_dtype == VM_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((__nv_bfloat16*)qkv, positions, seq_of_token, block_table, max_blocks,
            inv_freq, rot_dim, (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, H, Hkv, D, n_pages, err);
    else
        return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
