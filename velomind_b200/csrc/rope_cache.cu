// Rotary position encoding of queries and keys, fused with the write of the new keys and values into the
// paged cache.
//
// Reference: src/cpu/ops/rotary_embedding.cpp:30-44 (pairs (j, j + half): y[j] = a*c - b*s,
// y[j+half] = b*c + a*s) with the angle of examples/common/llama/llama_rope_mask.cpp:17-24
// (float(pos) * inv_freq[j] in float32, then cos/sin).  inv_freq comes from the host as a float32
// table, so a position encoding with other frequencies only changes the table; which two values of a head
// make pair j is an argument too (`pairing`: VM_PAIR_HALF_SPLIT = (j, j + rot_dim/2), what the reference
// does; VM_PAIR_INTERLEAVED = (2j, 2j + 1)).  Keys are cached after rotation
// (examples/common/llama/llama_graph.cpp:210-215).
//
// qkv is [T, (H + 2*Hkv) * D]: queries, then keys, then values of one token.  Queries are rotated in
// place; keys and values go to page block_table[seq, pos / 64], row pos % 64 of their kv head.
// With kpages == nullptr nothing is cached (the run reads another run's cache).
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                     int max_blocks, const float* __restrict__ inv_freq, int rot_dim, int pairing,
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
        const int ia = pairing == VM_PAIR_INTERLEAVED ? 2 * j : j;
        const int ib = pairing == VM_PAIR_INTERLEAVED ? 2 * j + 1 : j + half;
        const float a = vm_to_float(x[ia]), b = vm_to_float(x[ib]);
        float s, c;
        sincosf(fpos * inv_freq[j], &s, &c);
        const float ya = a * c - b * s;
        const float yb = b * c + a * s;
        if (head < H) {
            x[ia] = vm_from_float<T>(ya);
            x[ib] = vm_from_float<T>(yb);
        } else {
            T* dst = kpages + (size_t)page * page_stride + ((size_t)(head - H) * VM_PAGE_TOKENS + in_page) * D;
            dst[ia] = vm_from_float<T>(ya);
            dst[ib] = vm_from_float<T>(yb);
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

// bfloat16, rot_dim == D, D % 16 == 0: the angles of a token are computed once (not once per head), and every thread
// moves eight values of both halves of a head with 16-byte loads and stores.
__global__ void __launch_bounds__(128)
rope_kv_write_bf16_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                              const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_blocks,
                              const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ kpages,
                              __nv_bfloat16* __restrict__ vpages, int H, int Hkv, int D, int n_pages, int* __restrict__ err) {
    extern __shared__ float cs[];                       // [D/2] cosines, [D/2] sines
    // Launched with programmatic dependent launch: it reads nothing before its predecessor is complete, and lets its
    // successor start only then.  The successor may be the decode attention, which fetches the cache rows of EARLIER
    // tokens in its preamble and this kernel's new rows after its own wait (the rule is in common.cuh).
    vm_pdl_wait();
    vm_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int blk = pos / VM_PAGE_TOKENS;
    const int page = (blk < max_blocks) ? block_table[(size_t)seq * max_blocks + blk] : -1;
    const bool write_kv = (kpages != nullptr);
    if (write_kv && (page < 0 || page >= n_pages)) {
        if (threadIdx.x == 0 && err) atomicExch(err, 2);
        return;
    }
    const int half = D / 2;
    __nv_bfloat16* row = qkv + (size_t)t * (H + 2 * Hkv) * D;
    const size_t page_stride = (size_t)Hkv * VM_PAGE_TOKENS * D;
    const int in_page = pos % VM_PAGE_TOKENS;
    const int g8 = half / 8;                            // groups of eight pairs per head
    const int n_items = (write_kv ? H + Hkv : H) * g8;
    // each thread's first item is requested before the angles are computed: its latency passes under them
    const int it0 = threadIdx.x;
    uint4 first_a = make_uint4(0u, 0u, 0u, 0u), first_b = first_a;
    if (it0 < n_items) {
        const int head = it0 / g8, j0 = (it0 - head * g8) * 8;
        const __nv_bfloat16* x = row + (size_t)head * D;
        first_a = *reinterpret_cast<const uint4*>(x + j0); first_b = *reinterpret_cast<const uint4*>(x + half + j0);
    }
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        cs[j] = c; cs[half + j] = s;
    }
    __syncthreads();
    for (int it = threadIdx.x; it < n_items; it += blockDim.x) {
        const int head = it / g8, j0 = (it - head * g8) * 8;
        __nv_bfloat16* x = row + (size_t)head * D;
        uint4 a4 = first_a, b4 = first_b;
        if (it != it0) { a4 = *reinterpret_cast<const uint4*>(x + j0); b4 = *reinterpret_cast<const uint4*>(x + half + j0); }
        const unsigned aw[4] = {a4.x, a4.y, a4.z, a4.w}, bw[4] = {b4.x, b4.y, b4.z, b4.w};
        unsigned ya[4], yb[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 a2 = *reinterpret_cast<const __nv_bfloat162*>(&aw[k]), b2 = *reinterpret_cast<const __nv_bfloat162*>(&bw[k]);
            const float a0 = __low2float(a2), a1 = __high2float(a2), b0 = __low2float(b2), b1 = __high2float(b2);
            const float c0 = cs[j0 + 2 * k], c1 = cs[j0 + 2 * k + 1], s0 = cs[half + j0 + 2 * k], s1 = cs[half + j0 + 2 * k + 1];
            const __nv_bfloat162 oa = __floats2bfloat162_rn(a0 * c0 - b0 * s0, a1 * c1 - b1 * s1);
            const __nv_bfloat162 ob = __floats2bfloat162_rn(b0 * c0 + a0 * s0, b1 * c1 + a1 * s1);
            ya[k] = *reinterpret_cast<const unsigned*>(&oa); yb[k] = *reinterpret_cast<const unsigned*>(&ob);
        }
        __nv_bfloat16* dst = (head < H) ? x
                                        : kpages + (size_t)page * page_stride + ((size_t)(head - H) * VM_PAGE_TOKENS + in_page) * D;
        *reinterpret_cast<uint4*>(dst + j0) = make_uint4(ya[0], ya[1], ya[2], ya[3]);
        *reinterpret_cast<uint4*>(dst + half + j0) = make_uint4(yb[0], yb[1], yb[2], yb[3]);
    }
    if (!write_kv) return;
    const int v8 = D / 8;
    for (int it = threadIdx.x; it < Hkv * v8; it += blockDim.x) {            // values
        const int hk = it / v8, d = (it - hk * v8) * 8;
        *reinterpret_cast<uint4*>(vpages + (size_t)page * page_stride + ((size_t)hk * VM_PAGE_TOKENS + in_page) * D + d) =
            *reinterpret_cast<const uint4*>(row + (size_t)(H + Hkv + hk) * D + d);
    }
}

VM_API int vm_rope_kv_write(void* qkv, const int* positions, const int* seq_of_token, const int* block_table,
                            int max_blocks, const float* inv_freq, int rot_dim, int pairing, void* kpages, void* vpages,
                            int T, int H, int Hkv, int D, int n_pages, int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot_dim < 0 || rot_dim > D || (rot_dim & 1) || (rot_dim > 0 && inv_freq == nullptr)) return VM_ERR_BAD_ARG;
    if (pairing != VM_PAIR_HALF_SPLIT && pairing != VM_PAIR_INTERLEAVED) return VM_ERR_BAD_ARG;
    if (act_dtype == VM_BF16 && pairing == VM_PAIR_HALF_SPLIT && rot_dim == D && D % 16 == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
        ((reinterpret_cast<uintptr_t>(kpages) | reinterpret_cast<uintptr_t>(vpages)) & 15) == 0) {
        // (a thread takes eight pairs of a head: 64 threads cover this model's 9 + 3 heads of 64 in one round)
        const int threads = (H + Hkv) * (D / 16) <= 64 ? 64 : 128;
        vm_launch_pdl(rope_kv_write_bf16_vec_kernel, dim3(T), dim3(threads), (size_t)D * sizeof(float), stream,
                      (__nv_bfloat16*)qkv, positions, seq_of_token, block_table, max_blocks, inv_freq, (__nv_bfloat16*)kpages,
                      (__nv_bfloat16*)vpages, H, Hkv, D, n_pages, err);
        return vm_launch_status();
    }
    const int work = (H + Hkv) * (rot_dim / 2) + Hkv * D;
    const int threads = work >= 512 ? 256 : 128;
    if (act_dtype == VM_F32)
        rope_kv_write_kernel<float><<<T, threads, 0, stream>>>((float*)qkv, positions, seq_of_token, block_table, max_blocks,
            inv_freq, rot_dim, pairing, (float*)kpages, (float*)vpages, H, Hkv, D, n_pages, err);
    else if (act_dtype == VM_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((__nv_bfloat16*)qkv, positions, seq_of_token, block_table, max_blocks,
            inv_freq, rot_dim, pairing, (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, H, Hkv, D, n_pages, err);
    else
        return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
