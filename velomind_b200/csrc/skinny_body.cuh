// Device bodies of the weight-streaming products (see skinny_gemm.cu for what they compute and why).
#pragma once
#include "mma.cuh"

namespace vmsk {


enum : int { PRO_NONE = 0, PRO_RMSNORM = 1 };
enum : int { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_ROPE_KV = 4 };

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;

struct SkinnyParams {
    const void* A;               // bf16 [M, K] (PRO_NONE) or float32 residual [M, K] (PRO_RMSNORM)
    const float* norm_w;         // [K]
    float eps;
    const __nv_bfloat16* W;      // [N, K]
    int M, N, K;
    int pro, epi, tiles;         // tiles: n8 tiles per CTA (1 or 2)
    void* out;                   // bf16 or float32 [M, out_stride]
    int out_stride;
    float* h;                    // residual [M, N]
    int I;                       // swiglu: rows of Wg (and of Wu)
    // rope_kv
    const int* positions; const int* seq_of_token; const int* block_table; int max_blocks;
    const float* inv_freq; int rot_dim;
    __nv_bfloat16* kpages; __nv_bfloat16* vpages; int H, Hkv, D, n_pages; int* err;
    int n_items;                 // work items of the launch (a CTA takes items blockIdx.x, + gridDim.x, ...)
    int kc;                      // k chunk staged in shared memory at a time (multiple of 32)
    int row_bytes;               // shared-memory row pitch of the A tile, == 64 mod 128
    int stages;                  // (skinny_stream_kernel) stages of its ring of weight rows
};

// `item` is the work item (what item_index is for the stand-alone kernel); `smem` the CTA's dynamic shared memory.
// PDL: launched with programmatic dependent launch (weights may be fetched before the predecessor has finished).
// The output columns of a work item: tile A's first column, tile B's, and (rope_kv) the head they lie in.
struct SkinnyCols { int nA, nB, head; };
__device__ __forceinline__ SkinnyCols skinny_cols(const SkinnyParams& p, int item_index) {
    SkinnyCols c{0, 0, 0};
    if (p.epi == EPI_SWIGLU) { c.nA = 8 * item_index; c.nB = p.I + c.nA; }
    else if (p.epi == EPI_ROPE_KV) {
        const int per_head = p.D / 16;
        c.head = item_index / per_head;
        const int sub = item_index - c.head * per_head;
        if (c.head < p.H + p.Hkv && p.rot_dim > 0) { c.nA = c.head * p.D + 8 * sub; c.nB = c.nA + p.D / 2; }   // rotary pair (j, j + D/2)
        else { c.nA = c.head * p.D + 16 * sub; c.nB = c.nA + 8; }
    }
    else if (p.tiles == 2) { c.nA = 16 * item_index; c.nB = c.nA + 8; }
    else { c.nA = 8 * item_index; c.nB = c.nA; }
    return c;
}

// Work items first_item, first_item + item_stride, ... below n_items.  When all of K fits into the shared-memory tile
// (K <= p.kc), A is staged (and normalised) ONCE for all items of the CTA, and an item's first weight blocks are
// requested before the previous item's sums are joined and stored.
// PF: k blocks of 32 that a warp keeps in flight (8 warps x PF x 32 values of K per round).
// LOOP false: the CTA has the one item first_item (the code that looks ahead to a next item is left out).
template <int MT, bool PDL, int PF = 8, bool LOOP = true>
__device__ __forceinline__ void skinny_run(const SkinnyParams& p, const int first_item, const int item_stride, const int n_items,
                                           unsigned char* smem) {
    constexpr int ROWS = 16 * MT;
    unsigned char* sA = smem;                                              // ROWS x row_bytes
    float* red = reinterpret_cast<float*>(smem + (size_t)ROWS * p.row_bytes);   // [SK_WARPS][ROWS][16]
    float* inv = red + SK_WARPS * ROWS * 16;                               // [ROWS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    // (the kernel that writes the cache lets its successor, the attention, start only after its own wait: see there)
    if (PDL && p.epi != EPI_ROPE_KV) vm_pdl_launch_dependents();

    if (first_item >= n_items) return;
    // ---- which output columns
    SkinnyCols cols = skinny_cols(p, first_item);
    const __nv_bfloat16* wA = p.W + (size_t)(cols.nA + g) * p.K;
    const __nv_bfloat16* wB = p.W + (size_t)(cols.nB + g) * p.K;
    const bool two = (p.tiles == 2);
    const bool whole_k = p.K <= p.kc;                       // A is staged once for all items

    // ---- weight fragments do not depend on A: the first group of this warp's k blocks is requested before
    //      anything else, so that its DRAM latency overlaps the staging of A
    uint4 wa[PF], wb[PF];
    auto issue = [&](int kc0, int blocks, int group) {
#pragma unroll
        for (int u = 0; u < PF; ++u) {
            const int b = warp + SK_WARPS * (group * PF + u);
            if (b < blocks) {
                const int k = kc0 + 32 * b + 8 * t4;
                wa[u] = *reinterpret_cast<const uint4*>(wA + k);
                if (two) wb[u] = *reinterpret_cast<const uint4*>(wB + k);
            }
        }
    };
    issue(0, min(p.kc, p.K) / 32, 0);
    // the rotary frequencies of this thread's output column are constants of the model too
    float freq = 0.f;
    if (p.epi == EPI_ROPE_KV && cols.head < p.H + p.Hkv && p.rot_dim > 0) freq = p.inv_freq[(cols.nA - cols.head * p.D) + (tid & 7)];
    if (PDL) vm_pdl_wait();                                 // from here on: data written by earlier kernels
    if (PDL && p.epi == EPI_ROPE_KV) vm_pdl_launch_dependents();
    // the epilogue's per-row facts (position, cache page) are fetched now, long before they are needed
    int row_pos[MT], row_page[MT];
    if (p.epi == EPI_ROPE_KV) {
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            const int item = tid + SK_THREADS * i;
            const int row = item >> 3;
            row_pos[i] = 0; row_page[i] = -1;
            if (item < ROWS * 8 && row < p.M) {
                row_pos[i] = p.positions[row];
                if (p.kpages != nullptr && (LOOP || cols.head >= p.H)) {      // (a CTA with one item of a query head needs no page)
                    const int blk = row_pos[i] / VM_PAGE_TOKENS;
                    row_page[i] = (blk < p.max_blocks) ? p.block_table[(size_t)p.seq_of_token[row] * p.max_blocks + blk] : -1;
                }
            }
        }
    }

    int item_index = first_item;
    do {
    const int nA = cols.nA, nB = cols.nB, head = cols.head;
    const bool first = !LOOP || item_index == first_item;
    // the residual values this thread will add to are requested now: their latency passes under the product
    float res_a[MT], res_b[MT];
    if (p.epi == EPI_RESIDUAL) {
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            const int item = tid + SK_THREADS * i;
            const int row = item >> 3, c = item & 7;
            res_a[i] = res_b[i] = 0.f;
            if (item < ROWS * 8 && row < p.M) {
                const float* o = p.h + (size_t)row * p.N;      // from L2: another SM wrote it
                res_a[i] = __ldcg(o + nA + c);
                if (two) res_b[i] = __ldcg(o + nB + c);
            }
        }
    }
    float acc[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int t = 0; t < 2; ++t) acc[mt][t][0] = acc[mt][t][1] = acc[mt][t][2] = acc[mt][t][3] = 0.f;

    for (int kc0 = 0; kc0 < p.K; kc0 += p.kc) {
        const int kc = min(p.kc, p.K - kc0);
        if (kc0 > 0) __syncthreads();                       // the previous chunk has been consumed
        // ---- stage A[:, kc0 : kc0+kc] as bf16 (once per CTA when all of K fits)
        if (whole_k && !first) {
        } else if (p.pro == PRO_NONE) {
            // (rows past M are never read: their fragments are zeros in registers)
            const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.A);
            const int chunks = kc / 8;
            for (int r = warp; r < p.M; r += SK_WARPS) {
                unsigned char* dst = sA + (size_t)r * p.row_bytes;
                const __nv_bfloat16* src = A + (size_t)r * p.K + kc0;
                for (int ch = lane; ch < chunks; ch += 32) vm_cp_async16(dst + ch * 16, src + ch * 8);
            }
            vm_cp_async_commit();
            vm_cp_async_wait_all();
        } else {
            // x * w as bf16 (the row's 1/rms is applied to the float32 sums in the epilogue: a row scale
            // commutes with the product); a warp owns whole rows and sums their squares on the way
            const float* h = static_cast<const float*>(p.A);
            const int quads = kc / 4;
            for (int r = warp; r < p.M; r += SK_WARPS) {
                unsigned char* dst = sA + (size_t)r * p.row_bytes;
                const float4* hrow = reinterpret_cast<const float4*>(h + (size_t)r * p.K + kc0);
                const float4* wrow = reinterpret_cast<const float4*>(p.norm_w + kc0);
                float ss = 0.f;
                constexpr int NU = PF <= 4 ? 5 : 4;        // loads in flight per lane (5: a row of up to 640 values in one round)
                for (int q0 = lane; q0 < quads; q0 += 32 * NU) {
                    float4 x[NU], w[NU];
#pragma unroll
                    for (int u = 0; u < NU; ++u) {
                        const int qd = q0 + 32 * u;
                        if (qd < quads) { x[u] = __ldcg(hrow + qd); w[u] = wrow[qd]; }     // h: from L2, another SM may have written it
                    }
#pragma unroll
                    for (int u = 0; u < NU; ++u) {
                        const int qd = q0 + 32 * u;
                        if (qd < quads) {
                            ss += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
                            uint2 v;
                            v.x = vm_pack_bf16(x[u].x * w[u].x, x[u].y * w[u].y);
                            v.y = vm_pack_bf16(x[u].z * w[u].z, x[u].w * w[u].w);
                            *reinterpret_cast<uint2*>(dst + qd * 8) = v;
                        }
                    }
                }
                ss = vm_warp_sum(ss);
                if (lane == 0) inv[r] = (kc0 == 0 ? 0.f : inv[r]) + ss;        // sum of squares so far
            }
        }
        if (!(whole_k && !first)) __syncthreads();
        // ---- this warp's k blocks of the chunk: block b covers k = kc0 + 32 b .. + 31
        const int blocks = kc / 32;
        for (int group = 0; warp + SK_WARPS * group * PF < blocks; ++group) {
            if (group > 0 || kc0 > 0) issue(kc0, blocks, group);
#pragma unroll
            for (int u = 0; u < PF; ++u) {
                const int b = warp + SK_WARPS * (group * PF + u);
                if (b < blocks) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint4 a_lo = make_uint4(0u, 0u, 0u, 0u), a_hi = a_lo;
                        if (mt * 16 + g < p.M) a_lo = *reinterpret_cast<const uint4*>(sA + (size_t)(mt * 16 + g) * p.row_bytes + (32 * b + 8 * t4) * 2);
                        if (mt * 16 + g + 8 < p.M) a_hi = *reinterpret_cast<const uint4*>(sA + (size_t)(mt * 16 + g + 8) * p.row_bytes + (32 * b + 8 * t4) * 2);
                        vm_mma_bf16_16816(acc[mt][0], a_lo.x, a_hi.x, a_lo.y, a_hi.y, wa[u].x, wa[u].y);
                        vm_mma_bf16_16816(acc[mt][0], a_lo.z, a_hi.z, a_lo.w, a_hi.w, wa[u].z, wa[u].w);
                        if (two) {
                            vm_mma_bf16_16816(acc[mt][1], a_lo.x, a_hi.x, a_lo.y, a_hi.y, wb[u].x, wb[u].y);
                            vm_mma_bf16_16816(acc[mt][1], a_lo.z, a_hi.z, a_lo.w, a_hi.w, wb[u].z, wb[u].w);
                        }
                    }
                }
            }
        }
    }
    // ---- the next item's first weight blocks are on their way while this item's sums are joined and stored
    float next_freq = 0.f;
    if (LOOP && item_index + item_stride < n_items) {
        cols = skinny_cols(p, item_index + item_stride);
        wA = p.W + (size_t)(cols.nA + g) * p.K;
        wB = p.W + (size_t)(cols.nB + g) * p.K;
        issue(0, min(p.kc, p.K) / 32, 0);
        if (p.epi == EPI_ROPE_KV && cols.head < p.H + p.Hkv && p.rot_dim > 0) next_freq = p.inv_freq[(cols.nA - cols.head * p.D) + (tid & 7)];
    }
    // ---- join the warps' partial sums: red[warp][row][col], col 0..7 = tile A, 8..15 = tile B
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mt * 16 + g + 8 * half;
                if (row < p.M && (t == 0 || two))
                    *reinterpret_cast<float2*>(&red[((size_t)warp * ROWS + row) * 16 + t * 8 + 2 * t4]) =
                        make_float2(acc[mt][t][2 * half], acc[mt][t][2 * half + 1]);
            }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < MT; ++it) {
        const int item = tid + SK_THREADS * it;
        if (item >= ROWS * 8) break;
        const int row = item >> 3, c = item & 7;
        if (row >= p.M) continue;
        float vA = 0.f, vB = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
            vA += red[((size_t)w * ROWS + row) * 16 + c];
            if (two) vB += red[((size_t)w * ROWS + row) * 16 + 8 + c];
        }
        if (p.pro == PRO_RMSNORM) {
            const float rs = 1.0f / sqrtf(inv[row] / (float)p.K + p.eps);       // inv[] holds the row's sum of squares
            vA *= rs; vB *= rs;
        }
        switch (p.epi) {
            case EPI_STORE_BF16: {
                __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride;
                o[nA + c] = __float2bfloat16_rn(vA);
                if (two) o[nB + c] = __float2bfloat16_rn(vB);
            } break;
            case EPI_STORE_F32: {
                float* o = static_cast<float*>(p.out) + (size_t)row * p.out_stride;
                o[nA + c] = vA;
                if (two) o[nB + c] = vB;
            } break;
            case EPI_RESIDUAL: {
                float* o = p.h + (size_t)row * p.N;
                o[nA + c] = res_a[it] + vA;
                if (two) o[nB + c] = res_b[it] + vB;
            } break;
            case EPI_SWIGLU: {
                const float sig = 1.0f / (1.0f + expf(-vA));
                static_cast<__nv_bfloat16*>(p.out)[(size_t)row * p.out_stride + nA + c] = __float2bfloat16_rn((sig * vA) * vB);
            } break;
            case EPI_ROPE_KV: {
                const int pos = row_pos[it];
                float ya = vA, yb = vB;
                int da, db;                                 // the two columns' places inside the head
                if (head < p.H + p.Hkv && p.rot_dim > 0) {
                    da = (nA - head * p.D) + c; db = da + p.D / 2;
                    float s, co;
                    sincosf((float)pos * freq, &s, &co);
                    ya = vA * co - vB * s;
                    yb = vB * co + vA * s;
                } else { da = (nA - head * p.D) + c; db = da + 8; }
                if (head < p.H) {
                    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride + (size_t)head * p.D;
                    o[da] = __float2bfloat16_rn(ya); o[db] = __float2bfloat16_rn(yb);
                } else if (p.kpages != nullptr) {
                    const int page = row_page[it];
                    if (page < 0 || page >= p.n_pages) { if (p.err) atomicExch(p.err, 2); break; }
                    const bool is_k = head < p.H + p.Hkv;
                    const int hk = is_k ? head - p.H : head - p.H - p.Hkv;
                    __nv_bfloat16* dst = (is_k ? p.kpages : p.vpages) + (size_t)page * ((size_t)p.Hkv * VM_PAGE_TOKENS * p.D)
                                         + ((size_t)hk * VM_PAGE_TOKENS + pos % VM_PAGE_TOKENS) * p.D;
                    dst[da] = __float2bfloat16_rn(ya); dst[db] = __float2bfloat16_rn(yb);
                }
            } break;
        }
    }
    if (LOOP) freq = next_freq;
    __syncthreads();                                        // the sums' buffer is reused by the next item
    } while (LOOP && (item_index += item_stride) < n_items);
}

// One work item (the persistent decode kernel deals items out itself).
template <int MT, bool PDL, int PF = 8>
__device__ __forceinline__ void skinny_body(const SkinnyParams& p, const int item_index, unsigned char* smem) {
    skinny_run<MT, PDL, PF, false>(p, item_index, 1, item_index + 1, smem);
}

// The same product for MANY output columns (the vocabulary head): the warps of a CTA split N instead of K.
// Each warp owns 8 columns over all of K, so there is no cross-warp sum and the A tile is staged once per
// 64 columns.  Plain A (bf16), store epilogue (bf16 or float32).
template <int MT, bool PDL>
__device__ __forceinline__ void skinny_wide_body(const SkinnyParams& p, const int item_index, unsigned char* smem) {
    constexpr int ROWS = 16 * MT;
    constexpr int PF = 6;
    unsigned char* sA = smem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    if (PDL) vm_pdl_launch_dependents();
    const int n0 = (item_index * SK_WARPS + warp) * 8;
    const bool live = n0 < p.N;
    const __nv_bfloat16* wrow = p.W + (size_t)(live ? n0 + g : 0) * p.K;
    uint4 wa[PF];
    auto issue = [&](int first_block, int blocks) {
#pragma unroll
        for (int u = 0; u < PF; ++u) {
            const int b = first_block + u;
            if (live && b < blocks) wa[u] = *reinterpret_cast<const uint4*>(wrow + 32 * b + 8 * t4);
        }
    };
    const int blocks = p.K / 32;
    issue(0, blocks);
    if (PDL) vm_pdl_wait();
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
    {
        const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.A);
        const int chunks = p.K / 8;
        for (int r = warp; r < p.M; r += SK_WARPS) {         // rows past M are never read
            unsigned char* dst = sA + (size_t)r * p.row_bytes;
            const __nv_bfloat16* src = A + (size_t)r * p.K;
            for (int ch = lane; ch < chunks; ch += 32) vm_cp_async16(dst + ch * 16, src + ch * 8);
        }
        vm_cp_async_commit();
        vm_cp_async_wait_all();
    }
    __syncthreads();
    for (int b0 = 0; b0 < blocks; b0 += PF) {
        if (b0 > 0) issue(b0, blocks);
#pragma unroll
        for (int u = 0; u < PF; ++u) {
            const int b = b0 + u;
            if (live && b < blocks) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint4 a_lo = make_uint4(0u, 0u, 0u, 0u), a_hi = a_lo;
                    if (mt * 16 + g < p.M) a_lo = *reinterpret_cast<const uint4*>(sA + (size_t)(mt * 16 + g) * p.row_bytes + (32 * b + 8 * t4) * 2);
                    if (mt * 16 + g + 8 < p.M) a_hi = *reinterpret_cast<const uint4*>(sA + (size_t)(mt * 16 + g + 8) * p.row_bytes + (32 * b + 8 * t4) * 2);
                    vm_mma_bf16_16816(acc[mt], a_lo.x, a_hi.x, a_lo.y, a_hi.y, wa[u].x, wa[u].y);
                    vm_mma_bf16_16816(acc[mt], a_lo.z, a_hi.z, a_lo.w, a_hi.w, wa[u].z, wa[u].w);
                }
            }
        }
    }
    if (live) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = mt * 16 + g + 8 * half;
            if (row >= p.M) continue;
            const int col = n0 + 2 * t4;
            const float v0 = acc[mt][2 * half], v1 = acc[mt][2 * half + 1];
            if (p.epi == EPI_STORE_F32) {
                float* o = static_cast<float*>(p.out) + (size_t)row * p.out_stride + col;
                o[0] = v0; o[1] = v1;
            } else {
                __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride + col;
                o[0] = __float2bfloat16_rn(v0); o[1] = __float2bfloat16_rn(v1);
            }
        }
    }
    }
    __syncthreads();                                        // the A tile may be overwritten by another item
}

// shared-memory row pitch of the A tile (== 64 mod 128 bytes) and size of the whole buffer of skinny_body
__host__ __device__ inline int skinny_pitch(int kc) { int pitch = kc * 2; pitch += ((64 - pitch % 128) + 128) % 128; return pitch; }
__host__ __device__ inline int skinny_chunk(int K, int rows) { const int cap = (96 * 1024) / (rows * 2) / 128 * 128; return K > cap ? cap : K; }
__host__ __device__ inline size_t skinny_smem_bytes(int K, int rows) {
    return (size_t)rows * skinny_pitch(skinny_chunk(K, rows)) + (size_t)SK_WARPS * rows * 16 * sizeof(float) + rows * sizeof(float);
}

}  // namespace vmsk
