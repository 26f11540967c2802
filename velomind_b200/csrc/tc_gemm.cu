// Matrix products for many rows (prefill) on the fifth-generation tensor cores: y = x W^T with x [M, K] and
// W [N, K] bf16 (K contiguous), float32 accumulation in tensor memory, and the elementwise work that follows
// the product fused into the epilogue:
//
//   store      out[M, N] = x W^T                       bf16 or float32
//   residual   h[M, N] += x W^T                        float32 residual stream (llama_graph.cpp:225-226, :137)
//   swiglu     out[M, I] = silu(x Wg^T) * (x Wu^T)      W = [Wg; Wu] stacked (llama_graph.cpp:22-28)
//   rope_kv    W = [Wq; Wk; Wv] stacked, one head per tile: rotate q and k (rotary_embedding.cpp:30-44), q to
//              out [M, H*D], k and v into the paged cache (llama_graph.cpp:210-215)
//
// The reference multiplies with cuBLAS SGEMM (src/cuda/ops/matmul.cu:87-126) and runs each elementwise step
// as a kernel of its own.
//
// CTAs are persistent: each walks over 128 x BN output tiles (tile index += grid size).  Warp 0 (one lane) is
// the TMA producer: cp.async.bulk.tensor loads of a 128 x 64 tile of x and a BN x 64 tile of W per k block into
// a ring of 128-byte-swizzled shared-memory stages, completion on mbarriers.  Warp 1 (one lane) issues
// tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN, K = 16) four times per k block and frees each stage
// with tcgen05.commit.  The accumulator is double-buffered in tensor memory (2 x BN columns): warps 2..5, the
// epilogue, read tile t with tcgen05.ld, apply the fused operation and write global memory while the MMAs of
// tile t+1 run.  No multicast, no clusters.
//
// Every wait on an mbarrier is bounded; when a wait gives up, the CTA raises an error word, waits (bounded)
// for its own copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include "mma.cuh"

namespace {

enum : int { TC_STORE_BF16 = 0, TC_STORE_F32 = 1, TC_RESIDUAL = 2, TC_SWIGLU = 3, TC_ROPE_KV = 4 };

constexpr int TC_BM = 128, TC_BK = 64, TC_KPS = 2;
constexpr int TC_THREADS = 192;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 20;

struct TcParams {
    int M, N, K, epi;
    void* out; int out_stride;       // bf16 / float32 [M, out_stride]
    float* h;                        // residual [M, N]
    int I;                           // swiglu: rows of Wg
    const int* positions; const int* seq_of_token; const int* block_table; int max_blocks;
    const float* inv_freq; int rot_dim;
    __nv_bfloat16* kpages; __nv_bfloat16* vpages; int H, Hkv, D, n_pages;
    int* err;                        // cache faults (2) and abandoned waits (4)
    int tiles_m, tiles_n;
    int tma_residual;                // the residual sum leaves through TMA reduce-add (map_h is valid)
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle: start address
// (>> 4) in bits 0-13, leading byte offset (unused for this layout; 1) in bits 16-29, stride byte offset =
// 8 rows * 128 B = 1024 B (>> 4) in bits 32-45, descriptor version 1 in bits 46-47, layout 2 (128-byte swizzle) in
// bits 61-63.  A k step of 16 bf16 inside the 128-byte row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_h, const TcParams p) {
    // a stage holds TC_KPS k blocks of 64 (each an A tile and a B tile): one barrier round trip of the MMA warp per stage, and
    // a wait on an mbarrier costs it a few hundred cycles, as much as the four MMAs of one k block take on the tensor cores
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = TC_KPS * (A_BYTES + B_BYTES);
    constexpr int STAGES = 3;
    constexpr uint32_t TMEM_COLS = 2 * BN;                                // two accumulators; a power of two >= 32
    // instruction descriptor: float32 accumulate (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), both K-major,
    // N >> 3 in bits 17-22, M >> 4 in bits 24-28
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
    extern __shared__ __align__(1024) unsigned char smem_raw[];          // swizzled tiles want 1024-byte alignment (checked below)
    unsigned char* tiles = smem_raw;
    // no static shared memory: the bookkeeping sits behind the tiles, so that two CTAs fit one SM
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(tiles + (size_t)STAGES * STAGE_BYTES + 4 * 4096);   // full[S], empty[S], accum_full[2], accum_empty[2]
    uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    int& abort_flag = *reinterpret_cast<int*>(bars + 2 * STAGES + 5);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = BN / 2;
    const int num_kb = (p.K + TC_BK * TC_KPS - 1) / (TC_BK * TC_KPS);      // stages per tile (a last half-empty one is zero-filled by TMA)
    const int num_tiles = p.tiles_m * p.tiles_n;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t accf0 = smem_u32(&bars[2 * STAGES]), acce0 = smem_u32(&bars[2 * STAGES + 2]);

    if (threadIdx.x == 0) {
        abort_flag = (smem_u32(tiles) & 1023u) ? 1 : 0;       // misaligned tiles would give wrong sums: give up instead
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf0 + 8 * a, 1); mbar_init(acce0 + 8 * a, 4); }   // 4 epilogue warps free an accumulator
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                     // one warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int it = 0;                                  // k blocks issued so far, over all of this CTA's tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int tile_m = tile / p.tiles_n, tile_n = tile - tile_m * p.tiles_n;
                const int m0 = tile_m * TC_BM;
                int n0 = tile_n * BN, n1 = -1;           // where the tile's W rows start (two ranges for swiglu)
                if (p.epi == TC_SWIGLU) { n0 = tile_n * half; n1 = p.I + n0; }
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = (uint32_t)(it / STAGES);
                    ok = mbar_wait(empty0 + 8 * s, (round & 1u) ^ 1u, abort_p);
                    if (!ok) break;
                    const uint32_t full = full0 + 8 * s;
                    mbar_expect_tx(full, STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < TC_KPS; ++j) {
                        const uint32_t a_dst = smem_u32(tiles + (size_t)s * STAGE_BYTES) + j * (A_BYTES + B_BYTES), b_dst = a_dst + A_BYTES;
                        const int k0 = (kb * TC_KPS + j) * TC_BK;
                        tma_load_2d(a_dst, &map_a, k0, m0, full);
                        tma_load_2d(b_dst, &map_b, k0, n0, full);
                        if (n1 >= 0) tma_load_2d(b_dst + B_BYTES / 2, &map_b, k0, n1, full);   // half a tile each
                    }
                }
            }
            if (*abort_p) {
                // gave up somewhere: let the copies that are still in flight land before the CTA's memory goes away
                for (int j = max(0, it - STAGES); j < it; ++j) {
                    uint32_t done = 0;
                    for (uint32_t w = 0; w < TC_WAIT_LIMIT && !done; ++w)
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                     : "=r"(done) : "r"(full0 + 8 * (j % STAGES)), "r"((uint32_t)(j / STAGES) & 1u) : "memory");
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int it = 0, t = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
                const int a = t & 1;
                ok = mbar_wait(acce0 + 8 * a, (((uint32_t)t >> 1) & 1u) ^ 1u, abort_p);     // the epilogue has drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(a * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = (uint32_t)(it / STAGES);
                    ok = mbar_wait(full0 + 8 * s, round & 1u, abort_p);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int j = 0; j < TC_KPS; ++j) {
                        const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES) + j * (A_BYTES + B_BYTES), b_addr = a_addr + A_BYTES;
                        const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(b_addr);
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)  // +32 bytes per k step: +2 in the descriptor's 16-byte units
                            tc_mma_bf16(tmem_d, da + 2 * k, db + 2 * k, IDESC, (kb > 0 || j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(empty0 + 8 * s);            // the stage is free once these MMAs have read it
                }
                if (ok) tc_commit(accf0 + 8 * a);         // the accumulator is complete once all MMAs are done
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: warps 2..5, lanes 32 * (warp % 4) ..
        const int quarter = warp & 3;
        int t = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
        const int tile_m = tile / p.tiles_n, tile_n = tile - tile_m * p.tiles_n;
        const int m0 = tile_m * TC_BM;
        int n0 = tile_n * BN;
        if (p.epi == TC_SWIGLU) n0 = tile_n * half;
        const int acc = t & 1;
        const int row = m0 + quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const bool ready = __all_sync(0xffffffffu, mbar_wait(accf0 + 8 * acc, ((uint32_t)t >> 1) & 1u, abort_p));   // one answer per warp
        tc_fence_after();
        if (!ready) break;
        {
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            if (p.epi == TC_STORE_BF16 || p.epi == TC_STORE_F32 || p.epi == TC_RESIDUAL) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    __syncwarp();
                    tc_ld32(taddr + c0, v);
                    tc_ld_wait();
                    const int col0 = n0 + c0;
                    if (p.epi == TC_RESIDUAL && p.tma_residual) {
                        // h += chunk, asynchronously: the 32 x 32 float chunk goes to shared memory (128-byte swizzle, so
                        // that the lanes' 16-byte stores spread over the banks) and a TMA reduce-add carries it to global
                        // memory; rows and columns beyond the matrix are clipped by the copy engine
                        if (col0 >= p.N) continue;                     // warp-uniform
                        float* stg = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES) + (size_t)(warp - 2) * 1024;
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the last chunk has left the buffer
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int chunk = i ^ (lane & 7);
                            *reinterpret_cast<float4*>(stg + lane * 32 + chunk * 4) =
                                make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                                         ::"l"(&map_h), "r"(col0), "r"(m0 + quarter * 32), "r"(smem_u32(stg)) : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                        continue;
                    }
                    if (!row_ok || col0 >= p.N) continue;
                    if (p.epi == TC_STORE_BF16) {
                        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride + col0;
                        if (col0 + 32 <= p.N && (p.out_stride & 7) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 w;
                                w.x = vm_pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                                w.y = vm_pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                                w.z = vm_pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                                w.w = vm_pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                                *reinterpret_cast<uint4*>(o + j) = w;
                            }
                        } else {
                            for (int j = 0; j < 32 && col0 + j < p.N; ++j) o[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
                        }
                    } else if (p.epi == TC_STORE_F32) {
                        float* o = static_cast<float*>(p.out) + (size_t)row * p.out_stride + col0;
                        for (int j = 0; j < 32 && col0 + j < p.N; ++j) o[j] = __uint_as_float(v[j]);
                    } else {
                        float* o = p.h + (size_t)row * p.N + col0;
                        if (col0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 x = *reinterpret_cast<float4*>(o + j);
                                x.x += __uint_as_float(v[j]); x.y += __uint_as_float(v[j + 1]);
                                x.z += __uint_as_float(v[j + 2]); x.w += __uint_as_float(v[j + 3]);
                                *reinterpret_cast<float4*>(o + j) = x;
                            }
                        } else {
                            for (int j = 0; j < 32 && col0 + j < p.N; ++j) o[j] += __uint_as_float(v[j]);
                        }
                    }
                }
            } else {
                // paired epilogues: column c of the first half belongs with column c of the second half
                int pos = 0, page = -1, head = 0;
                if (p.epi == TC_ROPE_KV) {
                    head = tile_n;
                    if (row_ok) {
                        pos = p.positions[row];
                        if (head >= p.H && p.kpages != nullptr) {
                            const int blk = pos / VM_PAGE_TOKENS;
                            page = (blk < p.max_blocks) ? p.block_table[(size_t)p.seq_of_token[row] * p.max_blocks + blk] : -1;
                            if (page < 0 || page >= p.n_pages) { page = -1; if (p.err) atomicExch(p.err, 2); }
                        }
                    }
                }
#pragma unroll 1
                for (int c0 = 0; c0 < half; c0 += 32) {
                    uint32_t lo[32], hi[32];
                    __syncwarp();                                      // lanes that skipped the last round's stores are back
                    tc_ld32(taddr + c0, lo);
                    tc_ld32(taddr + half + c0, hi);
                    tc_ld_wait();
                    if (!row_ok) continue;
                    if (p.epi == TC_SWIGLU) {
                        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride + n0 + c0;
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            float r2[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const float g = __uint_as_float(lo[j + e]), u = __uint_as_float(hi[j + e]);
                                const float sig = 1.0f / (1.0f + expf(-g));
                                r2[e] = (sig * g) * u;
                            }
                            if (n0 + c0 + j + 1 < p.I) *reinterpret_cast<unsigned*>(o + j) = vm_pack_bf16(r2[0], r2[1]);
                            else if (n0 + c0 + j < p.I) o[j] = __float2bfloat16_rn(r2[0]);
                        }
                    } else {
                        const bool rotate = head < p.H + p.Hkv && p.rot_dim > 0;
                        __nv_bfloat16* dst = nullptr;
                        if (head < p.H) dst = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.out_stride + (size_t)head * p.D;
                        else if (page >= 0) {
                            const bool is_k = head < p.H + p.Hkv;
                            const int hk = is_k ? head - p.H : head - p.H - p.Hkv;
                            dst = (is_k ? p.kpages : p.vpages) + (size_t)page * ((size_t)p.Hkv * VM_PAGE_TOKENS * p.D)
                                  + ((size_t)hk * VM_PAGE_TOKENS + pos % VM_PAGE_TOKENS) * p.D;
                        }
                        if (dst == nullptr) continue;
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            float ya[2], yb[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const float a = __uint_as_float(lo[j + e]), b = __uint_as_float(hi[j + e]);
                                ya[e] = a; yb[e] = b;
                                if (rotate) {
                                    float s, c;
                                    sincosf((float)pos * p.inv_freq[c0 + j + e], &s, &c);
                                    ya[e] = a * c - b * s;
                                    yb[e] = b * c + a * s;
                                }
                            }
                            *reinterpret_cast<unsigned*>(dst + c0 + j) = vm_pack_bf16(ya[0], ya[1]);
                            *reinterpret_cast<unsigned*>(dst + half + c0 + j) = vm_pack_bf16(yb[0], yb[1]);
                        }
                    }
                }
            }
        }
        // this warp has read its part of the accumulator: hand it back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acce0 + 8 * acc) : "memory");
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // this lane's reduce-adds have landed
    }
    // ------------------------------------------------------------ teardown: everyone arrives, then the tensor memory goes back
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && p.err) atomicExch(p.err, 4);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// rows x cols bf16, row pitch `pitch` elements; a box of box_rows x 64 columns, 128-byte swizzle, zeros out of bounds
int make_map(CUtensorMap* map, const void* base, int rows, int cols, long long pitch, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return VM_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch * 2) % 16 != 0) return VM_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VM_ERR_BAD_ARG;
}

template <int BN>
int tc_launch(const void* A, long long lda, const void* W, TcParams p, int tiles_n, int b_box_rows, cudaStream_t stream) {
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, p.M, p.K, lda, TC_BM);
    if (rc) return rc;
    rc = make_map(&mb, W, p.epi == TC_SWIGLU ? 2 * p.I : p.N, p.K, p.K, b_box_rows);
    if (rc) return rc;
    CUtensorMap mh = ma;                                   // a placeholder unless the residual leaves through TMA
    p.tma_residual = 0;
    if (p.epi == TC_RESIDUAL && p.N % 4 == 0 && (reinterpret_cast<uintptr_t>(p.h) & 15) == 0) {
        EncodeTiledFn fn = encode_tiled_fn();
        cuuint64_t dims[2] = {(cuuint64_t)p.N, (cuuint64_t)p.M};
        cuuint64_t strides[1] = {(cuuint64_t)p.N * 4};
        cuuint32_t box[2] = {32, 32};
        cuuint32_t estr[2] = {1, 1};
        if (fn && fn(&mh, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p.h, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            p.tma_residual = 1;
    }
    constexpr int STAGES = 3;
    const size_t smem = (size_t)STAGES * TC_KPS * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 4 * 4096 + 128;   // stages, epilogue staging, barriers
    static bool configured = false;
    static int num_sms = 0;
    static int per_sm = 1;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        int occ = 1;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, tc_gemm_kernel<BN>, TC_THREADS, smem) != cudaSuccess || occ < 1) occ = 1;
        const int by_tmem = 512 / (2 * BN);                // tensor memory: 2 x BN columns per CTA of 512 per SM
        per_sm = occ < by_tmem ? occ : by_tmem;
        if (per_sm > 2) per_sm = 2;
        configured = true;
    }
    p.tiles_n = tiles_n;
    p.tiles_m = (p.M + TC_BM - 1) / TC_BM;
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    const int grid = (int)(tiles < (long long)num_sms * per_sm ? tiles : (long long)num_sms * per_sm);
    tc_gemm_kernel<BN><<<grid, TC_THREADS, smem, stream>>>(ma, mb, mh, p);
    return vm_launch_status();
}

}  // namespace

// out = A W^T (bf16, or float32 when out_f32), or residual_h += A W^T.  A [M, K] bf16 with row pitch lda.
VM_API int vm_tc_linear(const void* A, long long lda, const void* W, int M, int N, int K, void* out, int out_stride,
                        int out_f32, float* residual_h, int* err, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (K % 8 != 0 || N <= 0) return VM_ERR_UNSUPPORTED;
    TcParams p{};
    p.M = M; p.N = N; p.K = K; p.out = out; p.out_stride = out_stride; p.h = residual_h; p.err = err;
    p.epi = residual_h ? TC_RESIDUAL : (out_f32 ? TC_STORE_F32 : TC_STORE_BF16);
    // narrow tiles when wide ones would leave most SMs idle
    const long long tiles128 = (long long)((N + 127) / 128) * ((M + TC_BM - 1) / TC_BM);
    if (tiles128 >= 148) return tc_launch<128>(A, lda, W, p, (N + 127) / 128, 128, stream);
    return tc_launch<64>(A, lda, W, p, (N + 63) / 64, 64, stream);
}

// out[M, I] = silu(A Wg^T) * (A Wu^T); W = [Wg; Wu] is [2I, K].  I must be a multiple of 64.
VM_API int vm_tc_swiglu(const void* A, long long lda, const void* W, int M, int I, int K, void* out, int* err,
                        cudaStream_t stream) {
    if (M <= 0) return 0;
    if (K % 8 != 0 || I % 64 != 0) return VM_ERR_UNSUPPORTED;
    TcParams p{};
    p.M = M; p.N = 2 * I; p.K = K; p.out = out; p.out_stride = I; p.I = I; p.epi = TC_SWIGLU; p.err = err;
    return tc_launch<128>(A, lda, W, p, I / 64, 64, stream);
}

// One head per tile: q_out[M, H*D] = rope(A Wq^T); rope(A Wk^T) and A Wv^T go to the cache pages.  D is 64 or 128,
// rot_dim 0 or D; half-split pairing only (another pairing is refused: the caller takes the unfused path).
VM_API int vm_tc_qkv_rope(const void* A, long long lda, const void* W, int M, int K, void* q_out, const int* positions,
                          const int* seq_of_token, const int* block_table, int max_blocks, const float* inv_freq,
                          int rot_dim, int pairing, void* kpages, void* vpages, int H, int Hkv, int D, int n_pages, int* err,
                          cudaStream_t stream) {
    if (M <= 0) return 0;
    if (rot_dim > 0 && pairing != VM_PAIR_HALF_SPLIT) return VM_ERR_UNSUPPORTED;
    if (K % 8 != 0 || !(D == 64 || D == 128) || !(rot_dim == 0 || rot_dim == D) || (rot_dim > 0 && inv_freq == nullptr))
        return VM_ERR_UNSUPPORTED;
    TcParams p{};
    p.M = M; p.N = (H + 2 * Hkv) * D; p.K = K; p.out = q_out; p.out_stride = H * D; p.epi = TC_ROPE_KV; p.err = err;
    p.positions = positions; p.seq_of_token = seq_of_token; p.block_table = block_table; p.max_blocks = max_blocks;
    p.inv_freq = inv_freq; p.rot_dim = rot_dim; p.kpages = (__nv_bfloat16*)kpages; p.vpages = (__nv_bfloat16*)vpages;
    p.H = H; p.Hkv = Hkv; p.D = D; p.n_pages = n_pages;
    if (D == 64) return tc_launch<64>(A, lda, W, p, H + 2 * Hkv, 64, stream);
    return tc_launch<128>(A, lda, W, p, H + 2 * Hkv, 128, stream);
}
