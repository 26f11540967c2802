// Weight-streaming matrix products for few rows (M <= 64: decode steps and other small steps), bfloat16,
// with the neighbouring elementwise work fused in so that a decode layer is five launches:
//
//   prologue   none      A is bf16 [M, K]
//              rmsnorm   A = rmsnorm(h) * w from the float32 residual h [M, K] (src/cpu/ops/rmsnorm.cpp:42-59);
//                        h * w is staged as bf16 and the row's 1/rms multiplies the float32 sums afterwards
//   epilogue   store     out[M, N] = A W^T            (bf16, or float32 for logits)
//              residual  h[M, N] += A W^T             (float32 residual stream; llama_graph.cpp:225-226,137)
//              swiglu    out[M, I] = silu(A Wg^T) * (A Wu^T), W = [Wg; Wu] stacked (llama_graph.cpp:22-28)
//              rope_kv   W = [Wq; Wk; Wv] stacked: rotate q and k (rotary_embedding.cpp:30-44), write q to
//                        out [M, H*D], k and v into the paged cache (llama_graph.cpp:210-215)
//
// y = x W^T with W [N, K] row-major (K contiguous).  Every weight byte is read once per step, so the kernel
// is organised around the weight stream: a CTA owns 8 or 16 output columns, its eight warps split K, and
// each thread fetches 16 contiguous bytes of a weight row per 32-wide k block straight from global memory
// into the B fragments of two mma.sync m16n8k16 (bf16 in, float32 accumulate).  The k indices inside a
// block are permuted the same way for A and B, which leaves the dot product unchanged and makes the
// 16-byte loads possible.  A (at most 64 rows) sits in shared memory; when a product has more column tiles than the
// GPU holds CTAs and all of K fits the tile, a CTA takes several tiles one after another with A staged once.
// Under programmatic dependent launch the kernel requests its first weight blocks (and the rotary frequencies) before
// it waits for its predecessor; the rope_kv form lets ITS successor, the decode attention, start only after that wait
// (common.cuh says why).
//
// Products that read many megabytes of weights for at most 32 rows take skinny_stream_kernel (skinny_stream.cuh): the same
// work items and epilogues, the weights streamed through shared memory by a warp of their own.
//
// Sizes: K % 32 == 0, N % 8 == 0 (16 for the two-tile forms), head size % 16 == 0, I % 8 == 0; M <= 64.
// Anything else is refused with VM_ERR_UNSUPPORTED and the caller uses the library product.
#include "skinny_body.cuh"
#include "skinny_stream.cuh"

namespace {

using namespace vmsk;

// (two CTAs per SM for up to 16 rows, and for up to 32 rows when K is at most 1,024: 192 gate/up items then fit the GPU at once)
// (PF: weight blocks a warp keeps in flight; 4 cover K <= 1,024 in one round and leave registers to the prologue)
// (LOOP: a CTA takes several work items one after another; without it the grid has a CTA per item)
template <int MT, int PF, bool LOOP>
__global__ void __launch_bounds__(SK_THREADS, (MT == 1 || (MT == 2 && PF == 4)) ? 2 : 1)
skinny_gemm_kernel(const SkinnyParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    skinny_run<MT, true, PF, LOOP>(p, blockIdx.x, gridDim.x, p.n_items, smem);
}

template <int MT>
__global__ void __launch_bounds__(SK_THREADS)
skinny_wide_kernel(const SkinnyParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    skinny_wide_body<MT, true>(p, blockIdx.x, smem);
}

int skinny_wide_launch(SkinnyParams p, cudaStream_t stream) {
    if (p.M <= 0) return 0;
    if (p.M > 64 || p.K % 32 != 0 || p.K <= 0 || p.N % 8 != 0) return VM_ERR_UNSUPPORTED;
    const int mt = (p.M + 15) / 16;
    const int MT = mt <= 1 ? 1 : (mt <= 2 ? 2 : 4);
    const int rows = 16 * MT;
    int pitch = p.K * 2;
    pitch += ((64 - pitch % 128) + 128) % 128;
    p.row_bytes = pitch;
    const size_t smem = (size_t)rows * pitch;
    if (smem > 200 * 1024) return VM_ERR_UNSUPPORTED;
    const int grid = (p.N / 8 + SK_WARPS - 1) / SK_WARPS;
#define VM_SKW_CASE(X)                                                                                                \
    case X: {                                                                                                         \
        static size_t configured = 0;                                                                                 \
        if (smem > 48 * 1024 && smem > configured) {                                                                  \
            cudaError_t e = cudaFuncSetAttribute(skinny_wide_kernel<X>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e;                                                                      \
            configured = 200 * 1024;                                                                                  \
        }                                                                                                             \
        vm_launch_pdl(skinny_wide_kernel<X>, dim3(grid), dim3(SK_THREADS), smem, stream, p);                          \
    } break;
    switch (MT) { VM_SKW_CASE(1) VM_SKW_CASE(2) VM_SKW_CASE(4) }
#undef VM_SKW_CASE
    return vm_launch_status();
}

int skinny_launch(SkinnyParams p, int grid, cudaStream_t stream) {
    if (p.M <= 0 || grid <= 0) return 0;
    if (p.M > 64 || p.K % 32 != 0 || p.K <= 0) return VM_ERR_UNSUPPORTED;
    const int mt = (p.M + 15) / 16;
    const int MT = mt <= 1 ? 1 : (mt <= 2 ? 2 : 4);
    const int rows = 16 * MT;
    // A chunk in shared memory: at most ~96 KB, rows of kc bf16 plus padding to a pitch == 64 (mod 128) bytes
    int kc = p.K;
    const int cap = (96 * 1024) / (rows * 2) / 128 * 128;
    if (kc > cap) kc = cap;
    p.kc = kc;
    int pitch = kc * 2;
    pitch += ((64 - pitch % 128) + 128) % 128;
    p.row_bytes = pitch;
    const size_t smem = (size_t)rows * pitch + (size_t)SK_WARPS * rows * 16 * sizeof(float) + rows * sizeof(float);
    // all of K in shared memory: as many CTAs as the GPU holds at once, each staging A once and taking its share of the
    // items one after another; else one CTA per item
    p.n_items = grid;
    if (p.K <= kc) {
        static int sms = 0;
        if (sms == 0) {
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 1;
        }
        const int resident = sms * (((MT == 1 || (MT == 2 && kc <= SK_WARPS * 32 * 4)) && 2 * smem + 2048 <= 227 * 1024) ? 2 : 1);
        const int per_cta = (grid + resident - 1) / resident;
        grid = (grid + per_cta - 1) / per_cta;
    }
    const bool loop = grid < p.n_items;
    const bool few = kc <= SK_WARPS * 32 * 4;
#define VM_SK_CASE(X, P, L)                                                                                           \
    {                                                                                                                 \
        static size_t configured = 0;                                                                                 \
        if (smem > 48 * 1024 && smem > configured) {                                                                  \
            cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<X, P, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); \
            if (e != cudaSuccess) return (int)e;                                                                      \
            configured = 160 * 1024;                                                                                  \
        }                                                                                                             \
        vm_launch_pdl(skinny_gemm_kernel<X, P, L>, dim3(grid), dim3(SK_THREADS), smem, stream, p);                    \
    }
#define VM_SK_ROWS(X)                                                                                                 \
    if (few) { if (loop) VM_SK_CASE(X, 4, true) else VM_SK_CASE(X, 4, false) }                                        \
    else { if (loop) VM_SK_CASE(X, 8, true) else VM_SK_CASE(X, 8, false) }
    switch (MT) {
        case 1: VM_SK_ROWS(1) break;
        case 2: VM_SK_ROWS(2) break;
        case 4: VM_SK_ROWS(4) break;
    }
#undef VM_SK_ROWS
#undef VM_SK_CASE
    return vm_launch_status();
}

// Which kernel takes a product of `items` work items: the streaming one when the weights are large enough for memory
// bandwidth, not one chain of latencies, to set the time (measured at hidden sizes 960 and 2,048 against 576: from 9 MB, and
// from 4.5 MB for one or two rows: the down projection at hidden 960, 4.9 MB, takes 4.9 / 5.0 / 5.1 us at 1 / 2 / 4 rows in the
// register-fed kernel and 3.9 / 4.5 / 4.9 us in this one), or when
// vm_skinny_variant() asks for it.
int skinny_variant = 0;
constexpr long long STREAM_MIN_WEIGHT_BYTES = 9ll << 20;
constexpr long long STREAM_MIN_WEIGHT_BYTES_TWO_ROWS = 9ll << 19;      // 4.5 MB: with one or two rows there is next to no prologue

int skinny_dispatch(SkinnyParams p, int items, cudaStream_t stream) {
    const long long weight_bytes = (long long)p.N * p.K * 2;
    if (skinny_variant >= 2 || (skinny_variant == 0 && p.M <= 32 && weight_bytes >= (p.M <= 2 ? STREAM_MIN_WEIGHT_BYTES_TWO_ROWS : STREAM_MIN_WEIGHT_BYTES))) {
        const int rc = skinny_stream_launch(p, items, stream, skinny_variant == 3 ? 2 : (skinny_variant == 4 ? 1 : 0));
        if (rc != VM_ERR_UNSUPPORTED || skinny_variant >= 2) return rc;
    }
    return skinny_launch(p, items, stream);
}

}  // namespace

// 0: the launchers choose between the two weight-streaming kernels by size; 1: always skinny_gemm_kernel; 2: always
// skinny_stream_kernel (VM_ERR_UNSUPPORTED where it does not take the sizes); 3 / 4: the same in its form of one CTA with two
// pipelines per SM / of two CTAs per SM.  For tests and measurements.
VM_API void vm_skinny_variant(int variant) { skinny_variant = variant; }

// out = A W^T (pro 0) or rmsnorm(h) W^T (pro 1); out bf16 (out_f32 0) or float32 (1); or h += ... (residual 1).
VM_API int vm_skinny_linear(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int N, int K,
                            void* out, int out_stride, int out_f32, float* residual_h, int* err, cudaStream_t stream) {
    if (N % 8 != 0) return VM_ERR_UNSUPPORTED;
    SkinnyParams p{};
    p.err = err;
    p.A = A; p.pro = pro; p.norm_w = norm_w; p.eps = eps; p.W = (const __nv_bfloat16*)W; p.M = M; p.N = N; p.K = K;
    p.out = out; p.out_stride = out_stride; p.h = residual_h;
    p.epi = residual_h ? EPI_RESIDUAL : (out_f32 ? EPI_STORE_F32 : EPI_STORE_BF16);
    p.tiles = (N % 16 == 0 && N / 16 >= 148) ? 2 : 1;
    const int items = p.tiles == 2 ? N / 16 : N / 8;
    if (skinny_variant < 2 && pro == PRO_NONE && !residual_h && N >= 4096 && (size_t)((M + 15) / 16 * 16) * (K * 2 + 128) <= 200 * 1024) {
        // many columns (the vocabulary head): warps split N, not K; from K = 768 on the ring kernel is faster (49,152 columns,
        // 8 rows, K = 576 / 960 / 2,048: 13.0 / 20.7 / 48.5 us against 16.3 / 18.6 / 32.6 us)
        if (skinny_variant == 0 && M <= 32 && K >= 768) {
            const int rc = skinny_stream_launch(p, items, stream);
            if (rc != VM_ERR_UNSUPPORTED) return rc;
        }
        return skinny_wide_launch(p, stream);
    }
    return skinny_dispatch(p, items, stream);
}

// out[M, I] = silu(x Wg^T) * (x Wu^T) with x = A (pro 0) or rmsnorm(h) (pro 1); W = [Wg; Wu] is [2I, K].
VM_API int vm_skinny_swiglu(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int I, int K,
                            void* out, int* err, cudaStream_t stream) {
    if (I % 8 != 0) return VM_ERR_UNSUPPORTED;
    SkinnyParams p{};
    p.err = err;
    p.A = A; p.pro = pro; p.norm_w = norm_w; p.eps = eps; p.W = (const __nv_bfloat16*)W; p.M = M; p.N = 2 * I; p.K = K;
    p.out = out; p.out_stride = I; p.I = I; p.epi = EPI_SWIGLU; p.tiles = 2;
    return skinny_dispatch(p, I / 8, stream);
}

// q_out[M, H*D] = rope(x Wq^T); rope(x Wk^T) and x Wv^T go to the cache pages; W = [Wq; Wk; Wv] is [(H+2Hkv)*D, K].
// rot_dim must be 0 (no rotation) or D, the pairing half-split (another pairing is refused with VM_ERR_UNSUPPORTED: the
// caller then takes the unfused product followed by vm_rope_kv_write, which rotates either pairing).  kpages == nullptr:
// nothing is cached.
VM_API int vm_skinny_qkv_rope(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int K,
                              void* q_out, const int* positions, const int* seq_of_token, const int* block_table,
                              int max_blocks, const float* inv_freq, int rot_dim, int pairing, void* kpages, void* vpages, int H, int Hkv,
                              int D, int n_pages, int* err, cudaStream_t stream) {
    if (D % 16 != 0 || !(rot_dim == 0 || rot_dim == D) || (rot_dim > 0 && inv_freq == nullptr)) return VM_ERR_UNSUPPORTED;
    if (rot_dim > 0 && pairing != VM_PAIR_HALF_SPLIT) return VM_ERR_UNSUPPORTED;
    SkinnyParams p{};
    p.A = A; p.pro = pro; p.norm_w = norm_w; p.eps = eps; p.W = (const __nv_bfloat16*)W; p.M = M; p.N = (H + 2 * Hkv) * D; p.K = K;
    p.out = q_out; p.out_stride = H * D; p.epi = EPI_ROPE_KV; p.tiles = 2;
    p.positions = positions; p.seq_of_token = seq_of_token; p.block_table = block_table; p.max_blocks = max_blocks;
    p.inv_freq = inv_freq; p.rot_dim = rot_dim; p.kpages = (__nv_bfloat16*)kpages; p.vpages = (__nv_bfloat16*)vpages;
    p.H = H; p.Hkv = Hkv; p.D = D; p.n_pages = n_pages; p.err = err;
    return skinny_dispatch(p, (H + 2 * Hkv) * (D / 16), stream);
}
