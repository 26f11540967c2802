// kernels.h — every launcher of the CUDA kernel library (csrc/*.cu), as plain C declarations.
//
// The kernels are compiled for sm_100a.  Each launcher enqueues work on `stream` and returns at once:
// 0 on success, VM_ERR_UNSUPPORTED (-1) for a size or dtype the kernel does not take, VM_ERR_BAD_ARG (-2)
// for an argument that contradicts another, or a positive cudaError_t.  Pointers are device pointers
// unless a comment says otherwise.  `err` is an optional device int that kernels set to an error word
// (see VM_ERRWORD_*) instead of faulting; 0 means nothing happened.
//
// Activations are float32 or bfloat16 (`act_dtype`: VM_F32 / VM_BF16); the residual stream and all logits
// are float32.  The cache is paged: k/v pages are [n_pages, Hkv, VM_PAGE_TOKENS, D]; a block table
// int32 [B, max_blocks] names the page of every VM_PAGE_TOKENS-token block of each sequence (-1: none).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { VM_F32 = 0, VM_BF16 = 1 };
enum { VM_ERR_UNSUPPORTED = -1, VM_ERR_BAD_ARG = -2 };
// tokens per cache page: the one constant that the host's page bookkeeping and the kernels share
#define VM_PAGE_TOKENS 64
// which two values of a head a rotary position encoding turns together: (j, j + rot_dim/2) or (2j, 2j + 1)
enum { VM_PAIR_HALF_SPLIT = 0, VM_PAIR_INTERLEAVED = 1 };
// error words a kernel may leave in `err`
enum { VM_ERRWORD_TOKEN_ID = 1, VM_ERRWORD_CACHE_WRITE = 2, VM_ERRWORD_CACHE_READ = 3, VM_ERRWORD_BARRIER_WAIT = 4 };

// ---- elementwise.cu
void vm_set_pdl(int on);                      // programmatic dependent launch for the decode chain (default on)
int vm_embed_gather(const void* table, int table_dtype, const int* tokens, float* out, int T, int hid, int vocab, int* err,
                    cudaStream_t stream);
int vm_add_rmsnorm(float* h, const void* delta, const float* w, void* out, const int* rows, int n_out, int hid, float eps,
                   int act_dtype, cudaStream_t stream);
int vm_residual_add(float* h, const void* delta, long long n, int act_dtype, cudaStream_t stream);
int vm_swiglu(const void* gate_up, void* out, int T, int I, int act_dtype, cudaStream_t stream);
int vm_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream);

// ---- rope_cache.cu
int vm_rope_kv_write(void* qkv, const int* positions, const int* seq_of_token, const int* block_table, int max_blocks,
                     const float* inv_freq, int rot_dim, int pairing, void* kpages, void* vpages, int T, int H, int Hkv, int D,
                     int n_pages, int act_dtype, int* err, cudaStream_t stream);

// ---- attention
int vm_attention_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                         int max_blocks, const int* positions, const int* seq_of_token, void* out, int n_tokens, int H, int Hkv,
                         int D, float scale, int window, int n_pages, int act_dtype, int* err, cudaStream_t stream);
int vm_attention_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                              int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, void* out, int H,
                              int Hkv, int D, float scale, int window, int n_pages, int* err, int groups, cudaStream_t stream);
int vm_attention_prefill_tc_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                 int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, void* out, int H,
                                 int Hkv, int D, float scale, int window, int n_pages, int* err, int groups, cudaStream_t stream);
// the warp-specialised tcgen05 kernel: host_cu_tokens [B + 1] (host memory) repeats cu_tokens, the launch is shaped from it
int vm_attention_prefill_ws_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                 int max_blocks, const int* positions, const int* cu_tokens, const int* host_cu_tokens, int B,
                                 void* out, int H, int Hkv, int D, float scale, int window, int n_pages, int* err, int groups,
                                 cudaStream_t stream);
long long vm_attention_decode_scratch_floats(int B, int H, int D, int n_splits);
int vm_attention_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                             int max_blocks, const int* positions, void* out, float* partial, int* counters, int B, int H,
                             int Hkv, int D, int n_splits, float scale, int window, int n_pages, int* err, cudaStream_t stream);

// ---- skinny_gemm.cu: weight-streaming products for few rows (bfloat16 weights [N, K])
// (err: the step's error word, may be null; the kernel for large weight matrices reports a wait that ran out there)
int vm_skinny_linear(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int N, int K, void* out,
                     int out_stride, int out_f32, float* residual_h, int* err, cudaStream_t stream);
int vm_skinny_swiglu(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int I, int K, void* out,
                     int* err, cudaStream_t stream);
void vm_skinny_variant(int variant);       // 0 choose by size, 1 / 2 force one of the two kernels (tests, measurements)
int vm_skinny_qkv_rope(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int K, void* q_out,
                       const int* positions, const int* seq_of_token, const int* block_table, int max_blocks,
                       const float* inv_freq, int rot_dim, int pairing, void* kpages, void* vpages, int H, int Hkv, int D,
                       int n_pages, int* err, cudaStream_t stream);

// ---- tc_gemm.cu: tcgen05 + TMA products for many rows, with fused epilogues
int vm_tc_linear(const void* A, long long lda, const void* W, int M, int N, int K, void* out, int out_stride, int out_f32,
                 float* residual_h, int* err, cudaStream_t stream);
int vm_tc_swiglu(const void* A, long long lda, const void* W, int M, int I, int K, void* out, int* err, cudaStream_t stream);
int vm_tc_qkv_rope(const void* A, long long lda, const void* W, int M, int K, void* q_out, const int* positions,
                   const int* seq_of_token, const int* block_table, int max_blocks, const float* inv_freq, int rot_dim,
                   int pairing, void* kpages, void* vpages, int H, int Hkv, int D, int n_pages, int* err, cudaStream_t stream);

// ---- sampling.cu
int vm_sample(const float* logits, long long row_stride, int R, int V, const float* temperature, const float* top_p,
              const long long* seed, const long long* stream_id, const long long* step, long long step_add, int* out,
              cudaStream_t stream);
int vm_decode_advance(const int* sampled, int* tokens, int* positions, int* ctx_len, long long* draw_step, int* history,
                      int* iteration, int B, cudaStream_t stream);

// ---- host_transfer.cu (no kernels)
void* vm_host_device_pointer(void* host);     // the address under which kernels reach pinned host memory, or null
void* vm_event_create(void);
int vm_event_destroy(void* event);
int vm_event_synchronize(void* event);
int vm_upload_record(void* dst, const void* src, long long nbytes, void* event, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
