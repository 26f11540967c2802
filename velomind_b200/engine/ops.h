// ops.h (internal) — the device operations the parts are made of: checked wrappers over the CUDA launchers and the
// library matrix product.  There is no other implementation: a missing device or a refused launch throws.
//
// Debugging switches, read once from the environment (the reference has VELOMIND_CUDA_SYNC and VELOMIND_FAIL_BACKEND for
// the same purposes: src/cuda/cuda_context.cu:115-118, src/cuda/ops/backend_error.h:31-51); both act on the host only:
//   VELOMIND_B200_SYNC=1        wait for the device after every launch, so that a CUDA error names the operation
//   VELOMIND_B200_FAIL_OP=name  the operation of that name throws after its launch (fault injection)
#pragma once

#include <cublas_v2.h>

#include <string>

#include "velomind_b200/kernels.h"
#include "velomind_b200/velomind.h"

namespace vmb {
namespace ops {

struct Counters {
    long long own_launches = 0;     // this library's own kernels
    long long library_calls = 0;    // library matrix products (cuBLAS)
    long long h2d_bytes = 0;        // bytes of step inputs copied from pinned host memory
    long long d2h_bytes = 0;        // bytes of step results that reached the host
    long long tc_attention_calls = 0;
};
Counters& counters();

// per-operation device time (two events around every launch), switched on by OpTimes
struct OpTimes {
    OpTimes();
    ~OpTimes();
    std::string table();            // name, launches, milliseconds; the events are read here (synchronises)
};
bool op_times_active();
void op_time_begin(const char* name, cudaStream_t stream);
void op_time_end(const char* name, cudaStream_t stream);

bool sync_every_op();
void check(int status, const char* name, cudaStream_t stream);      // counts the launch; throws KernelError on a refusal
void cuda_check(cudaError_t e, const char* what);

inline int code(DType t) {
    if (t == DType::F32) return VM_F32;
    if (t == DType::BF16) return VM_BF16;
    throw KernelError(std::string("dtype ") + dtype_name(t) + " has no kernel (float32 and bfloat16 do)");
}

struct Timed {                      // brackets one launch with events when op times are on
    const char* name;
    cudaStream_t stream;
    Timed(const char* n, cudaStream_t s) : name(n), stream(s) { if (op_times_active()) op_time_begin(n, s); }
    ~Timed() { if (op_times_active()) op_time_end(name, stream); }
};

inline void embed_gather(const DeviceTensor& table, const int* tokens, float* out, int T, int hid, int* err, cudaStream_t s) {
    Timed t("embed_gather", s);
    check(vm_embed_gather(table.ptr, code(table.dtype), tokens, out, T, hid, static_cast<int>(table.rows()), err, s), "embed_gather", s);
}

inline void add_rmsnorm(float* h, const void* delta, const float* weight, float eps, void* out, const int* rows, int n_out, int hid, DType act,
                        cudaStream_t s) {
    Timed t("add_rmsnorm", s);
    check(vm_add_rmsnorm(h, delta, weight, out, rows, n_out, hid, eps, code(act), s), "add_rmsnorm", s);
}

inline void residual_add(float* h, const void* delta, long long n, DType act, cudaStream_t s) {
    Timed t("residual_add", s);
    check(vm_residual_add(h, delta, n, code(act), s), "residual_add", s);
}

inline void swiglu(const void* gate_up, void* out, int T, int I, DType act, cudaStream_t s) {
    Timed t("swiglu", s);
    check(vm_swiglu(gate_up, out, T, I, code(act), s), "swiglu", s);
}

inline void convert(const void* in, DType in_dtype, void* out, DType out_dtype, long long n, cudaStream_t s) {
    Timed t("convert", s);
    check(vm_convert(in, code(in_dtype), out, code(out_dtype), n, s), "convert", s);
}

inline void rope_kv_write(void* qkv, const StepContext& ctx, const KVView& kv, const RotaryTable& rot, int H, int Hkv, int D, DType act) {
    Timed t("rope_kv_write", ctx.stream);
    check(vm_rope_kv_write(qkv, ctx.positions, ctx.seq_of_token, kv.block_table, kv.table_width, rot.inv_freq, rot.rotary_dim, rot.pairing,
                           kv.owns ? kv.k_pages : nullptr, kv.owns ? kv.v_pages : nullptr, ctx.T, H, Hkv, D, kv.owns ? kv.n_pages : 0, code(act),
                           ctx.err, ctx.stream),
          "rope_kv_write", ctx.stream);
}

// out = x W^T.  x [T, K] (row stride ldx), W [N, K], out [T, N]; a library matrix product, as in the reference
// (src/cuda/ops/matmul.cu:87-126); float32 runs without any reduced-precision mode.
void linear(const void* x, DType x_dtype, long long ldx, const DeviceTensor& W, void* out, DType out_dtype, int T, cudaStream_t s);
// h[T, N] += x W^T with the float32 residual stream h as the product's own accumulator (x and W bfloat16): the sum happens in
// the library's float32 epilogue, and the kernel after it reads h alone.
void linear_residual(const void* x, long long ldx, const DeviceTensor& W, float* h, int T, cudaStream_t s);

// attention of the step's tokens over the cache; picks the kernel for the step's shape and dtype
void attention(StepContext& ctx, const void* q, int q_row_stride, const KVView& kv, void* out, int H, int Hkv, int D, float scale, int window);

// the weight-streaming products for few rows (bfloat16 weights)
extern int SKINNY_MAX_ROWS;        // beyond this many rows the library product takes over
extern int SKINNY_NORM_ROWS;       // up to this many rows the norm is fused into the product that follows it
extern int SKINNY_HEAD_MAX_ROWS;   // up to this many rows the head streams its table with the weight-streaming kernels
extern int SKINNY_MAX_ROWS_LARGE;  // the same limit for a part whose largest weight matrix has SKINNY_LARGE_WEIGHT_BYTES and more
extern long long SKINNY_LARGE_WEIGHT_BYTES;
// rows (of a step's capacity) up to which the weight-streaming kernels take a part whose largest weight matrix has `weight_bytes`
inline int skinny_max_rows(long long weight_bytes) {
    return weight_bytes >= SKINNY_LARGE_WEIGHT_BYTES && SKINNY_MAX_ROWS_LARGE < SKINNY_MAX_ROWS ? SKINNY_MAX_ROWS_LARGE : SKINNY_MAX_ROWS;
}
inline bool skinny_ok(int M, long long K, const DeviceTensor& W) { return M > 0 && M <= SKINNY_MAX_ROWS && K % 32 == 0 && W.dtype == DType::BF16; }

inline void skinny_linear(const void* x, const float* norm_w, float eps, const DeviceTensor& W, int M, void* out, int out_stride, bool out_f32,
                          float* residual, int* err, cudaStream_t s) {
    Timed t("skinny_linear", s);
    check(vm_skinny_linear(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, M, static_cast<int>(W.rows()), static_cast<int>(W.cols()), out, out_stride,
                           out_f32 ? 1 : 0, residual, err, s),
          "skinny_linear", s);
}

inline void skinny_swiglu(const void* x, const float* norm_w, float eps, const DeviceTensor& W, int M, int I, void* out, int* err, cudaStream_t s) {
    Timed t("skinny_swiglu", s);
    check(vm_skinny_swiglu(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, M, I, static_cast<int>(W.cols()), out, err, s), "skinny_swiglu", s);
}

inline void skinny_qkv_rope(const void* x, const float* norm_w, float eps, const DeviceTensor& W, void* q_out, const StepContext& ctx, const KVView& kv,
                            const RotaryTable& rot, int H, int Hkv, int D) {
    Timed t("skinny_qkv_rope", ctx.stream);
    check(vm_skinny_qkv_rope(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, ctx.T, static_cast<int>(W.cols()), q_out, ctx.positions, ctx.seq_of_token,
                             kv.block_table, kv.table_width, rot.inv_freq, rot.rotary_dim, rot.pairing, kv.owns ? kv.k_pages : nullptr,
                             kv.owns ? kv.v_pages : nullptr, H, Hkv, D, kv.owns ? kv.n_pages : 0, ctx.err, ctx.stream),
          "skinny_qkv_rope", ctx.stream);
}

// the tcgen05 + TMA products for many rows
inline bool tc_fused_rows(const StepContext& ctx) { return ctx.fused_prefill_rows > 0 && ctx.T_cap >= ctx.fused_prefill_rows; }

inline void tc_linear(const void* x, long long ldx, const DeviceTensor& W, int M, void* out, int out_stride, bool out_f32, float* residual, int* err,
                      cudaStream_t s) {
    Timed t("tc_linear", s);
    check(vm_tc_linear(x, ldx, W.ptr, M, static_cast<int>(W.rows()), static_cast<int>(W.cols()), out, out_stride, out_f32 ? 1 : 0, residual, err, s),
          "tc_linear", s);
}

inline void tc_swiglu(const void* x, long long ldx, const DeviceTensor& W, int M, int I, void* out, int* err, cudaStream_t s) {
    Timed t("tc_swiglu", s);
    check(vm_tc_swiglu(x, ldx, W.ptr, M, I, static_cast<int>(W.cols()), out, err, s), "tc_swiglu", s);
}

inline void tc_qkv_rope(const void* x, long long ldx, const DeviceTensor& W, void* q_out, const StepContext& ctx, const KVView& kv,
                        const RotaryTable& rot, int H, int Hkv, int D) {
    Timed t("tc_qkv_rope", ctx.stream);
    check(vm_tc_qkv_rope(x, ldx, W.ptr, ctx.T, static_cast<int>(W.cols()), q_out, ctx.positions, ctx.seq_of_token, kv.block_table, kv.table_width,
                         rot.inv_freq, rot.rotary_dim, rot.pairing, kv.owns ? kv.k_pages : nullptr, kv.owns ? kv.v_pages : nullptr, H, Hkv, D,
                         kv.owns ? kv.n_pages : 0, ctx.err, ctx.stream),
          "tc_qkv_rope", ctx.stream);
}

inline void sample(const float* logits, long long row_stride, int R, int V, const float* temperature, const float* top_p, const long long* seed,
                   const long long* stream_id, const long long* step, long long step_add, int* out, cudaStream_t s) {
    Timed t("sample", s);
    check(vm_sample(logits, row_stride, R, V, temperature, top_p, seed, stream_id, step, step_add, out, s), "sample", s);
}

inline void decode_advance(const int* sampled, int* tokens, int* positions, int* ctx_len, long long* draw_step, int* history, int* iteration, int B,
                           cudaStream_t s) {
    Timed t("decode_advance", s);
    check(vm_decode_advance(sampled, tokens, positions, ctx_len, draw_step, history, iteration, B, s), "decode_advance", s);
}

int sm_count();                     // streaming multiprocessors of the current device, asked once

}  // namespace ops
}  // namespace vmb
