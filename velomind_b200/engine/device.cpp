// Device memory, the checked launch wrappers' common parts, the library matrix product and the attention dispatch.
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "ops.h"

namespace vmb {

// ------------------------------------------------------------------------------------------------ memory
namespace ops {
void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw KernelError(format("%s: CUDA error %d (%s)", what, static_cast<int>(e), cudaGetErrorString(e)));
}
}  // namespace ops

namespace {
// The stream that clears new buffers, one per device.  A buffer must be clear BEFORE its constructor returns: the engine's
// streams are non-blocking, so nothing orders their work after a clearing put on the default stream, and a late clearing would
// wipe what a step has meanwhile copied into the buffer (a bucket's first descriptors, for one).
cudaStream_t clearing_stream() {
    static cudaStream_t per_device[64] = {};
    int dev = 0;
    ops::cuda_check(cudaGetDevice(&dev), "asking for the current device");
    cudaStream_t& s = per_device[dev < 0 || dev >= 64 ? 0 : dev];
    if (!s) ops::cuda_check(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "creating the stream that clears new buffers");
    return s;
}
}  // namespace

DeviceBuffer::DeviceBuffer(size_t n, bool zero) : bytes(n) {
    if (n == 0) return;
    ops::cuda_check(cudaMalloc(&ptr, n), "allocating device memory");
    if (zero) {
        cudaStream_t s = clearing_stream();
        ops::cuda_check(cudaMemsetAsync(ptr, 0, n, s), "clearing device memory");
        ops::cuda_check(cudaStreamSynchronize(s), "clearing device memory");
    }
}

DeviceBuffer::~DeviceBuffer() {
    if (ptr) cudaFree(ptr);
}

PinnedBuffer::PinnedBuffer(size_t n) : bytes(n) {
    if (n == 0) return;
    ops::cuda_check(cudaHostAlloc(&ptr, n, cudaHostAllocMapped), "allocating page-locked host memory");
    std::memset(ptr, 0, n);
}

PinnedBuffer::~PinnedBuffer() {
    if (ptr) cudaFreeHost(ptr);
}

int require_cuda(const std::string& device) {
    int index = 0;
    if (device == "cuda") index = 0;
    else if (device.rfind("cuda:", 0) == 0) index = std::atoi(device.c_str() + 5);
    else throw KernelError(format("device %s refused: this library has CUDA kernels only and no CPU fallback", device.c_str()));
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        throw KernelError("no CUDA device is available; this library has no CPU fallback");
    }
    if (index < 0 || index >= n) throw KernelError(format("device %s does not exist (%d CUDA device%s)", device.c_str(), n, n == 1 ? "" : "s"));
    ops::cuda_check(cudaSetDevice(index), "selecting the device");
    return index;
}

// ------------------------------------------------------------------------------------------------ BindContext
namespace {
// host-side conversion of a stored tensor to the dtype it is kept in on the device
std::vector<uint8_t> converted(const HostTensor& t, DType as) {
    const long long n = t.numel();
    std::vector<uint8_t> out(static_cast<size_t>(n) * dtype_size(as));
    auto read_float = [&](long long i) -> float {
        switch (t.dtype) {
            case DType::F32: { float f; std::memcpy(&f, t.data + 4 * i, 4); return f; }
            case DType::BF16: { uint16_t h; std::memcpy(&h, t.data + 2 * i, 2); return bf16_to_float(h); }
            case DType::F16: { uint16_t h; std::memcpy(&h, t.data + 2 * i, 2); return f16_to_float(h); }
            default: throw WeightError("an integer tensor cannot be kept as floating point");
        }
    };
    auto read_int = [&](long long i) -> long long {
        switch (t.dtype) {
            case DType::I64: { long long v; std::memcpy(&v, t.data + 8 * i, 8); return v; }
            case DType::I32: { int v; std::memcpy(&v, t.data + 4 * i, 4); return v; }
            case DType::I16: { int16_t v; std::memcpy(&v, t.data + 2 * i, 2); return v; }
            case DType::I8: return static_cast<int8_t>(t.data[i]);
            case DType::U8: case DType::BOOL: return t.data[i];
            default: throw WeightError("a floating-point tensor cannot be kept as an integer table");
        }
    };
    if (as == DType::F32)
        for (long long i = 0; i < n; ++i) { const float f = read_float(i); std::memcpy(out.data() + 4 * i, &f, 4); }
    else if (as == DType::BF16)
        for (long long i = 0; i < n; ++i) { const uint16_t h = float_to_bf16(read_float(i)); std::memcpy(out.data() + 2 * i, &h, 2); }
    else if (as == DType::I32)
        for (long long i = 0; i < n; ++i) { const int v = static_cast<int>(read_int(i)); std::memcpy(out.data() + 4 * i, &v, 4); }
    else throw WeightError(std::string("weights are kept as float32, bfloat16 or int32 on the device, not ") + dtype_name(as));
    return out;
}

void copy_in(void* dst, const HostTensor& t, DType as, cudaStream_t stream) {
    if (t.nbytes == 0) return;
    if (t.dtype == as) {
        ops::cuda_check(cudaMemcpyAsync(dst, t.data, t.nbytes, cudaMemcpyHostToDevice, stream), "uploading a weight");
        ops::cuda_check(cudaStreamSynchronize(stream), "uploading a weight");
        return;
    }
    const std::vector<uint8_t> bytes = converted(t, as);
    ops::cuda_check(cudaMemcpyAsync(dst, bytes.data(), bytes.size(), cudaMemcpyHostToDevice, stream), "uploading a weight");
    ops::cuda_check(cudaStreamSynchronize(stream), "uploading a weight");     // `bytes` leaves scope
}
}  // namespace

DeviceTensor BindContext::upload(const HostTensor& t, DType as) {
    const auto key = std::make_pair(t.data, static_cast<int>(as));
    auto it = uploads_.find(key);
    if (it != uploads_.end() && it->second.shape == t.shape) return it->second;
    DeviceTensor d;
    d.dtype = as;
    d.shape = t.shape;
    d.owner = std::make_shared<DeviceBuffer>(static_cast<size_t>(t.numel()) * dtype_size(as));
    d.ptr = d.owner->ptr;
    copy_in(d.ptr, t, as, stream);
    uploads_[key] = d;
    return d;
}

DeviceTensor BindContext::upload_stacked(const std::vector<const HostTensor*>& parts, DType as) {
    if (parts.size() == 1) return upload(*parts[0], as);
    long long rows = 0;
    const long long cols = parts[0]->shape.size() > 1 ? parts[0]->shape[1] : 1;
    for (const HostTensor* p : parts) rows += p->shape[0];
    DeviceTensor d;
    d.dtype = as;
    d.shape = {rows, cols};
    d.owner = std::make_shared<DeviceBuffer>(static_cast<size_t>(rows * cols) * dtype_size(as));
    d.ptr = d.owner->ptr;
    size_t off = 0;
    for (const HostTensor* p : parts) {
        copy_in(static_cast<char*>(d.ptr) + off, *p, as, stream);
        off += static_cast<size_t>(p->numel()) * dtype_size(as);
    }
    return d;
}

DeviceTensor BindContext::upload_floats(const std::vector<float>& values) {
    HostTensor t;
    t.dtype = DType::F32;
    t.shape = {static_cast<long long>(values.size())};
    t.data = reinterpret_cast<const uint8_t*>(values.data());
    t.nbytes = values.size() * sizeof(float);
    DeviceTensor d;
    d.dtype = DType::F32;
    d.shape = t.shape;
    d.owner = std::make_shared<DeviceBuffer>(t.nbytes);
    d.ptr = d.owner->ptr;
    copy_in(d.ptr, t, DType::F32, stream);
    return d;
}

DType BindContext::matrix_dtype(const std::vector<const HostTensor*>& stored) const {
    if (dtype == DType::F32) return DType::F32;
    for (const HostTensor* t : stored)
        if (t->dtype == DType::F32) return DType::F32;
    return dtype;
}

// ------------------------------------------------------------------------------------------------ launch bookkeeping
namespace ops {

int SKINNY_MAX_ROWS = 32;      // beyond this the library product wins (the A tile is staged once per CTA; measured per decode step at
                               // 33 / 48 / 64 rows: 1.07 / 1.20 / 1.25 ms fused against 1.02 / 1.07 / 1.05 ms with the library product)
// Large weight matrices: the library product streams them at 3.5 to 5.5 TB/s from 16 rows on, whatever the row count (hidden
// 2,048, 32 rows: 7.2 / 12.1 / 12.5 us for qkv / gate-up / down), the weight-streaming kernels slow down with every row they
// stage.  Decode steps of the 1.7B shape (24 layers), fused against library path: 8 rows 1.32 / 1.63 ms, 12 rows 1.81 / 1.87,
// 16 rows 1.96 / 1.85, 24 rows 2.83 / 2.12, 32 rows 3.22 / 2.30; the 360M shape (largest matrix 9.8 MB) stays fused up to 32
// rows (0.79 / 1.29 ms at 8 rows, 1.45 / 1.43 at 32).
int SKINNY_MAX_ROWS_LARGE = 8;
// The head (49,152 rows of K = 576 / 960 / 2,048): own kernels 13.0 / 18.1 / 31.8 us at 8 rows, 24.0 / 35.8 / 55.8 us at 32; the
// library product 11 to 35 us whatever the row count (17.6 / 34.6 us at 8 rows of K = 960 / 2,048, 11.2 / 18.2 / 35.5 us at 32).
int SKINNY_HEAD_MAX_ROWS = 8;
long long SKINNY_LARGE_WEIGHT_BYTES = 16ll << 20;
int SKINNY_NORM_ROWS = 32;     // up to this many rows the norm is fused into the product that follows it (measured per decode step at
                               // 17 / 24 / 32 rows: 0.70 / 0.72 / 0.86 ms against 0.82 / 0.84 / 0.92 ms with a norm kernel of its own)

Counters& counters() {
    static Counters c;
    return c;
}

namespace {
struct Switches {
    bool sync = false;
    std::string fail_op;
    Switches() {
        const char* s = std::getenv("VELOMIND_B200_SYNC");
        sync = s && std::string(s) == "1";
        const char* f = std::getenv("VELOMIND_B200_FAIL_OP");
        if (f) fail_op = f;
    }
};
const Switches& switches() {
    static Switches s;
    return s;
}

struct TimedOp { std::string name; cudaEvent_t a, b; };
struct OpTimeState {
    int depth = 0;
    std::vector<TimedOp> ops;
    cudaEvent_t open = nullptr;
};
OpTimeState& op_state() {
    static OpTimeState s;
    return s;
}
}  // namespace

bool sync_every_op() { return switches().sync; }

void check(int status, const char* name, cudaStream_t stream) {
    ++counters().own_launches;
    if (status == 0) {
        if (!switches().fail_op.empty() && switches().fail_op == name)
            throw KernelError(format("%s: injected failure (VELOMIND_B200_FAIL_OP)", name));
        if (switches().sync) {
            const cudaError_t e = cudaStreamSynchronize(stream);
            if (e != cudaSuccess) throw KernelError(format("%s: CUDA error %d (%s)", name, static_cast<int>(e), cudaGetErrorString(e)));
        }
        return;
    }
    if (status == VM_ERR_UNSUPPORTED) throw KernelError(format("%s: this size or dtype is not supported by the kernel", name));
    if (status == VM_ERR_BAD_ARG) throw KernelError(format("%s: bad argument", name));
    throw KernelError(format("%s: CUDA error %d (%s)", name, status, cudaGetErrorString(static_cast<cudaError_t>(status))));
}

bool op_times_active() { return op_state().depth > 0; }

void op_time_begin(const char* name, cudaStream_t stream) {
    OpTimeState& st = op_state();
    TimedOp op;
    op.name = name;
    if (cudaEventCreate(&op.a) != cudaSuccess || cudaEventCreate(&op.b) != cudaSuccess) return;
    cudaEventRecord(op.a, stream);
    st.ops.push_back(op);
}

void op_time_end(const char* name, cudaStream_t stream) {
    OpTimeState& st = op_state();
    for (auto it = st.ops.rbegin(); it != st.ops.rend(); ++it)
        if (it->name == name) { cudaEventRecord(it->b, stream); return; }
}

OpTimes::OpTimes() { ++op_state().depth; }

OpTimes::~OpTimes() {
    OpTimeState& st = op_state();
    if (--st.depth == 0) {
        for (auto& op : st.ops) { cudaEventDestroy(op.a); cudaEventDestroy(op.b); }
        st.ops.clear();
    }
}

std::string OpTimes::table() {
    OpTimeState& st = op_state();
    cudaDeviceSynchronize();
    std::map<std::string, std::pair<int, double>> sums;
    double total = 0.0;
    for (auto& op : st.ops) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, op.a, op.b) != cudaSuccess) { cudaGetLastError(); continue; }
        sums[op.name].first += 1;
        sums[op.name].second += ms;
        total += ms;
    }
    std::string out = format("%-22s %8s %12s %7s\n", "operation", "launches", "device ms", "share");
    for (const auto& kv : sums)
        out += format("%-22s %8d %12.3f %6.1f%%\n", kv.first.c_str(), kv.second.first, kv.second.second, total > 0 ? 100.0 * kv.second.second / total : 0.0);
    out += format("%-22s %8zu %12.3f\n", "total", st.ops.size(), total);
    return out;
}

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) cached[dev] = n;
        else return 1;
    }
    return cached[dev];
}

// ------------------------------------------------------------------------------------------------ the library product
namespace {
struct Blas {
    cublasHandle_t handle = nullptr;
    std::unique_ptr<DeviceBuffer> workspace;
    cudaStream_t stream = nullptr;        // the stream the handle was last given (with the workspace, which a new stream resets)
    bool bound = false;
    // The handle's stream and scratch are set when they change, not per product: a step multiplies a hundred times and more on one stream.
    void bind(cudaStream_t s, const char* who) {
        if (bound && stream == s) return;
        if (cublasSetStream(handle, s) != CUBLAS_STATUS_SUCCESS || cublasSetWorkspace(handle, workspace->ptr, workspace->bytes) != CUBLAS_STATUS_SUCCESS)
            throw KernelError(std::string(who) + ": the matrix-product library refused the stream");
        stream = s;
        bound = true;
    }
};
Blas& blas() {
    static Blas per_device[64];
    int dev = 0;
    cuda_check(cudaGetDevice(&dev), "asking for the current device");
    Blas& b = per_device[dev < 0 || dev >= 64 ? 0 : dev];
    if (!b.handle) {
        if (cublasCreate(&b.handle) != CUBLAS_STATUS_SUCCESS) throw KernelError("the matrix-product library could not be set up");
        // its scratch is given once, so that a product inside a recorded step allocates nothing
        b.workspace = std::make_unique<DeviceBuffer>(64u << 20);
        // float32 products stay float32 (no TF32), and bfloat16 products sum in float32 throughout (no reduced-precision reduction)
        cublasSetMathMode(b.handle, static_cast<cublasMath_t>(CUBLAS_DEFAULT_MATH | CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION));
    }
    return b;
}
}  // namespace

void linear(const void* x, DType x_dtype, long long ldx, const DeviceTensor& W, void* out, DType out_dtype, int T, cudaStream_t s) {
    if (T <= 0) return;
    if (x_dtype != W.dtype) throw KernelError(format("linear: input %s does not fit weights kept in %s", dtype_name(x_dtype), dtype_name(W.dtype)));
    if (!(out_dtype == x_dtype || out_dtype == DType::F32)) throw KernelError("linear: the result has the input's dtype or float32");
    Timed t("linear", s);
    Blas& b = blas();
    const int N = static_cast<int>(W.rows()), K = static_cast<int>(W.cols());
    const cudaDataType_t in_t = x_dtype == DType::F32 ? CUDA_R_32F : CUDA_R_16BF;
    const cudaDataType_t out_t = out_dtype == DType::F32 ? CUDA_R_32F : CUDA_R_16BF;
    const float one = 1.f, zero = 0.f;
    b.bind(s, "linear");
    // row-major out[T, N] = x[T, K] W[N, K]^T  is  column-major out^T[N, T] = W^T(K x N)^T x^T(K x T)
    const cublasStatus_t st = cublasGemmEx(b.handle, CUBLAS_OP_T, CUBLAS_OP_N, N, T, K, &one, W.ptr, in_t, K, x, in_t, static_cast<int>(ldx), &zero, out,
                                           out_t, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    ++counters().library_calls;
    if (st != CUBLAS_STATUS_SUCCESS) throw KernelError(format("linear: the matrix-product library reported status %d", static_cast<int>(st)));
    if (!switches().fail_op.empty() && switches().fail_op == "linear") throw KernelError("linear: injected failure (VELOMIND_B200_FAIL_OP)");
    if (switches().sync) cuda_check(cudaStreamSynchronize(s), "linear");
}

void linear_residual(const void* x, long long ldx, const DeviceTensor& W, float* h, int T, cudaStream_t s) {
    if (T <= 0) return;
    if (W.dtype != DType::BF16) throw KernelError(format("linear_residual: weights kept in %s (bfloat16 only)", dtype_name(W.dtype)));
    Timed t("linear", s);
    Blas& b = blas();
    const int N = static_cast<int>(W.rows()), K = static_cast<int>(W.cols());
    const float one = 1.f;
    b.bind(s, "linear_residual");
    const cublasStatus_t st = cublasGemmEx(b.handle, CUBLAS_OP_T, CUBLAS_OP_N, N, T, K, &one, W.ptr, CUDA_R_16BF, K, x, CUDA_R_16BF, static_cast<int>(ldx), &one, h,
                                           CUDA_R_32F, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    ++counters().library_calls;
    if (st != CUBLAS_STATUS_SUCCESS) throw KernelError(format("linear_residual: the matrix-product library reported status %d", static_cast<int>(st)));
    if (!switches().fail_op.empty() && switches().fail_op == "linear") throw KernelError("linear: injected failure (VELOMIND_B200_FAIL_OP)");
    if (switches().sync) cuda_check(cudaStreamSynchronize(s), "linear_residual");
}

// ------------------------------------------------------------------------------------------------ attention
namespace {
constexpr int DECODE_COUNTERS = 1 << 16;
constexpr int MAX_DECODE_SPLITS = 16;
constexpr int DECODE_ONE_CTA_BLOCKS = 16;     // block tables up to this wide (1,024 tokens): at most two rounds of pages for ten warps
constexpr int TC_ATTENTION_MIN_BLOCKS = 20;   // head size 64: the tcgen05 prefill attention when a tile may see this many key blocks
constexpr int TC_ATTENTION_CTAS_PER_SM = 3;   // CTAs of that kernel an SM holds at once (registers and shared memory)
int WS_ATTENTION_MIN_BLOCKS = 32;             // head size 64: the warp-specialised tcgen05 attention when a tile may see this many key blocks

int* decode_counters() {
    static std::unique_ptr<DeviceBuffer> per_device[64];
    int dev = 0;
    cuda_check(cudaGetDevice(&dev), "asking for the current device");
    auto& b = per_device[dev < 0 || dev >= 64 ? 0 : dev];
    if (!b) b = std::make_unique<DeviceBuffer>(DECODE_COUNTERS * sizeof(int), /*zero=*/true);   // the kernel leaves them zero after every launch
    return static_cast<int*>(b->ptr);
}

// How many CTAs share the keys of one (sequence, kv head): enough to fill the GPU, a function of the step's SHAPE only
// (so that a recorded launch stays valid as sequences grow).
int decode_splits(int B, int Hkv, int G, int table_width) {
    const int groups = B * Hkv * ((G + 15) / 16);           // a CTA serves up to 16 query heads of one kv head
    const int sms = sm_count();
    if (groups <= sms && table_width <= DECODE_ONE_CTA_BLOCKS) return 1;   // short sequences: one CTA of ten warps holds all pages
    const int want = (sms + groups - 1) / groups;            // about one CTA per SM ...
    const int by_width = std::max(1, table_width / 4);       // ... and at least a page per warp of a CTA (the width bounds the pages)
    return std::max(1, std::min(want, std::min(MAX_DECODE_SPLITS, by_width)));
}
}  // namespace

void attention(StepContext& ctx, const void* q, int q_row_stride, const KVView& kv, void* out, int H, int Hkv, int D, float scale, int window) {
    cudaStream_t s = ctx.stream;
    const bool fast = ctx.act_dtype == DType::BF16 && D % 16 == 0 && D <= 128 && q_row_stride % 8 == 0;
    if (fast && ctx.one_token_each && static_cast<long long>(ctx.B) * H <= DECODE_COUNTERS) {
        const int n_splits = decode_splits(ctx.B, Hkv, H / Hkv, kv.table_width);
        float* partial = static_cast<float*>(ctx.take(static_cast<long long>(ctx.B_cap) * H * MAX_DECODE_SPLITS * (D + 2), DType::F32));   // sized by shape
        {
            Timed t("attention_decode_bf16", s);
            check(vm_attention_decode_bf16(q, q_row_stride, kv.k_pages, kv.v_pages, kv.block_table, kv.table_width, ctx.positions, out, partial,
                                           decode_counters(), ctx.B, H, Hkv, D, n_splits, scale, window, kv.n_pages, ctx.err, s),
                  "attention_decode_bf16", s);
        }
        ctx.give(partial);
        return;
    }
    if (fast) {
        // Which kernel, and how its work is cut, follows from the step's SHAPE alone (new tokens per sequence, table width), never
        // from its lengths: a recorded step keeps its choice.  The table width bounds the key blocks a tile may walk.
        int most_blocks = kv.table_width;
        if (window > 0) most_blocks = std::min(most_blocks, window / VM_PAGE_TOKENS + 2);
        long long tiles128 = 0, tiles64 = 0;
        for (int b = 0; b < ctx.B; ++b) {
            const int n = ctx.host_cu_tokens[b + 1] - ctx.host_cu_tokens[b];
            tiles128 += (n + 127) / 128;
            tiles64 += (n + 63) / 64;
        }
        if (D == 64 && most_blocks >= WS_ATTENTION_MIN_BLOCKS && ctx.err != nullptr) {
            // the longest prompts: softmax warps, a copy warp and product warps, clusters dealt out to pairs of tile groups
            // (measured, 9 heads: 4,096 tokens 78 us against 88 us for the kernel below, 8,192: 224 / 262; 2,048: 32 / 33;
            //  2,560: 37 / 48, 3,072: 51 / 58, 1,536: 27 / 24, 1,024: 22 / 18: every CTA pays for its set-up and its cluster's exchange once, whatever its share of the keys;
            //  with one query head per kv head a CTA takes three row tiles of the head: 32 heads, 2,048 tokens 70 / 80 us, 3,072: 88 / 148)
            ++counters().tc_attention_calls;
            Timed t("attention_prefill_ws_bf16", s);
            check(vm_attention_prefill_ws_bf16(q, q_row_stride, kv.k_pages, kv.v_pages, kv.block_table, kv.table_width, ctx.positions, ctx.cu_tokens,
                                               ctx.host_cu_tokens, ctx.B, out, H, Hkv, D, scale, window, kv.n_pages, ctx.err, 0, s),
                  "attention_prefill_ws_bf16", s);
            return;
        }
        if (D == 64 && most_blocks >= TC_ATTENTION_MIN_BLOCKS && ctx.err != nullptr) {
            // long prompts: the tcgen05 kernel, a tile's key blocks dealt out to as many CTAs (2 to 4) as still fit the GPU at once
            // (measured, 9 heads: 1,536 tokens 23.7 us against 32.2 us for the mma.sync kernel; 2,048: 33.6 / 39.4; 4,096: 89.9 / 123.8;
            //  1,024: 17.6 / 16.6, hence the threshold)
            const long long slots = static_cast<long long>(sm_count()) * TC_ATTENTION_CTAS_PER_SM;
            const int groups = static_cast<int>(std::max<long long>(2, std::min<long long>(4, slots / std::max<long long>(1, tiles128 * H))));
            ++counters().tc_attention_calls;
            Timed t("attention_prefill_tc_bf16", s);
            check(vm_attention_prefill_tc_bf16(q, q_row_stride, kv.k_pages, kv.v_pages, kv.block_table, kv.table_width, ctx.positions, ctx.cu_tokens, ctx.B,
                                               static_cast<int>(tiles128), out, H, Hkv, D, scale, window, kv.n_pages, ctx.err, groups, s),
                  "attention_prefill_tc_bf16", s);
            return;
        }
        const int groups = most_blocks >= 8 ? 2 : 1;      // measured at 9 heads of 64: 2 groups 39 us, 1 group 43 us, 4 groups 46 us (2,048 tokens)
        Timed t("attention_prefill_bf16", s);
        check(vm_attention_prefill_bf16(q, q_row_stride, kv.k_pages, kv.v_pages, kv.block_table, kv.table_width, ctx.positions, ctx.cu_tokens, ctx.B,
                                        static_cast<int>(tiles64), out, H, Hkv, D, scale, window, kv.n_pages, ctx.err, groups, s),
              "attention_prefill_bf16", s);
        return;
    }
    Timed t("attention_generic", s);
    check(vm_attention_generic(q, q_row_stride, kv.k_pages, kv.v_pages, kv.block_table, kv.table_width, ctx.positions, ctx.seq_of_token, out, ctx.T, H,
                               Hkv, D, scale, window, kv.n_pages, code(ctx.act_dtype), ctx.err, s),
          "attention_generic", s);
}

}  // namespace ops
}  // namespace vmb
