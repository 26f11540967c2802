// linear.h (internal) — a bias-free linear map y = x W^T with W in the checkpoint's [out, in] layout.
//
// Several checkpoint matrices that read the same input can be stacked into one (q/k/v, gate/up): one product instead of
// three.  The reference transposes each matrix to [in, out] and multiplies one by one
// (examples/smollm2/model_loader.cpp:176-233, examples/common/llama/llama_graph.cpp:63-65); [out, in] rows are
// K-contiguous, which is what the tensor-core and weight-streaming kernels want.
#pragma once

#include "../engine/ops.h"

namespace vmb {

struct Linear {
    DeviceTensor weight;
    long long out_features = 0, in_features = 0;

    void bind(const std::vector<const HostTensor*>& stored, BindContext& bc) {
        weight = bc.upload_stacked(stored, bc.matrix_dtype(stored));
        out_features = weight.rows();
        in_features = weight.cols();
    }

    // out[rows, N] = x[rows, K] W^T.  `out_dtype` is x's dtype or float32 (logits).  A matrix stored in 32-bit stays float32
    // under bfloat16 activations: the input is widened, the product runs in float32, the result is narrowed.  Scratch is taken
    // for `rows_cap` rows (the capacity of the step's bucket), so that every step of a bucket asks for the same buffers.
    void apply(StepContext& ctx, const void* x, DType x_dtype, void* out, DType out_dtype, int rows, long long rows_cap) const {
        if (x_dtype == weight.dtype) {
            ops::linear(x, x_dtype, in_features, weight, out, out_dtype, rows, ctx.stream);
            return;
        }
        if (weight.dtype != DType::F32)
            throw KernelError(format("linear: input %s does not fit weights kept in %s", dtype_name(x_dtype), dtype_name(weight.dtype)));
        void* x32 = ctx.take(rows_cap * in_features, DType::F32);
        if (rows > 0) ops::convert(x, x_dtype, x32, DType::F32, static_cast<long long>(rows) * in_features, ctx.stream);
        if (out_dtype == DType::F32) {
            ops::linear(x32, DType::F32, in_features, weight, out, DType::F32, rows, ctx.stream);
        } else {
            void* y32 = ctx.take(rows_cap * out_features, DType::F32);
            ops::linear(x32, DType::F32, in_features, weight, y32, DType::F32, rows, ctx.stream);
            if (rows > 0) ops::convert(y32, DType::F32, out, out_dtype, static_cast<long long>(rows) * out_features, ctx.stream);
            ctx.give(y32);
        }
        ctx.give(x32);
    }
};

}  // namespace vmb
