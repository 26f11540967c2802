// Position encodings.  A position part owns constants only; the mixer's kernels apply them.
#include "args.h"
#include "velomind_b200/kernels.h"

namespace vmb {

// Rotary positions.  Frequencies as the reference builds them, in float32: inv_freq[j] = 1 / pow(theta, 2j / rotary_dim)
// (examples/common/llama/llama_rope_mask.cpp:17-19); the angle pos * inv_freq[j] and its sine and cosine are computed in
// float32 on the device.  Which two values of a head make pair j is the `pairing`: the reference's half-split
// (j, j + rotary_dim/2) (src/cpu/ops/rotary_embedding.cpp:30-44), or interleaved (2j, 2j + 1).
class Rotary : public Position {
public:
    Rotary(int head_dim, double theta, int rotary_dim, int pairing) : head_dim_(head_dim), rotary_dim_(rotary_dim), pairing_(pairing), theta_(theta) {
        if (rotary_dim_ % 2 || rotary_dim_ <= 0 || rotary_dim_ > head_dim_)
            throw ConfigError(format("rotary_dim %d must be even and within the head size %d", rotary_dim_, head_dim_));
    }
    bool graph_safe() const override { return true; }
    std::vector<float> inv_freq_host() const {
        std::vector<float> f(static_cast<size_t>(rotary_dim_ / 2));
        for (int j = 0; j < rotary_dim_ / 2; ++j) {
            const float exponent = (2.0f * static_cast<float>(j)) / static_cast<float>(rotary_dim_);
            f[j] = 1.0f / powf(static_cast<float>(theta_), exponent);
        }
        return f;
    }
    RotaryTable tables(BindContext& bc) override {
        if (!table_.ptr) table_ = bc.upload_floats(inv_freq_host());
        return RotaryTable{static_cast<const float*>(table_.ptr), rotary_dim_, pairing_};
    }

private:
    int head_dim_, rotary_dim_, pairing_;
    double theta_;
    DeviceTensor table_;
};

// No position encoding: queries and keys pass unrotated.
class NoPosition : public Position {
public:
    bool graph_safe() const override { return true; }
    RotaryTable tables(BindContext&) override { return RotaryTable{}; }
};

namespace {
std::shared_ptr<Part> make_rotary(const json::Value& a, int pairing, const char* kind) {
    const int head_dim = static_cast<int>(arg_int(a, "head_dim", kind));
    return std::make_shared<Rotary>(head_dim, arg_number(a, "theta", kind), static_cast<int>(arg_int_or(a, "rotary_dim", head_dim, kind)), pairing);
}
RegisterPart reg_half("position", "rotary_half_split", [](const json::Value& a) { return make_rotary(a, VM_PAIR_HALF_SPLIT, "rotary_half_split"); });
RegisterPart reg_inter("position", "rotary_interleaved", [](const json::Value& a) { return make_rotary(a, VM_PAIR_INTERLEAVED, "rotary_interleaved"); });
RegisterPart reg_none("position", "none", [](const json::Value&) { return std::make_shared<NoPosition>(); });
}  // namespace

}  // namespace vmb
