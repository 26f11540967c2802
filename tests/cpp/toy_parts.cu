// Parts and architectures defined HERE, in the tests, and registered through the library's public header alone: a
// plug-in library that the tests load beside the library itself.  Nothing of the library is changed for them.
//
//   toy_decaying_sum          a mixer whose whole memory is a fixed-size state per sequence (no keys, no values):
//                             state <- decay * state + x W_in ; out = state W_out
//   toy_top_one_experts       a feed-forward with routing: a router (float32 logits) picks one of several small
//                             two-layer ReLU networks per token
//   toy_evenly_spaced_rotary  a position encoding with frequencies of its own (evenly spaced instead of geometric)
//   identity (norm, head), mixer_only / feed_forward_only (arrangements)
//                             probes that let a test see ONE part's output: the residual stream passes unchanged
//                             through everything else
// Architectures: "ToyForCausalLM" mixes the toy parts with the built-in attention and SwiGLU layer by layer;
// "LoopedLlamaForCausalLM" runs the Llama layers in another order (a layer twice, a run that reads another run's
// cache); "WindowedLlamaForCausalLM" gives every odd layer a window; "ProbeForCausalLM" builds whatever parts its
// config.json names.  They are toys that exercise the interfaces; they are nobody's model.
#include <cuda_bf16.h>

#include "velomind_b200/kernels.h"
#include "velomind_b200/velomind.h"

using namespace vmb;

namespace {

// ------------------------------------------------------------------------------------------------ small kernels
template <typename T> __device__ float to_f(T x);
template <> __device__ float to_f<float>(float x) { return x; }
template <> __device__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ T from_f(float x);
template <> __device__ float from_f<float>(float x) { return x; }
template <> __device__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// y[t, n] = sum_k x[t, k] * W[n, k]   (W float32 [N, K]); one thread per output
template <typename TX, typename TY> __global__ void matmul_kernel(const TX* x, const float* W, TY* y, int T, int N, int K) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)T * N) return;
    const int t = (int)(i / N), n = (int)(i % N);
    float acc = 0.f;
    for (int k = 0; k < K; ++k) acc += to_f(x[(size_t)t * K + k]) * W[(size_t)n * K + k];
    y[i] = from_f<TY>(acc);
}

// the scan of the state mixer: one block per sequence, one thread per state value, tokens in order
__global__ void decay_scan_kernel(float* u /* [T, W] in, states out */, float* state /* [slots, W] */, const int* cu_tokens, const int* slots,
                                  int W, float decay) {
    const int s = blockIdx.x, j = threadIdx.x;
    if (j >= W) return;
    float st = state[(size_t)slots[s] * W + j];
    for (int t = cu_tokens[s]; t < cu_tokens[s + 1]; ++t) {
        st = decay * st + u[(size_t)t * W + j];
        u[(size_t)t * W + j] = st;
    }
    state[(size_t)slots[s] * W + j] = st;
}

// routed feed-forward: one block per token; router logits in float32, lowest index wins a tie
template <typename T> __global__ void experts_kernel(const T* x, const float* router, const float* up, const float* down, T* out, int hid, int inner,
                                                     int experts) {
    extern __shared__ float sm[];               // [hid] input, [inner] activations, [1] choice
    float* xs = sm;
    float* act = sm + hid;
    int* choice = reinterpret_cast<int*>(sm + hid + inner);
    const int t = blockIdx.x;
    for (int k = threadIdx.x; k < hid; k += blockDim.x) xs[k] = to_f(x[(size_t)t * hid + k]);
    __syncthreads();
    if (threadIdx.x == 0) {
        int best = 0;
        float best_v = -INFINITY;
        for (int e = 0; e < experts; ++e) {
            float acc = 0.f;
            for (int k = 0; k < hid; ++k) acc += xs[k] * router[(size_t)e * hid + k];
            if (acc > best_v) { best_v = acc; best = e; }
        }
        *choice = best;
    }
    __syncthreads();
    const int e = *choice;
    for (int j = threadIdx.x; j < inner; j += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < hid; ++k) acc += xs[k] * up[((size_t)e * inner + j) * hid + k];
        act[j] = fmaxf(acc, 0.f);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < inner; ++j) acc += act[j] * down[((size_t)e * hid + i) * inner + j];
        out[(size_t)t * hid + i] = from_f<T>(acc);
    }
}

// identity norm: h += delta; out[r] = h[rows ? rows[r] : r]
template <typename T> __global__ void identity_norm_kernel(float* h, const T* delta, T* out, const int* rows, int n_out, int hid) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)n_out * hid) return;
    const int r = (int)(i / hid), c = (int)(i % hid);
    const int src = rows ? rows[r] : r;
    float v = h[(size_t)src * hid + c];
    if (delta) v += to_f(delta[(size_t)src * hid + c]);
    if (!rows) h[(size_t)src * hid + c] = v;
    out[i] = from_f<T>(v);
}

void launch_check(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw KernelError(std::string(what) + ": " + cudaGetErrorString(e));
}

long long arg_i(const json::Value& a, const char* k) {
    const json::Value* v = a.find(k);
    if (!v || !v->is_integer()) throw ConfigError(std::string("toy part: argument '") + k + "' must be an integer");
    return v->as_int();
}
double arg_d(const json::Value& a, const char* k) {
    const json::Value* v = a.find(k);
    if (!v || !v->is_number()) throw ConfigError(std::string("toy part: argument '") + k + "' must be a number");
    return v->as_double();
}

template <typename F> void by_dtype(DType t, F&& f) {
    if (t == DType::F32) f(static_cast<float*>(nullptr));
    else f(static_cast<__nv_bfloat16*>(nullptr));
}

// ------------------------------------------------------------------------------------------------ the toy parts
class DecayingSumMixer : public Mixer {
public:
    DecayingSumMixer(int hidden, int width, float decay) : hidden_(hidden), width_(width), decay_(decay) {}
    WeightTable weight_specs() const override {
        WeightTable t;
        t["in.weight"].shape = {width_, hidden_};
        t["out.weight"].shape = {hidden_, width_};
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override {
        in_ = bc.upload(w.at("in.weight"), DType::F32);
        out_ = bc.upload(w.at("out.weight"), DType::F32);
    }
    bool graph_safe() const override { return true; }        // slots and token offsets are read on the device
    CacheNeed cache_need() const override {
        CacheNeed n;
        n.state_floats = width_;                              // kind None: no keys, no values
        return n;
    }
    void forward(StepContext& ctx, const void* x, void* out) override {
        float* u = static_cast<float*>(ctx.take_tokens(width_, DType::F32));
        const long long n_u = (long long)ctx.T * width_, n_o = (long long)ctx.T * hidden_;
        by_dtype(ctx.act_dtype, [&](auto* tag) {
            using T = std::remove_pointer_t<decltype(tag)>;
            matmul_kernel<T, float><<<(unsigned)((n_u + 127) / 128), 128, 0, ctx.stream>>>(static_cast<const T*>(x), static_cast<const float*>(in_.ptr), u,
                                                                                           ctx.T, width_, hidden_);
            decay_scan_kernel<<<ctx.B, ((width_ + 31) / 32) * 32, 0, ctx.stream>>>(u, ctx.state(), ctx.cu_tokens, ctx.slots, width_, decay_);
            matmul_kernel<float, T><<<(unsigned)((n_o + 127) / 128), 128, 0, ctx.stream>>>(u, static_cast<const float*>(out_.ptr), static_cast<T*>(out),
                                                                                           ctx.T, hidden_, width_);
        });
        launch_check("toy_decaying_sum");
        ctx.give(u);
    }

private:
    int hidden_, width_;
    float decay_;
    DeviceTensor in_, out_;
};

class TopOneExperts : public FeedForward {
public:
    TopOneExperts(int hidden, int inner, int experts) : hidden_(hidden), inner_(inner), experts_(experts) {}
    WeightTable weight_specs() const override {
        WeightTable t;
        t["router.weight"].shape = {experts_, hidden_};
        for (int e = 0; e < experts_; ++e) {
            t[format("experts.%d.up.weight", e)].shape = {inner_, hidden_};
            t[format("experts.%d.down.weight", e)].shape = {hidden_, inner_};
        }
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override {
        router_ = bc.upload(w.at("router.weight"), DType::F32);
        std::vector<const HostTensor*> ups, downs;
        for (int e = 0; e < experts_; ++e) {
            ups.push_back(&w.at(format("experts.%d.up.weight", e)));
            downs.push_back(&w.at(format("experts.%d.down.weight", e)));
        }
        up_ = bc.upload_stacked(ups, DType::F32);
        down_ = bc.upload_stacked(downs, DType::F32);
    }
    bool graph_safe() const override { return true; }
    void forward(StepContext& ctx, const void* x, void* out) override {
        const size_t smem = (size_t)(hidden_ + inner_ + 1) * sizeof(float);
        by_dtype(ctx.act_dtype, [&](auto* tag) {
            using T = std::remove_pointer_t<decltype(tag)>;
            experts_kernel<T><<<ctx.T, 128, smem, ctx.stream>>>(static_cast<const T*>(x), static_cast<const float*>(router_.ptr),
                                                                static_cast<const float*>(up_.ptr), static_cast<const float*>(down_.ptr),
                                                                static_cast<T*>(out), hidden_, inner_, experts_);
        });
        launch_check("toy_top_one_experts");
    }

private:
    int hidden_, inner_, experts_;
    DeviceTensor router_, up_, down_;
};

// Rotary pairs whose frequencies are evenly spaced between 0 and `top` instead of geometric: a position part owns
// constants only, so another table (and, if wanted, another pairing) is all there is to it.
class EvenlySpacedRotary : public Position {
public:
    EvenlySpacedRotary(int head_dim, double top, int pairing) : head_dim_(head_dim), top_(top), pairing_(pairing) {}
    bool graph_safe() const override { return true; }
    RotaryTable tables(BindContext& bc) override {
        if (!table_.ptr) {
            const int half = head_dim_ / 2;
            std::vector<float> f((size_t)half);
            for (int j = 0; j < half; ++j) f[(size_t)j] = (float)(j + 1) * (float)(top_ / half);
            table_ = bc.upload_floats(f);
        }
        return RotaryTable{static_cast<const float*>(table_.ptr), head_dim_, pairing_};
    }

private:
    int head_dim_;
    double top_;
    int pairing_;
    DeviceTensor table_;
};

class IdentityNorm : public Norm {
public:
    explicit IdentityNorm(int size) : size_(size) {}
    bool graph_safe() const override { return true; }
    void forward(StepContext& ctx, float* h, const void* delta, void* out, const int* rows, int n_rows) override {
        const int n_out = rows ? n_rows : ctx.T;
        const long long n = (long long)n_out * size_;
        if (n == 0) return;
        by_dtype(ctx.act_dtype, [&](auto* tag) {
            using T = std::remove_pointer_t<decltype(tag)>;
            identity_norm_kernel<T><<<(unsigned)((n + 127) / 128), 128, 0, ctx.stream>>>(h, static_cast<const T*>(delta), static_cast<T*>(out), rows, n_out,
                                                                                         size_);
        });
        launch_check("identity norm");
    }

private:
    int size_;
};

// logits = x (vocabulary = width): what reaches the head is what the test sees
class IdentityHead : public Head {
public:
    explicit IdentityHead(int size) : size_(size) {}
    bool graph_safe() const override { return true; }
    void forward(StepContext& ctx, const void* x, float* logits) override {
        const long long n = (long long)ctx.R * size_;
        if (ctx.act_dtype == DType::F32) {
            if (cudaMemcpyAsync(logits, x, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, ctx.stream) != cudaSuccess)
                throw KernelError("identity head: the copy failed");
        } else if (vm_convert(x, VM_BF16, logits, VM_F32, n, ctx.stream) != 0) {
            throw KernelError("identity head: the conversion kernel refused");
        }
    }

private:
    int size_;
};

// out = part(norm(h)) left pending: the sum h + part(h) reaches the head, nothing else runs
class MixerOnly : public Arrangement {
public:
    explicit MixerOnly(const BlockParts& p) : p_(p) {}
    bool graph_safe() const override { return true; }
    void* forward(StepContext& ctx, float* h, void* pending) override {
        void* x = ctx.take_tokens(ctx.hidden, ctx.act_dtype);
        p_.mixer_norm->forward(ctx, h, pending, x, nullptr, 0);
        ctx.give(pending);
        void* out = ctx.take_tokens(ctx.hidden, ctx.act_dtype);
        p_.mixer->forward(ctx, x, out);
        ctx.give(x);
        return out;
    }

private:
    BlockParts p_;
};

class FeedForwardOnly : public Arrangement {
public:
    explicit FeedForwardOnly(const BlockParts& p) : p_(p) {}
    bool graph_safe() const override { return true; }
    void* forward(StepContext& ctx, float* h, void* pending) override {
        void* x = ctx.take_tokens(ctx.hidden, ctx.act_dtype);
        p_.feed_forward_norm->forward(ctx, h, pending, x, nullptr, 0);
        ctx.give(pending);
        void* out = ctx.take_tokens(ctx.hidden, ctx.act_dtype);
        p_.feed_forward->forward(ctx, x, out);
        ctx.give(x);
        return out;
    }

private:
    BlockParts p_;
};

// ------------------------------------------------------------------------------------------------ the toy architectures
json::Value obj(std::initializer_list<std::pair<const char*, json::Value>> members) {
    json::Value o;
    o.object();
    for (const auto& m : members) o.set(m.first, m.second);
    return o;
}

ModelPlan toy_plan(const json::Value& data, const std::string& where) {
    KeyReader r(data, where);
    const int vocab = (int)r.integer("vocab"), width = (int)r.integer("width"), layers = (int)r.integer("layers"), state = (int)r.integer("state");
    const int heads = (int)r.integer("heads"), experts = (int)r.integer("experts"), limit = (int)r.integer("limit");
    const double decay = r.number("decay"), eps = r.number("eps"), theta = r.number("theta");
    const int even_rotary = (int)r.integer("even_rotary", 0);      // 0: geometric; 1: evenly spaced, half-split; 2: evenly spaced, interleaved
    const PartSpec norm{"rmsnorm", obj({{"size", width}, {"eps", eps}})};
    ModelPlan plan;
    plan.hidden_size = width;
    plan.vocab_size = vocab;
    for (int l = 0; l < layers; ++l) {
        BlockSpec b;
        b.arrangement = "prenorm";
        b.prefix = format("toy.layers.%d.", l);
        if (l % 2 == 0) {       // state mixer + built-in SwiGLU
            b.mixer = PartSpec{"toy_decaying_sum", obj({{"hidden", width}, {"width", state}, {"decay", decay}})};
            b.feed_forward = PartSpec{"swiglu", obj({{"hidden", width}, {"intermediate", 2 * width}})};
        } else {                // built-in attention (the last one with the toy position encoding) + routed feed-forward
            const int hd = width / heads;
            json::Value position = obj({{"kind", "rotary_half_split"}, {"args", obj({{"head_dim", hd}, {"theta", theta}})}});
            if (even_rotary && l == layers - 1)
                position = obj({{"kind", "toy_evenly_spaced_rotary"}, {"args", obj({{"head_dim", hd}, {"top", 0.5}, {"interleaved", even_rotary == 2 ? 1 : 0}})}});
            b.mixer = PartSpec{"grouped_query_attention", obj({{"hidden", width}, {"heads", heads}, {"kv_heads", 1}, {"head_dim", hd}, {"position", position}})};
            b.feed_forward = PartSpec{"toy_top_one_experts", obj({{"hidden", width}, {"inner", width}, {"experts", experts}})};
        }
        b.mixer_norm = norm;
        b.feed_forward_norm = norm;
        plan.blocks.push_back(b);
        plan.schedule.push_back(ScheduleEntry{l, -1});
    }
    plan.embedding = PartSpec{"token_table", obj({{"vocab", vocab}, {"hidden", width}})};
    plan.embedding_prefix = "toy.embed.";
    plan.final_norm = norm;
    plan.final_norm_prefix = "toy.norm.";
    plan.head = PartSpec{"linear", obj({{"vocab", vocab}, {"hidden", width}})};
    plan.head_prefix = "toy.head.";
    plan.max_positions = limit;
    return plan;
}

// the Llama layers in another order: "schedule": [[layer, cache_of or -1], ...] in config.json
ModelPlan looped_plan(const json::Value& data, const std::string& where) {
    ModelPlan plan = llama_plan(LlamaConfig::from_json(data, where));
    const json::Value* s = data.find("schedule");
    if (!s || !s->is_array()) throw ConfigError(where + ": missing required key 'schedule'");
    plan.schedule.clear();
    for (const auto& e : s->as_array()) plan.schedule.push_back(ScheduleEntry{(int)e.as_array()[0].as_int(), (int)e.as_array()[1].as_int()});
    return plan;
}

// every odd layer sees only the last "window" keys
ModelPlan windowed_plan(const json::Value& data, const std::string& where) {
    ModelPlan plan = llama_plan(LlamaConfig::from_json(data, where));
    const int window = (int)KeyReader(data, where).integer("window");
    for (size_t l = 1; l < plan.blocks.size(); l += 2) plan.blocks[l].mixer.args.set("window", window);
    return plan;
}

// whatever config.json names: "embedding", "final_norm", "head" as parts, "blocks": [{arrangement, mixer, feed_forward, mixer_norm,
// feed_forward_norm}], "hidden", "vocab", "limit"
ModelPlan probe_plan(const json::Value& data, const std::string& where) {
    KeyReader r(data, where);
    ModelPlan plan;
    plan.hidden_size = (int)r.integer("hidden");
    plan.vocab_size = (int)r.integer("vocab");
    plan.max_positions = (int)r.integer("limit");
    auto part = [&](const json::Value& o, const char* key) {
        const json::Value* v = o.find(key);
        if (!v) throw ConfigError(where + ": missing part '" + key + "'");
        return part_spec_from_json(*v, where + ": " + key);
    };
    plan.embedding = part(data, "embedding");
    plan.embedding_prefix = "embed.";
    plan.final_norm = part(data, "final_norm");
    plan.final_norm_prefix = "norm.";
    plan.head = part(data, "head");
    plan.head_prefix = "head.";
    if (const json::Value* blocks = data.find("blocks")) {
        int l = 0;
        for (const auto& b : blocks->as_array()) {
            BlockSpec spec;
            spec.arrangement = b.find("arrangement")->as_string();
            spec.prefix = format("layers.%d.", l);
            spec.mixer = part(b, "mixer");
            spec.feed_forward = part(b, "feed_forward");
            spec.mixer_norm = part(b, "mixer_norm");
            spec.feed_forward_norm = part(b, "feed_forward_norm");
            plan.blocks.push_back(spec);
            plan.schedule.push_back(ScheduleEntry{l++, -1});
        }
    }
    return plan;
}

struct RegisterToys {
    RegisterToys() {
        register_part("mixer", "toy_decaying_sum", [](const json::Value& a) {
            return std::make_shared<DecayingSumMixer>((int)arg_i(a, "hidden"), (int)arg_i(a, "width"), (float)arg_d(a, "decay"));
        });
        register_part("feed_forward", "toy_top_one_experts", [](const json::Value& a) {
            return std::make_shared<TopOneExperts>((int)arg_i(a, "hidden"), (int)arg_i(a, "inner"), (int)arg_i(a, "experts"));
        });
        register_part("position", "toy_evenly_spaced_rotary", [](const json::Value& a) {
            return std::make_shared<EvenlySpacedRotary>((int)arg_i(a, "head_dim"), arg_d(a, "top"),
                                                        arg_i(a, "interleaved") ? VM_PAIR_INTERLEAVED : VM_PAIR_HALF_SPLIT);
        });
        register_part("norm", "identity", [](const json::Value& a) { return std::make_shared<IdentityNorm>((int)arg_i(a, "size")); });
        register_part("head", "identity", [](const json::Value& a) { return std::make_shared<IdentityHead>((int)arg_i(a, "size")); });
        register_arrangement("mixer_only", [](const json::Value&, const BlockParts& p) { return std::make_shared<MixerOnly>(p); });
        register_arrangement("feed_forward_only", [](const json::Value&, const BlockParts& p) { return std::make_shared<FeedForwardOnly>(p); });
        register_architecture("ToyForCausalLM", toy_plan);
        register_architecture("LoopedLlamaForCausalLM", looped_plan);
        register_architecture("WindowedLlamaForCausalLM", windowed_plan);
        register_architecture("ProbeForCausalLM", probe_plan);
    }
} register_toys;

}  // namespace

// lets a test check that the plug-in is loaded and what it registered
extern "C" const char* toy_parts_registered() {
    return "toy_decaying_sum toy_top_one_experts toy_evenly_spaced_rotary identity mixer_only feed_forward_only ToyForCausalLM "
           "LoopedLlamaForCausalLM WindowedLlamaForCausalLM ProbeForCausalLM";
}
