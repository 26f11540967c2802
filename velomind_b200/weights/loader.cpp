// Weights bound by tensor name and checked against what the model expects; the random-weights mode.
//
// The model publishes a table `name -> WeightSpec`; `load_weights` reads `model.safetensors` and reports everything that
// does not fit in ONE error: missing tensors, unexpected tensors, wrong shapes, wrong kinds of dtype.  Dtypes stay as
// stored: casting for a compute path is the business of the part that owns the tensor.
//
// Random weights: the reference's `--synthetic` switch fills device buffers with uniform noise and never writes a file
// (examples/common/llama/llama_engine.cpp:168-230); here the random model is an ordinary folder, so everything that
// reads a model (engine, replay, tests) takes it through the same loader.
#include <cmath>
#include <cstring>
#include <fstream>
#include <sys/stat.h>
#include <thread>

#include "velomind_b200/velomind.h"

namespace vmb {

namespace {
bool file_exists(const std::string& p) {
    struct stat st;
    return ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

std::string shape_text(const std::vector<long long>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); ++i) out += (i ? ", " : "") + std::to_string(s[i]);
    return out + "]";
}

std::string joined(const std::vector<std::string>& v, const char* sep) {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? sep : "") + v[i];
    return s;
}
}  // namespace

HostTensors check_and_bind(const HostTensors& found, const WeightTable& specs, const std::string& where) {
    std::vector<std::string> missing, unexpected, wrong_shape, wrong_kind;
    HostTensors bound;
    for (const auto& kv : specs) {
        const std::string& name = kv.first;
        const WeightSpec& spec = kv.second;
        auto it = found.find(name);
        if (it == found.end()) {
            if (!spec.alias_of.empty() && found.count(spec.alias_of)) continue;   // resolved below, after the target has been checked
            missing.push_back(name);
            continue;
        }
        const HostTensor& t = it->second;
        if (t.shape != spec.shape) {
            wrong_shape.push_back(format("%s: expected %s, found %s", name.c_str(), shape_text(spec.shape).c_str(), shape_text(t.shape).c_str()));
            continue;
        }
        if (spec.is_float != dtype_is_float(t.dtype)) {
            wrong_kind.push_back(format("%s: expected %s tensor, found %s", name.c_str(), spec.is_float ? "a floating-point" : "an integer",
                                        dtype_name(t.dtype)));
            continue;
        }
        bound[name] = t;
    }
    for (const auto& kv : found)
        if (!specs.count(kv.first)) unexpected.push_back(kv.first);
    if (!missing.empty() || !unexpected.empty() || !wrong_shape.empty() || !wrong_kind.empty()) {
        std::string msg = where + ": the tensors do not match the model";
        if (!missing.empty()) msg += format("\n  missing (%zu): ", missing.size()) + joined(missing, ", ");
        if (!unexpected.empty()) msg += format("\n  unexpected (%zu): ", unexpected.size()) + joined(unexpected, ", ");
        if (!wrong_shape.empty()) msg += format("\n  wrong shape (%zu): ", wrong_shape.size()) + joined(wrong_shape, "; ");
        if (!wrong_kind.empty()) msg += format("\n  wrong dtype (%zu): ", wrong_kind.size()) + joined(wrong_kind, "; ");
        throw WeightError(msg);
    }
    for (const auto& kv : specs)
        if (!bound.count(kv.first)) bound[kv.first] = bound.at(kv.second.alias_of);   // the same bytes: a tied tensor is really tied
    return bound;
}

HostTensors load_weights(const std::string& folder, const WeightTable& specs) {
    const std::string path = folder + "/model.safetensors";
    if (!file_exists(path)) {
        std::string hint;
        if (file_exists(folder + "/model.safetensors.index.json"))
            hint = " (a sharded checkpoint with model.safetensors.index.json is not supported; merge the shards)";
        throw WeightError(path + ": no such file" + hint);
    }
    return check_and_bind(load_safetensors(path), specs, path);
}

// ------------------------------------------------------------------------------------------------ random weights
namespace {

// Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011): a counter-based generator, so the
// value of (seed, tensor name, index) does not depend on which other tensors or elements exist.
inline void philox(uint32_t c[4], uint32_t k0, uint32_t k1) {
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = 0xD2511F53ull * c[0], p1 = 0xCD9E8D57ull * c[2];
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0, n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
        c[1] = static_cast<uint32_t>(p1);
        c[3] = static_cast<uint32_t>(p0);
        c[0] = n0;
        c[2] = n2;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

uint64_t fnv1a(const std::string& s) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char ch : s) { h ^= ch; h *= 1099511628211ull; }
    return h;
}

void fill_random(const std::string& name, const WeightSpec& spec, uint64_t seed, const RandomInit& init, DType dtype, uint8_t* out, long long numel) {
    const uint64_t key = fnv1a(std::to_string(seed) + ":" + name);
    const uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
    auto work = [&](long long a, long long b) {
        for (long long i = a; i < b; ++i) {
            uint32_t c[4] = {static_cast<uint32_t>(i), static_cast<uint32_t>(static_cast<uint64_t>(i) >> 32), 0u, 0u};
            philox(c, k0, k1);
            const double u = (c[0] + 0.5) / 4294967296.0, v = (c[1] + 0.5) / 4294967296.0;
            float x;
            if (spec.init_ones) x = static_cast<float>(1.0 + (2.0 * u - 1.0) * init.norm_jitter);
            else x = static_cast<float>(std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586 * v) * init.std);
            if (dtype == DType::F32) std::memcpy(out + 4 * i, &x, 4);
            else {
                const uint16_t h = float_to_bf16(x);
                std::memcpy(out + 2 * i, &h, 2);
            }
        }
    };
    const unsigned threads = numel > (1 << 18) ? std::max(1u, std::min(16u, std::thread::hardware_concurrency())) : 1u;
    if (threads == 1) { work(0, numel); return; }
    std::vector<std::thread> pool;
    const long long chunk = (numel + threads - 1) / threads;
    for (unsigned t = 0; t < threads; ++t) {
        const long long a = t * chunk, b = std::min(numel, a + chunk);
        if (a < b) pool.emplace_back(work, a, b);
    }
    for (auto& th : pool) th.join();
}

void make_dirs(const std::string& path) {
    std::string cur;
    for (size_t i = 0; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty()) ::mkdir(cur.c_str(), 0777);
        }
        if (i < path.size()) cur.push_back(path[i]);
    }
}
}  // namespace

std::string write_random_model(const std::string& folder, const json::Value& config, uint64_t seed, const RandomInit& init) {
    const std::string where = "config";
    const PlanFunction plan_of = resolve_architecture(config, where);
    const ModelPlan plan = plan_of(config, where);
    const WeightTable specs = weight_table(plan);
    DType dtype;
    if (init.dtype == "bfloat16") dtype = DType::BF16;
    else if (init.dtype == "float32") dtype = DType::F32;
    else throw ArgumentError(format("random weights are written as bfloat16 or float32, not '%s'", init.dtype.c_str()));
    HostTensors tensors;
    for (const auto& kv : specs) {
        if (!kv.second.alias_of.empty()) continue;           // stored once, under the name it aliases
        if (!kv.second.is_float) throw ConfigError(format("tensor '%s': the random-weights mode has no rule for integer tables", kv.first.c_str()));
        HostTensor t;
        t.dtype = dtype;
        t.shape = kv.second.shape;
        const long long numel = t.numel();
        auto bytes = std::make_shared<std::vector<uint8_t>>(static_cast<size_t>(numel) * dtype_size(dtype));
        fill_random(kv.first, kv.second, seed, init, dtype, bytes->data(), numel);
        t.data = bytes->data();
        t.nbytes = bytes->size();
        t.owner = bytes;
        tensors[kv.first] = std::move(t);
    }
    make_dirs(folder);
    {
        std::ofstream f(folder + "/config.json");
        if (!f) throw WeightError(folder + "/config.json: cannot write");
        f << config.dump(2) << "\n";
    }
    save_safetensors(tensors, folder + "/model.safetensors",
                     {{"format", "pt"}, {"generator", "velomind_b200 random weights"}, {"seed", std::to_string(seed)}});
    return folder;
}

}  // namespace vmb
