// Typed reading of config.json keys with errors that name the key; the Llama configuration; the registry from an
// architecture's name to its model; dtype helpers.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <sys/stat.h>

#include "velomind_b200/velomind.h"

namespace vmb {

// ------------------------------------------------------------------------------------------------ dtypes
size_t dtype_size(DType t) {
    switch (t) {
        case DType::F32: case DType::I32: return 4;
        case DType::BF16: case DType::F16: case DType::I16: return 2;
        case DType::I64: return 8;
        case DType::I8: case DType::U8: case DType::BOOL: return 1;
    }
    return 0;
}

const char* dtype_name(DType t) {
    switch (t) {
        case DType::F32: return "F32";
        case DType::BF16: return "BF16";
        case DType::F16: return "F16";
        case DType::I32: return "I32";
        case DType::I64: return "I64";
        case DType::I16: return "I16";
        case DType::I8: return "I8";
        case DType::U8: return "U8";
        case DType::BOOL: return "BOOL";
    }
    return "?";
}

std::optional<DType> dtype_from_name(const std::string& n) {
    static const std::pair<const char*, DType> table[] = {
        {"F32", DType::F32}, {"BF16", DType::BF16}, {"F16", DType::F16}, {"I32", DType::I32}, {"I64", DType::I64},
        {"I16", DType::I16}, {"I8", DType::I8}, {"U8", DType::U8}, {"BOOL", DType::BOOL}};
    for (const auto& e : table)
        if (n == e.first) return e.second;
    return std::nullopt;
}

bool dtype_is_float(DType t) { return t == DType::F32 || t == DType::BF16 || t == DType::F16; }

uint16_t float_to_bf16(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);   // NaN stays NaN
    u += 0x7fffu + ((u >> 16) & 1u);                                                        // round to nearest even
    return static_cast<uint16_t>(u >> 16);
}

float bf16_to_float(uint16_t x) {
    const uint32_t u = static_cast<uint32_t>(x) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

float f16_to_float(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {                                   // subnormal: normalise
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            u = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

DType compute_dtype(const std::string& name) {
    if (name == "bfloat16" || name == "bf16") return DType::BF16;
    if (name == "float32" || name == "fp32") return DType::F32;
    throw ArgumentError(format("dtype '%s': choose bfloat16 or float32", name.c_str()));
}

// ------------------------------------------------------------------------------------------------ KeyReader
KeyReader::KeyReader(const json::Value& data, std::string where) : data_(data), where_(std::move(where)) {
    if (!data.is_object()) throw ConfigError(where_ + ": top level is not a JSON object");
}

const json::Value* KeyReader::get(const std::string& key) const {
    const json::Value* v = data_.find(key);
    return (v && !v->is_null()) ? v : nullptr;
}

bool KeyReader::has(const std::string& key) const { return get(key) != nullptr; }

static std::string shown(const json::Value& v) { return v.dump(); }

long long KeyReader::integer(const std::string& key, long long minimum) const {
    const json::Value* v = get(key);
    if (!v) throw ConfigError(format("%s: missing required key '%s'", where_.c_str(), key.c_str()));
    if (!v->is_integer()) throw ConfigError(format("%s: key '%s' must be an integer, found %s", where_.c_str(), key.c_str(), shown(*v).c_str()));
    if (v->as_int() < minimum)
        throw ConfigError(format("%s: key '%s' must be >= %lld, found %lld", where_.c_str(), key.c_str(), minimum, v->as_int()));
    return v->as_int();
}

long long KeyReader::integer_or(const std::string& key, long long fallback, long long minimum) const {
    return get(key) ? integer(key, minimum) : fallback;
}

double KeyReader::number(const std::string& key, bool positive) const {
    const json::Value* v = get(key);
    if (!v) throw ConfigError(format("%s: missing required key '%s'", where_.c_str(), key.c_str()));
    if (!v->is_number() || !std::isfinite(v->as_double()))
        throw ConfigError(format("%s: key '%s' must be a finite number, found %s", where_.c_str(), key.c_str(), shown(*v).c_str()));
    if (positive && v->as_double() <= 0)
        throw ConfigError(format("%s: key '%s' must be > 0, found %s", where_.c_str(), key.c_str(), shown(*v).c_str()));
    return v->as_double();
}

double KeyReader::number_or(const std::string& key, double fallback, bool positive) const {
    return get(key) ? number(key, positive) : fallback;
}

bool KeyReader::boolean_or(const std::string& key, bool fallback) const {
    const json::Value* v = get(key);
    if (!v) return fallback;
    if (!v->is_bool()) throw ConfigError(format("%s: key '%s' must be true or false, found %s", where_.c_str(), key.c_str(), shown(*v).c_str()));
    return v->as_bool();
}

std::string KeyReader::string_or(const std::string& key, const std::string& fallback) const {
    const json::Value* v = get(key);
    if (!v) return fallback;
    if (!v->is_string()) throw ConfigError(format("%s: key '%s' must be a string, found %s", where_.c_str(), key.c_str(), shown(*v).c_str()));
    return v->as_string();
}

std::vector<int> KeyReader::int_or_list(const std::string& key) const {
    const json::Value* v = get(key);
    std::vector<int> out;
    if (!v) return out;
    auto one = [&](const json::Value& x) {
        if (!x.is_integer() || x.is_bool())
            throw ConfigError(format("%s: key '%s' must be an integer or a list of integers, found %s", where_.c_str(), key.c_str(), shown(*v).c_str()));
        out.push_back(static_cast<int>(x.as_int()));
    };
    if (v->is_array()) for (const auto& x : v->as_array()) one(x);
    else one(*v);
    return out;
}

void KeyReader::absent_or(const std::string& key, const std::vector<json::Value>& allowed, const std::string& why) const {
    const json::Value* v = get(key);
    if (!v) return;
    for (const auto& a : allowed)
        if (a == *v) return;
    throw ConfigError(format("%s: key '%s' = %s is not supported (%s)", where_.c_str(), key.c_str(), shown(*v).c_str(), why.c_str()));
}

static bool is_dir(const std::string& p) {
    struct stat st;
    return ::stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

json::Value read_config_json(const std::string& folder_or_file) {
    std::string path = folder_or_file;
    if (is_dir(path)) path += "/config.json";
    std::ifstream f(path, std::ios::binary);
    if (!f) throw ConfigError(path + ": no such file (a model folder holds config.json and model.safetensors)");
    std::stringstream ss;
    ss << f.rdbuf();
    json::Value data;
    try {
        data = json::parse(ss.str(), path, /*no_duplicate_keys=*/false);
    } catch (const Error& e) {
        throw ConfigError(e.what());
    }
    if (!data.is_object()) throw ConfigError(path + ": top level is not a JSON object");
    return data;
}

// ------------------------------------------------------------------------------------------------ LlamaConfig
namespace {
// llama_config.h:22 — what the reference's struct holds when config.json gives no context limit.
constexpr int kDefaultMaxPositions = 2048;
}  // namespace

LlamaConfig LlamaConfig::from_json(const json::Value& data, const std::string& where) {
    KeyReader r(data, where);
    LlamaConfig c;
    c.hidden_size = static_cast<int>(r.integer("hidden_size"));
    c.num_attention_heads = static_cast<int>(r.integer("num_attention_heads"));
    // llama_config.h:14-16: zero kv heads means "as many as heads".
    c.num_key_value_heads = static_cast<int>(r.integer("num_key_value_heads", 0));
    if (c.num_key_value_heads == 0) c.num_key_value_heads = c.num_attention_heads;
    if (c.num_attention_heads % c.num_key_value_heads != 0)      // llama_graph.cpp:179-182
        throw ConfigError(format("%s: num_attention_heads (%d) must be divisible by num_key_value_heads (%d)", where.c_str(),
                                 c.num_attention_heads, c.num_key_value_heads));
    if (r.has("head_dim")) c.head_dim = static_cast<int>(r.integer("head_dim"));
    else {
        if (c.hidden_size % c.num_attention_heads != 0)          // llama_graph.cpp:172-174
            throw ConfigError(format("%s: hidden_size (%d) must be divisible by num_attention_heads (%d)", where.c_str(), c.hidden_size,
                                     c.num_attention_heads));
        c.head_dim = c.hidden_size / c.num_attention_heads;      // llama_config.h:17-19
    }
    if (c.head_dim % 2 != 0) throw ConfigError(format("%s: head size %d is odd; rotary pairs need an even size", where.c_str(), c.head_dim));
    r.absent_or("rope_scaling", {}, "scaled rotary positions are not implemented");
    r.absent_or("attention_bias", {json::Value(false)}, "projection biases are not implemented");
    r.absent_or("mlp_bias", {json::Value(false)}, "feed-forward biases are not implemented");
    r.absent_or("hidden_act", {json::Value("silu")}, "the feed-forward gate is SiLU");
    r.absent_or("sliding_window", {}, "this architecture attends to all earlier tokens");
    if (r.has("bos_token_id")) {
        const json::Value* b = data.find("bos_token_id");
        if (!b->is_integer()) throw ConfigError(format("%s: key 'bos_token_id' must be an integer, found %s", where.c_str(), b->dump().c_str()));
        c.bos_token_id = static_cast<int>(b->as_int());
    }
    c.vocab_size = static_cast<int>(r.integer("vocab_size"));
    c.intermediate_size = static_cast<int>(r.integer("intermediate_size"));
    c.num_hidden_layers = static_cast<int>(r.integer("num_hidden_layers"));
    c.rms_norm_eps = r.number("rms_norm_eps");
    c.rope_theta = r.number("rope_theta");
    // config_parser.cpp:213 falls back to the tied constant of examples/smollm2/model.h:21
    c.tie_word_embeddings = r.boolean_or("tie_word_embeddings", true);
    c.max_position_embeddings = static_cast<int>(r.integer_or("max_position_embeddings", kDefaultMaxPositions));
    c.eos_token_ids = r.int_or_list("eos_token_id");
    std::vector<int> special = c.eos_token_ids;
    if (c.bos_token_id) special.push_back(*c.bos_token_id);
    for (int t : special)
        if (t < 0 || t >= c.vocab_size)
            throw ConfigError(format("%s: special token id %d lies outside the vocabulary of %d", where.c_str(), t, c.vocab_size));
    return c;
}

json::Value LlamaConfig::to_json() const {
    json::Value d;
    d.set("architectures", json::Array{json::Value("LlamaForCausalLM")});
    d.set("model_type", "llama");
    d.set("vocab_size", vocab_size);
    d.set("hidden_size", hidden_size);
    d.set("intermediate_size", intermediate_size);
    d.set("num_hidden_layers", num_hidden_layers);
    d.set("num_attention_heads", num_attention_heads);
    d.set("num_key_value_heads", num_key_value_heads);
    d.set("head_dim", head_dim);
    d.set("rms_norm_eps", rms_norm_eps);
    d.set("rope_theta", rope_theta);
    d.set("tie_word_embeddings", tie_word_embeddings);
    d.set("max_position_embeddings", max_position_embeddings);
    d.set("hidden_act", "silu");
    if (eos_token_ids.size() == 1) d.set("eos_token_id", eos_token_ids[0]);
    else if (!eos_token_ids.empty()) {
        json::Array a;
        for (int t : eos_token_ids) a.emplace_back(t);
        d.set("eos_token_id", std::move(a));
    }
    if (bos_token_id) d.set("bos_token_id", *bos_token_id);
    return d;
}

// ------------------------------------------------------------------------------------------------ plan
void ModelPlan::validate() const {
    const int n = static_cast<int>(blocks.size());
    for (size_t i = 0; i < schedule.size(); ++i) {
        const ScheduleEntry& e = schedule[i];
        if (e.layer < 0 || e.layer >= n) throw ConfigError(format("schedule[%zu] names layer %d, the plan has %d", i, e.layer, n));
        if (e.cache_of >= 0) {
            if (e.cache_of >= static_cast<int>(i))
                throw ConfigError(format("schedule[%zu] reads the cache of run %d, which does not come before it", i, e.cache_of));
            if (schedule[e.cache_of].cache_of >= 0)
                throw ConfigError(format("schedule[%zu] reads the cache of run %d, which owns none", i, e.cache_of));
        }
    }
}

// ------------------------------------------------------------------------------------------------ registry
// The reference has no such table (the model family is fixed at compile time, examples/smollm2/smollm2_engine.cpp:43-68);
// here config.json chooses.
namespace {
std::map<std::string, PlanFunction>& architectures() {
    static std::map<std::string, PlanFunction> table;
    return table;
}
std::mutex& registry_lock() {
    static std::mutex m;
    return m;
}
std::string joined(const std::vector<std::string>& v) {
    if (v.empty()) return "(none)";
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + v[i];
    return s;
}
}  // namespace

void register_architecture(const std::string& name, PlanFunction plan) {
    std::lock_guard<std::mutex> g(registry_lock());
    architectures()[name] = std::move(plan);
}

void unregister_architecture(const std::string& name) {
    std::lock_guard<std::mutex> g(registry_lock());
    architectures().erase(name);
}

std::vector<std::string> registered_architectures() {
    std::lock_guard<std::mutex> g(registry_lock());
    std::vector<std::string> out;
    for (const auto& kv : architectures()) out.push_back(kv.first);
    return out;
}

std::string architecture_name(const json::Value& config, const std::string& where) {
    const json::Value* a = config.find("architectures");
    if (!a || !a->is_array() || a->as_array().empty() || !a->as_array()[0].is_string())
        throw ConfigError(where + ": missing required key 'architectures' (a list whose first entry names the model class)");
    return a->as_array()[0].as_string();
}

const PlanFunction& resolve_architecture(const json::Value& config, const std::string& where) {
    const std::string name = architecture_name(config, where);
    {
        std::lock_guard<std::mutex> g(registry_lock());
        auto it = architectures().find(name);
        if (it != architectures().end()) return it->second;
    }
    throw ConfigError(format("%s: architecture '%s' is not registered; registered: %s", where.c_str(), name.c_str(),
                             joined(registered_architectures()).c_str()));
}

}  // namespace vmb
