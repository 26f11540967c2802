// The C ABI over the C++ API (see c_api.h): every function catches, records the message and returns a status.
#include "velomind_b200/c_api.h"

#include <cstring>

#include "../engine/ops.h"

using namespace vmb;

namespace {

thread_local std::string g_error;
thread_local int g_kind = VMB_ERROR_OTHER;
thread_local std::string g_text;       // the text a function returned last (valid until the thread's next call)

void note(const std::exception& ex) {
    g_error = ex.what();
    if (dynamic_cast<const ConfigError*>(&ex)) g_kind = VMB_ERROR_CONFIG;
    else if (dynamic_cast<const WeightError*>(&ex)) g_kind = VMB_ERROR_WEIGHT;
    else if (dynamic_cast<const CacheError*>(&ex)) g_kind = VMB_ERROR_CACHE;
    else if (dynamic_cast<const KernelError*>(&ex)) g_kind = VMB_ERROR_KERNEL;
    else if (dynamic_cast<const ArgumentError*>(&ex)) g_kind = VMB_ERROR_ARGUMENT;
    else g_kind = VMB_ERROR_OTHER;
}

template <class F> int status(F&& f) {
    try {
        return f();
    } catch (const std::exception& ex) {
        note(ex);
        return -1;
    }
}

template <class F> void* pointer(F&& f) {
    try {
        return f();
    } catch (const std::exception& ex) {
        note(ex);
        return nullptr;
    }
}

template <class F> const char* text(F&& f) {
    try {
        g_text = f();
        return g_text.c_str();
    } catch (const std::exception& ex) {
        note(ex);
        return nullptr;
    }
}

struct ModelHandle { std::shared_ptr<DecoderModel> model; };
struct TokenizerHandle { std::shared_ptr<Tokenizer> tokenizer; };

Engine& engine_of(void* h) {
    if (!h) throw ArgumentError("null engine handle");
    return *static_cast<Engine*>(h);
}
TextEngine& text_of(void* h) {
    if (!h) throw ArgumentError("null text engine handle");
    return *static_cast<TextEngine*>(h);
}

json::Value int_array(const std::vector<int>& v) {
    json::Array a;
    for (int x : v) a.emplace_back(x);
    return json::Value(std::move(a));
}

json::Value results_json(const std::vector<Result>& results, const Timing& timing, bool with_text) {
    json::Array rs;
    for (const Result& r : results) {
        json::Value o;
        o.set("tokens", int_array(r.tokens));
        o.set("finish_reason", r.finish_reason);
        o.set("prompt_tokens", r.prompt_tokens);
        if (with_text) {
            o.set("text", r.text);
            o.set("elapsed_seconds", r.elapsed_seconds);
            o.set("tokens_per_second", r.tokens_per_second);
        }
        rs.push_back(std::move(o));
    }
    json::Value t;
    t.set("prefill_seconds", timing.prefill_seconds);
    t.set("decode_seconds", timing.decode_seconds);
    t.set("decode_steps", timing.decode_steps);
    t.set("generated_tokens", timing.generated_tokens);
    json::Value out;
    out.set("results", json::Value(std::move(rs)));
    out.set("timing", t);
    return out;
}

std::vector<SamplingParams> params_of(int n, const float* temperature, const float* top_p, const long long* seed) {
    std::vector<SamplingParams> p(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) {
        p[i].temperature = temperature[i];
        p[i].top_p = top_p[i];
        p[i].seed = seed[i];
    }
    return p;
}

}  // namespace

extern "C" {

const char* vmb_last_error(void) { return g_error.c_str(); }
int vmb_last_error_kind(void) { return g_kind; }

// ------------------------------------------------------------------------------------------------ configuration and weights
const char* vmb_config_describe(const char* config_json) {
    return text([&] {
        const json::Value cfg = json::parse(config_json, "config.json", false);
        const ModelPlan plan = resolve_architecture(cfg, "config.json")(cfg, "config.json");
        json::Value out;
        out.set("architecture", architecture_name(cfg, "config.json"));
        out.set("hidden_size", plan.hidden_size);
        out.set("vocab_size", plan.vocab_size);
        out.set("layers", static_cast<int>(plan.blocks.size()));
        out.set("runs", static_cast<int>(plan.schedule.size()));
        out.set("max_positions", plan.max_positions);
        out.set("stop_tokens", int_array(plan.stop_tokens));
        out.set("bos_token", plan.bos_token ? json::Value(*plan.bos_token) : json::Value());
        out.set("describe", plan.describe);
        if (architecture_name(cfg, "config.json") == "LlamaForCausalLM") out.set("typed", LlamaConfig::from_json(cfg, "config.json").to_json());
        json::Array blocks;
        for (const BlockSpec& b : plan.blocks) {
            json::Value o;
            o.set("arrangement", b.arrangement);
            o.set("prefix", b.prefix);
            json::Value mixer;
            mixer.set("kind", b.mixer.kind);
            mixer.set("args", b.mixer.args);
            o.set("mixer", mixer);
            json::Value ff;
            ff.set("kind", b.feed_forward.kind);
            ff.set("args", b.feed_forward.args);
            o.set("feed_forward", ff);
            json::Value norm;
            norm.set("kind", b.mixer_norm.kind);
            norm.set("args", b.mixer_norm.args);
            o.set("mixer_norm", norm);
            blocks.push_back(std::move(o));
        }
        out.set("blocks", json::Value(std::move(blocks)));
        return out.dump();
    });
}

const char* vmb_weight_table(const char* config_json) {
    return text([&] {
        const json::Value cfg = json::parse(config_json, "config.json", false);
        const WeightTable table = weight_table(resolve_architecture(cfg, "config.json")(cfg, "config.json"));
        json::Value out;
        out.object();
        for (const auto& kv : table) {
            json::Value o;
            json::Array shape;
            for (long long d : kv.second.shape) shape.emplace_back(d);
            o.set("shape", json::Value(std::move(shape)));
            o.set("float", kv.second.is_float);
            o.set("ones", kv.second.init_ones);
            o.set("alias_of", kv.second.alias_of.empty() ? json::Value() : json::Value(kv.second.alias_of));
            out.set(kv.first, o);
        }
        return out.dump();
    });
}

int vmb_check_model_folder(const char* folder) {
    return status([&] {
        const json::Value cfg = read_config_json(folder);
        const std::string where = std::string(folder) + "/config.json";
        DecoderModel model(resolve_architecture(cfg, where)(cfg, where));
        load_weights(folder, model.weight_table());
        return 0;
    });
}

int vmb_write_random_model(const char* folder, const char* config_json, unsigned long long seed, double std_, double norm_jitter, const char* dtype) {
    return status([&] {
        RandomInit init;
        init.std = std_;
        init.norm_jitter = norm_jitter;
        init.dtype = dtype ? dtype : "bfloat16";
        write_random_model(folder, json::parse(config_json, "config", false), seed, init);
        return 0;
    });
}

int vmb_safetensors_check_header(const char* blob, long long n, long long data_bytes) {
    return status([&] { return static_cast<int>(parse_safetensors_header(std::string(blob, static_cast<size_t>(n)), data_bytes).size()); });
}

const char* vmb_safetensors_info(const char* path) {
    return text([&] {
        json::Value out;
        out.object();
        for (const auto& kv : load_safetensors(path)) {
            json::Value o;
            o.set("dtype", dtype_name(kv.second.dtype));
            json::Array shape;
            for (long long d : kv.second.shape) shape.emplace_back(d);
            o.set("shape", json::Value(std::move(shape)));
            out.set(kv.first, o);
        }
        return out.dump();
    });
}

const char* vmb_registered_architectures(void) {
    return text([&] {
        json::Array a;
        for (const std::string& n : registered_architectures()) a.emplace_back(n);
        return json::Value(std::move(a)).dump();
    });
}

const char* vmb_smollm2_135m_config(void) { return SMOLLM2_135M_CONFIG; }

// ------------------------------------------------------------------------------------------------ tokenizer
void* vmb_tokenizer_load(const char* path) {
    return pointer([&]() -> void* { return new TokenizerHandle{Tokenizer::from_file(path)}; });
}
void* vmb_tokenizer_from_json(const char* tokenizer_json) {
    return pointer([&]() -> void* { return new TokenizerHandle{Tokenizer::from_json(json::parse(tokenizer_json, "tokenizer.json", false), "tokenizer.json")}; });
}
void vmb_tokenizer_free(void* t) { delete static_cast<TokenizerHandle*>(t); }
int vmb_tokenizer_encode(void* t, const char* text_, int* out, int capacity) {
    return status([&] {
        const std::vector<int> ids = static_cast<TokenizerHandle*>(t)->tokenizer->encode(text_);
        for (int i = 0; i < static_cast<int>(ids.size()) && i < capacity; ++i) out[i] = ids[static_cast<size_t>(i)];
        return static_cast<int>(ids.size());
    });
}
const char* vmb_tokenizer_decode(void* t, const int* ids, int n) {
    return text([&] { return static_cast<TokenizerHandle*>(t)->tokenizer->decode(std::vector<int>(ids, ids + n)); });
}
const char* vmb_pretokenize(const char* text_) {
    return text([&] {
        json::Array a;
        for (const std::string& p : Tokenizer::pretokenize(text_)) a.emplace_back(p);
        return json::Value(std::move(a)).dump();
    });
}
int vmb_tokenizer_special(void* t, int which) {
    const Tokenizer& tok = *static_cast<TokenizerHandle*>(t)->tokenizer;
    return which == 0 ? tok.bos_id : which == 1 ? tok.eos_id : which == 2 ? tok.pad_id : tok.unk_id;
}

// ------------------------------------------------------------------------------------------------ model and engine
void* vmb_model_load(const char* folder, const char* dtype, const char* device) {
    return pointer([&]() -> void* { return new ModelHandle{load_model(folder, compute_dtype(dtype), device)}; });
}
void vmb_model_free(void* m) { delete static_cast<ModelHandle*>(m); }

static std::string model_info(const DecoderModel& m) {
    json::Value out;
    out.set("vocab_size", m.plan.vocab_size);
    out.set("hidden_size", m.plan.hidden_size);
    out.set("max_positions", m.plan.max_positions);
    out.set("stop_tokens", int_array(m.plan.stop_tokens));
    out.set("bos_token", m.plan.bos_token ? json::Value(*m.plan.bos_token) : json::Value());
    out.set("runs", static_cast<int>(m.plan.schedule.size()));
    out.set("graph_safe", m.graph_safe());
    out.set("dtype", m.dtype == DType::F32 ? "float32" : "bfloat16");
    out.set("describe", m.plan.describe);
    return out.dump();
}
const char* vmb_model_info(void* m) {
    return text([&] { return model_info(*static_cast<ModelHandle*>(m)->model); });
}

void* vmb_engine_create(void* model, long long max_tokens, int max_slots, int max_step_tokens, int use_graphs, int fused_prefill_rows, int poison_freed) {
    return pointer([&]() -> void* {
        if (!model) throw ArgumentError("null model handle");
        EngineOptions o;
        o.max_tokens = max_tokens;
        o.max_slots = max_slots;
        if (max_step_tokens > 0) o.max_step_tokens = max_step_tokens;
        o.use_graphs = use_graphs;
        o.fused_prefill_rows = fused_prefill_rows;
        o.poison_freed = poison_freed != 0;
        return new Engine(static_cast<ModelHandle*>(model)->model, o);
    });
}
void vmb_engine_free(void* e) { delete static_cast<Engine*>(e); }
int vmb_engine_open(void* e) { return status([&] { return engine_of(e).open(); }); }
int vmb_engine_close(void* e, int slot) { return status([&] { engine_of(e).close(slot); return 0; }); }
int vmb_engine_length(void* e, int slot) {
    return status([&] {
        Engine& en = engine_of(e);
        if (!en.cache->book.slots.is_held(slot)) throw CacheError(format("slot %d is not open", slot));
        return en.length(slot);
    });
}

int vmb_engine_step(void* e, int n_entries, const int* slots, const int* n_tokens, const int* tokens, const int* n_want, const int* want,
                    const float** logits, int* rows) {
    return status([&] {
        std::vector<Entry> entries(static_cast<size_t>(n_entries));
        size_t t = 0, w = 0;
        for (int i = 0; i < n_entries; ++i) {
            entries[i].slot = slots[i];
            entries[i].tokens.assign(tokens + t, tokens + t + n_tokens[i]);
            entries[i].want.assign(want + w, want + w + n_want[i]);
            t += static_cast<size_t>(n_tokens[i]);
            w += static_cast<size_t>(n_want[i]);
        }
        *logits = engine_of(e).step(entries, rows);
        return 0;
    });
}

int vmb_engine_sample(void* e, const float* logits, int rows, const float* temperature, const float* top_p, const long long* seed,
                      const long long* streams, const long long* steps, int* out_tokens) {
    return status([&] {
        const std::vector<int> got = engine_of(e).sample(logits, rows, params_of(rows, temperature, top_p, seed), std::vector<long long>(streams, streams + rows),
                                                         std::vector<long long>(steps, steps + rows));
        std::memcpy(out_tokens, got.data(), got.size() * sizeof(int));
        return 0;
    });
}

int vmb_engine_decode_many(void* e, int n, const int* slots, const int* last_tokens, const float* temperature, const float* top_p,
                           const long long* seed, const long long* streams, const long long* steps, int k, int* out_tokens) {
    return status([&] {
        const auto rows = engine_of(e).decode_many(std::vector<int>(slots, slots + n), std::vector<int>(last_tokens, last_tokens + n),
                                                   params_of(n, temperature, top_p, seed), std::vector<long long>(streams, streams + n),
                                                   std::vector<long long>(steps, steps + n), k);
        for (size_t i = 0; i < rows.size(); ++i) std::memcpy(out_tokens + i * static_cast<size_t>(n), rows[i].data(), static_cast<size_t>(n) * sizeof(int));
        return 0;
    });
}

int vmb_engine_synchronize(void* e) { return status([&] { engine_of(e).synchronize(); return 0; }); }
int vmb_engine_raise_if_error(void* e) { return status([&] { engine_of(e).raise_if_error(); return 0; }); }
int vmb_engine_logits_to_host(void* e, const float* dev, int rows, float* host) {
    return status([&] { engine_of(e).copy_logits_to_host(dev, rows, host); return 0; });
}
int vmb_engine_cache_check(void* e) { return status([&] { engine_of(e).cache->book.check(); return 0; }); }
int vmb_engine_set_fail_after(void* e, long long n) { return status([&] { engine_of(e).ws.fail_after = n; return 0; }); }
unsigned long long vmb_engine_stream(void* e) { return e ? reinterpret_cast<unsigned long long>(static_cast<Engine*>(e)->stream) : 0ull; }

const char* vmb_engine_stats(void* e) {
    return text([&] {
        Engine& en = engine_of(e);
        const CacheBook& book = en.cache->book;
        json::Value c;
        c.set("own_launches", en.counters.own_launches);
        c.set("library_calls", en.counters.library_calls);
        c.set("h2d_bytes", en.counters.h2d_bytes);
        c.set("d2h_bytes", en.counters.d2h_bytes);
        c.set("steps", en.counters.steps);
        c.set("graphs_recorded", en.counters.graphs_recorded);
        c.set("tc_attention_calls", en.counters.tc_attention_calls);
        json::Value cache;
        cache.set("n_pages", book.n_pages);
        cache.set("max_slots", book.max_slots);
        cache.set("max_positions", book.max_positions);
        cache.set("slots_held", book.slots.held_count());
        cache.set("tokens_held", book.tokens_held());
        json::Array groups;
        for (size_t g = 0; g < book.groups.size(); ++g) {
            json::Value o;
            o.set("kind", book.groups[g].need.kind == CacheNeed::Window ? "window" : "all");
            o.set("window", book.groups[g].need.window);
            o.set("layers", book.layers_in_group[g]);
            o.set("pages_held", book.groups[g].pages.held_count());
            o.set("pages_free", book.groups[g].pages.free_count());
            groups.push_back(std::move(o));
        }
        cache.set("groups", json::Value(std::move(groups)));
        json::Value out;
        out.set("counters", c);
        out.set("cache", cache);
        out.set("vocab", en.vocab);
        out.set("dtype", en.dtype == DType::F32 ? "float32" : "bfloat16");
        out.set("use_graphs", en.use_graphs);
        out.set("arena_bytes", static_cast<long long>(en.ws.arena_bytes()));
        out.set("arena_generation", static_cast<long long>(en.ws.generation));
        return out.dump();
    });
}

const char* vmb_engine_generate(void* e, int n, const int* prompt_lens, const int* prompts, const float* temperature, const float* top_p,
                                const int* max_tokens, const long long* seed, const long long* streams, const int* n_stop, const int* stops,
                                int n_default_stop, const int* default_stop, int max_batch, int steps_per_sync, vmb_token_callback on_token, void* user) {
    return text([&] {
        Engine& en = engine_of(e);
        std::vector<Request> requests(static_cast<size_t>(n));
        size_t p = 0, s = 0;
        for (int i = 0; i < n; ++i) {
            Request& r = requests[static_cast<size_t>(i)];
            r.prompt.assign(prompts + p, prompts + p + prompt_lens[i]);
            p += static_cast<size_t>(prompt_lens[i]);
            r.params.temperature = temperature[i];
            r.params.top_p = top_p[i];
            r.params.max_tokens = max_tokens[i];
            r.params.seed = seed[i];
            r.stream = streams[i];
            if (n_stop[i] > 0) {
                r.params.stop_tokens.assign(stops + s, stops + s + n_stop[i]);
                s += static_cast<size_t>(n_stop[i]);
            }
        }
        EngineStepper stepper(en);
        GenerationLoop loop(stepper, en.cache->book.n_pages, max_batch, std::vector<int>(default_stop, default_stop + std::max(n_default_stop, 0)), steps_per_sync);
        TokenCallback cb;
        if (on_token) cb = [&](int i, int tok) { on_token(user, i, tok); };
        const std::vector<Result> results = loop.run(requests, cb);
        return results_json(results, loop.timing, false).dump();
    });
}

// ------------------------------------------------------------------------------------------------ the text engine
void* vmb_text_create(const char* engine_config_json) {
    return pointer([&]() -> void* {
        const json::Value j = json::parse(engine_config_json, "engine configuration", false);
        KeyReader r(j, "engine configuration");
        EngineConfig c;
        c.model_path = r.string_or("model_path", "");
        c.tokenizer_path = r.string_or("tokenizer_path", "");
        c.device = r.string_or("device", "cuda:0");
        c.use_synthetic = r.boolean_or("use_synthetic", false);
        if (const json::Value* mc = j.find("model_config")) c.model_config = *mc;
        c.seed = r.integer_or("seed", 42, 0);
        c.dtype = r.string_or("dtype", "bfloat16");
        c.max_tokens = r.integer_or("max_tokens", 65536);
        c.max_batch = static_cast<int>(r.integer_or("max_batch", 64));
        c.use_graphs = static_cast<int>(r.integer_or("use_graphs", -1, -1));
        return new TextEngine(c);
    });
}
void vmb_text_free(void* t) { delete static_cast<TextEngine*>(t); }
int vmb_text_load(void* t) { return status([&] { text_of(t).load(); return 0; }); }
void* vmb_text_engine(void* t) { return t ? static_cast<TextEngine*>(t)->engine.get() : nullptr; }
void* vmb_text_model(void* t) {
    return pointer([&]() -> void* { return new ModelHandle{text_of(t).model}; });
}
void* vmb_text_tokenizer(void* t) {
    return pointer([&]() -> void* { return text_of(t).tokenizer ? new TokenizerHandle{text_of(t).tokenizer} : nullptr; });
}
const char* vmb_text_describe(void* t) {
    return text([&] { return text_of(t).describe().dump(); });
}

const char* vmb_text_generate(void* t, int n, const int* prompt_lens, const int* prompts, const char* options_json, vmb_piece_callback on_token,
                              vmb_sample_callback sample_fn, void* user) {
    return text([&] {
        TextEngine& te = text_of(t);
        const json::Value j = json::parse(options_json && *options_json ? options_json : "{}", "generation options", false);
        KeyReader r(j, "generation options");
        GenerateOptions o;
        o.temperature = static_cast<float>(r.number_or("temperature", 0.7, false));
        o.top_p = static_cast<float>(r.number_or("top_p", 0.9, false));
        o.max_tokens = static_cast<int>(r.integer_or("max_tokens", 32, 0));
        o.seed = r.integer_or("seed", 42, 0);
        o.steps_per_sync = static_cast<int>(r.integer_or("steps_per_sync", 1));
        if (r.has("stop_tokens")) o.stop_tokens = r.int_or_list("stop_tokens");
        if (on_token) o.on_token = [&](int i, int tok, const std::string& piece) { on_token(user, i, tok, piece.c_str()); };
        if (sample_fn) o.sample_fn = [&](const float* row, int vocab) { return sample_fn(user, row, vocab); };
        std::vector<std::vector<int>> ps(static_cast<size_t>(n));
        size_t p = 0;
        for (int i = 0; i < n; ++i) {
            ps[static_cast<size_t>(i)].assign(prompts + p, prompts + p + prompt_lens[i]);
            p += static_cast<size_t>(prompt_lens[i]);
        }
        const std::vector<Result> results = te.generate(ps, o);
        return results_json(results, te.last_timing, true).dump();
    });
}

int vmb_text_reset_session(void* t) { return status([&] { text_of(t).reset_session(); return 0; }); }
int vmb_text_session_length(void* t) { return status([&] { return text_of(t).session_length(); }); }
int vmb_text_prefill(void* t, const int* tokens, int n, float* logits) {
    return status([&] {
        const std::vector<float> l = text_of(t).prefill(std::vector<int>(tokens, tokens + n));
        std::memcpy(logits, l.data(), l.size() * sizeof(float));
        return 0;
    });
}
int vmb_text_forward_step(void* t, int token, long long pos, float* logits) {
    return status([&] {
        const std::vector<float> l = text_of(t).forward_step(token, pos);
        std::memcpy(logits, l.data(), l.size() * sizeof(float));
        return 0;
    });
}
int vmb_text_forward_logits(void* t, const int* tokens, int n, float* logits) {
    return status([&] {
        const std::vector<float> l = text_of(t).forward_logits(std::vector<int>(tokens, tokens + n));
        std::memcpy(logits, l.data(), l.size() * sizeof(float));
        return 0;
    });
}
int vmb_text_forward_full_logits(void* t, const int* tokens, int n, float* logits) {
    return status([&] {
        const std::vector<float> l = text_of(t).forward_full_logits(std::vector<int>(tokens, tokens + n));
        std::memcpy(logits, l.data(), l.size() * sizeof(float));
        return 0;
    });
}

// ------------------------------------------------------------------------------------------------ debugging aids
void* vmb_op_times_begin(void) {
    return pointer([&]() -> void* { return new ops::OpTimes(); });
}
const char* vmb_op_times_table(void* h) {
    return text([&] { return static_cast<ops::OpTimes*>(h)->table(); });
}
void vmb_op_times_end(void* h) { delete static_cast<ops::OpTimes*>(h); }

}  // extern "C"
