// The entry point: load a model folder (or make a random one) and generate.
//
// Names follow the reference's engine facade (examples/smollm2/smollm2_engine.h:16-81,
// examples/common/llama/llama_engine.h:59-155): an EngineConfig with model_path, tokenizer_path, device, use_synthetic,
// model_config; load(); generate(...); and the single-session calls prefill, forward_step, forward_logits,
// forward_full_logits, reset_session.  Unlike the reference, generate takes a batch of prompts, and config.json chooses the
// model class.
#include <chrono>
#include <cstdlib>
#include <sys/stat.h>
#include <unistd.h>

#include "ops.h"

namespace vmb {

namespace {
bool is_file(const std::string& p) {
    struct stat st;
    return ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

std::string temp_folder() {
    const char* base = std::getenv("TMPDIR");
    std::string tmpl = std::string(base && *base ? base : "/tmp") + "/velomind_b200_synthetic_XXXXXX";
    std::vector<char> buf(tmpl.begin(), tmpl.end());
    buf.push_back('\0');
    if (!::mkdtemp(buf.data())) throw Error("cannot create a temporary folder for the random model");
    return std::string(buf.data());
}

void remove_model_folder(const std::string& folder) {
    ::unlink((folder + "/config.json").c_str());
    ::unlink((folder + "/model.safetensors").c_str());
    ::rmdir(folder.c_str());
}
}  // namespace

TextEngine::TextEngine(EngineConfig c) : config(std::move(c)) {}

TextEngine::~TextEngine() {
    engine.reset();
    model.reset();
}

TextEngine& TextEngine::load() {
    const DType dt = compute_dtype(config.dtype);
    std::string folder = config.model_path;
    std::string made;
    if (config.use_synthetic) {
        const json::Value cfg = config.model_config.is_object() ? config.model_config : json::parse(SMOLLM2_135M_CONFIG, "the built-in configuration");
        made = temp_folder();
        folder = write_random_model(made, cfg, static_cast<uint64_t>(config.seed));
    } else if (folder.empty()) {
        throw ArgumentError("EngineConfig.model_path is empty (or set use_synthetic)");
    }
    if (is_file(folder)) {                           // the reference takes the path of model.safetensors itself
        const size_t slash = folder.find_last_of('/');
        folder = slash == std::string::npos ? "." : folder.substr(0, slash);
    }
    try {
        model = load_model(folder, dt, config.device);
    } catch (...) {
        if (!made.empty()) remove_model_folder(made);
        throw;
    }
    if (!made.empty()) remove_model_folder(made);
    EngineOptions o;
    o.max_tokens = config.max_tokens;
    o.use_graphs = config.use_graphs;
    engine = std::make_unique<Engine>(model, o);
    const std::string tok_path = !config.tokenizer_path.empty() ? config.tokenizer_path : folder + "/tokenizer.json";
    if (made.empty() && is_file(tok_path)) tokenizer = Tokenizer::from_file(tok_path);
    else if (!config.tokenizer_path.empty() && is_file(config.tokenizer_path)) tokenizer = Tokenizer::from_file(config.tokenizer_path);
    return *this;
}

std::vector<int> TextEngine::encode(const std::string& prompt) const {
    if (!tokenizer) throw ArgumentError("a text prompt needs tokenizer.json; pass token ids instead");
    std::vector<int> ids = tokenizer->encode(prompt);
    const int bos = tokenizer->bos_id;
    if (bos >= 0 && (ids.empty() || ids[0] != bos)) ids.insert(ids.begin(), bos);
    return ids;
}

std::vector<int> TextEngine::default_stop_tokens() const {
    if (tokenizer && tokenizer->eos_id >= 0) return {tokenizer->eos_id};
    return model ? model->plan.stop_tokens : std::vector<int>{};
}

std::vector<Result> TextEngine::generate_text(const std::vector<std::string>& prompts, const GenerateOptions& options) {
    std::vector<std::vector<int>> ids;
    for (const std::string& p : prompts) ids.push_back(encode(p));
    return generate(ids, options);
}

std::vector<Result> TextEngine::generate(const std::vector<std::vector<int>>& prompts, const GenerateOptions& o) {
    if (!engine) throw Error("call load() first");
    const std::vector<int> stops = o.stop_tokens ? *o.stop_tokens : default_stop_tokens();
    std::vector<Request> requests;
    for (size_t i = 0; i < prompts.size(); ++i) {
        Request r;
        r.prompt = prompts[i];
        r.params.temperature = o.temperature;
        r.params.top_p = o.top_p;
        r.params.max_tokens = o.max_tokens;
        r.params.seed = o.seed;
        r.params.stop_tokens = stops;
        r.stream = static_cast<long long>(i);
        requests.push_back(std::move(r));
    }
    EngineStepper stepper(*engine);
    stepper.sample_fn = o.sample_fn;
    // (a host sampling function runs after every step; and an explicit empty stop list means "never stop early")
    GenerationLoop loop(stepper, engine->cache->book.n_pages, config.max_batch, o.stop_tokens && o.stop_tokens->empty() ? std::vector<int>{} : stops,
                        o.sample_fn ? 1 : o.steps_per_sync);
    std::vector<TextStreamer> streamers(prompts.size(), TextStreamer(tokenizer));
    TokenCallback callback;
    if (o.on_token) callback = [&](int i, int tok) { o.on_token(i, tok, streamers[static_cast<size_t>(i)].put(tok)); };
    const auto t0 = std::chrono::steady_clock::now();
    std::vector<Result> results = loop.run(requests, callback);
    const double elapsed = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    last_timing = loop.timing;
    engine->raise_if_error();
    for (size_t i = 0; i < results.size(); ++i) {                 // the reference's result fields (llama_engine.h:32-38)
        Result& res = results[i];
        if (tokenizer) res.text = tokenizer->decode(res.tokens);
        else for (int t : res.tokens) res.text += format("[%d]", t);
        res.elapsed_seconds = elapsed;
        res.tokens_per_second = elapsed > 0 ? res.tokens.size() / elapsed : 0.0;
        // what the streamer still holds back (an incomplete character at the very end), with token -1, as the reference's loop
        // closes its stream (llama_engine.cpp:654-655)
        if (o.on_token) {
            const std::string rest = streamers[i].flush();
            if (!rest.empty()) o.on_token(static_cast<int>(i), -1, rest);
        }
    }
    return results;
}

json::Value TextEngine::describe() const {
    json::Value d;
    d.set("Backend", config.device);
    d.set("Mode", config.use_synthetic ? "Synthetic" : "Real model");
    if (model && model->plan.describe.is_object())
        for (const auto& m : model->plan.describe.as_object()) d.set(m.first, m.second);
    d.set("Dtype", config.dtype);
    return d;
}

// ---- the reference's single-session calls
void TextEngine::reset_session() {
    if (session_slot_ >= 0 && engine) engine->close(session_slot_);
    session_slot_ = -1;
}

int TextEngine::session_length() const { return session_slot_ < 0 ? 0 : engine->length(session_slot_); }

namespace {
std::vector<float> host_rows(Engine& e, const float* dev, int rows) {
    std::vector<float> out(static_cast<size_t>(rows) * e.vocab);
    e.copy_logits_to_host(dev, rows, out.data());
    return out;
}
}  // namespace

// Start a session with `tokens`; float32 logits [vocab] of the last one (llama_engine.cpp:333-393).
std::vector<float> TextEngine::prefill(const std::vector<int>& tokens) {
    if (!engine) throw Error("call load() first");
    if (tokens.empty()) throw ArgumentError("prefill: no tokens");
    reset_session();
    session_slot_ = engine->open();
    int rows = 0;
    const float* l = engine->step({Entry{session_slot_, tokens, {static_cast<int>(tokens.size()) - 1}}}, &rows);
    return host_rows(*engine, l, rows);
}

// Feed one more token to the session; logits [vocab] (llama_engine.cpp:395-455).  `pos`, the reference's second argument, is
// the token's place in the session: it can only be the session's length, and is checked when given.
std::vector<float> TextEngine::forward_step(int token, long long pos) {
    if (session_slot_ < 0) throw Error("forward_step needs a session: call prefill first");
    if (pos >= 0 && pos != session_length()) throw ArgumentError(format("forward_step: pos %lld is not the session's length %d", pos, session_length()));
    int rows = 0;
    const float* l = engine->step({Entry{session_slot_, {token}, {0}}}, &rows);
    return host_rows(*engine, l, rows);
}

// Stateless: logits [len, vocab] of a whole sequence (llama_engine.cpp:523-585).
std::vector<float> TextEngine::forward_full_logits(const std::vector<int>& tokens) {
    if (!engine) throw Error("call load() first");
    const int slot = engine->open();
    try {
        std::vector<int> want(tokens.size());
        for (size_t i = 0; i < want.size(); ++i) want[i] = static_cast<int>(i);
        int rows = 0;
        const float* l = engine->step({Entry{slot, tokens, want}}, &rows);
        std::vector<float> out = host_rows(*engine, l, rows);
        engine->close(slot);
        return out;
    } catch (...) {
        try { engine->close(slot); } catch (...) {}
        throw;
    }
}

// Stateless: logits [vocab] of the last token (llama_engine.cpp:457-521).
std::vector<float> TextEngine::forward_logits(const std::vector<int>& tokens) {
    if (!engine) throw Error("call load() first");
    if (tokens.empty()) throw ArgumentError("forward_logits: no tokens");
    const int slot = engine->open();
    try {
        int rows = 0;
        const float* l = engine->step({Entry{slot, tokens, {static_cast<int>(tokens.size()) - 1}}}, &rows);
        std::vector<float> out = host_rows(*engine, l, rows);
        engine->close(slot);
        return out;
    } catch (...) {
        try { engine->close(slot); } catch (...) {}
        throw;
    }
}

}  // namespace vmb
