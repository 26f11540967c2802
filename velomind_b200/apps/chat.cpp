// Command line in the manner of the reference's `smollm2_chat` (examples/smollm2/interactive_main.cpp:21-137): the same
// option names and defaults where it has them.
//
//   --device <cuda[:N]>   target device (the reference also takes cpu and ispc; this library has CUDA only)
//   --model <path>        model folder (config.json + model.safetensors), or the path of model.safetensors
//   --tokenizer <path>    tokenizer.json (default: the one in the model folder, if any)
//   --synthetic           random weights at the SmolLM2-135M sizes (or --config) instead of a model folder
//   --temp <float>        sampling temperature (default 0.7, 0 for greedy)
//   --top-p <float>       nucleus sampling top-p (default 0.9)
//   --max-tokens <int>    max generated tokens per turn (default 32)
//   --prompt <string>     single non-interactive prompt; without it a `>>>` loop reads prompts and the reference console's
//                         commands (examples/common/llama/llama_interactive_console.cpp:125-309):
//                         /help /temp /top_p /max /system /clear /history /model /save /load /exit /quit
// Additions: --prompt-ids 1,2,3 (token ids, for models without a tokenizer), --prompt-file <path>, --seed (default 42, the
// reference's fixed seed), --dtype bfloat16|float32 (--fp32 for short), --config <config.json> for --synthetic, --op-times
// (device time per kind of operation after each response).  The reference's --download is not offered (no network).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include "../engine/ops.h"

namespace vmb {

namespace {

struct ChatArgs {
    std::string device = "cuda:0", model, tokenizer, config, prompt, prompt_ids, prompt_file, dtype = "bfloat16";
    bool synthetic = false, op_times = false;
    float temp = 0.7f, top_p = 0.9f;
    int max_tokens = 32;
    long long seed = 42;
};

const char* const kUsage =
    "Usage: smollm2_chat [options]\n"
    "  --device <cuda[:N]>   Target device (default: cuda:0)\n"
    "  --model <path>        Model folder (config.json + model.safetensors) or path of model.safetensors\n"
    "  --tokenizer <path>    Path to tokenizer.json (default: the one in the model folder)\n"
    "  --synthetic           Use random weights (SmolLM2-135M sizes, or --config <config.json>)\n"
    "  --config <path>       config.json for --synthetic\n"
    "  --temp <float>        Sampling temperature (default: 0.7, 0 for greedy)\n"
    "  --top-p <float>       Nucleus sampling top-p (default: 0.9)\n"
    "  --max-tokens <int>    Max generated tokens per turn (default: 32)\n"
    "  --prompt <string>     Single non-interactive prompt\n"
    "  --prompt-ids <ids>    Single non-interactive prompt as token ids: 1,2,3\n"
    "  --prompt-file <path>  A file holding the prompt: text, or token ids when the model has no tokenizer\n"
    "  --seed <int>          Sampling seed (default: 42)\n"
    "  --dtype <name>        bfloat16 (default) or float32; --fp32 is short for --dtype float32\n"
    "  --op-times            After each response, print the device time per kind of operation\n"
    "  -h, --help            Show this help\n";

std::vector<int> parse_ids(const std::string& text) {
    std::vector<int> ids;
    std::string cur;
    auto flush = [&]() {
        if (cur.empty()) return;
        char* end = nullptr;
        const long v = std::strtol(cur.c_str(), &end, 10);
        if (*end) throw ArgumentError("'" + cur + "' is not a token id");
        ids.push_back(static_cast<int>(v));
        cur.clear();
    };
    for (char c : text) {
        if (c == ',' || c == ' ' || c == '\t' || c == '\n' || c == '\r') flush();
        else cur.push_back(c);
    }
    flush();
    return ids;
}

std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw Error(path + ": cannot open");
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

std::string trimmed(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace(static_cast<unsigned char>(s[a]))) ++a;
    while (b > a && std::isspace(static_cast<unsigned char>(s[b - 1]))) --b;
    return s.substr(a, b - a);
}

struct Turn { int tokens = 0; double seconds = 0.0; std::string text; };

// One response, streamed to the terminal.
Turn run_turn(TextEngine& engine, const std::vector<int>& prompt, const ChatArgs& a) {
    std::printf("Output: ");
    std::fflush(stdout);
    Turn turn;
    GenerateOptions o;
    o.temperature = a.temp;
    o.top_p = a.top_p;
    o.max_tokens = a.max_tokens;
    o.seed = a.seed;
    o.on_token = [&](int, int, const std::string& piece) {
        turn.text += piece;
        std::fputs(piece.c_str(), stdout);
        std::fflush(stdout);
    };
    const auto t0 = std::chrono::steady_clock::now();
    std::vector<Result> res;
    std::string table;
    if (a.op_times) {
        ops::OpTimes times;
        res = engine.generate({prompt}, o);
        table = times.table();
    } else {
        res = engine.generate({prompt}, o);
    }
    turn.seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    turn.tokens = static_cast<int>(res[0].tokens.size());
    if (!table.empty()) std::printf("\n\n%s", table.c_str());
    std::printf("\n\n[%d tokens in %.3fs (%.1f tok/s)]\n", turn.tokens, turn.seconds, turn.seconds > 0 ? turn.tokens / turn.seconds : 0.0);
    std::fflush(stdout);
    return turn;
}

// The `>>>` loop's state and slash commands, with the meanings the reference's console gives them
// (llama_interactive_console.cpp:25-41 state, :125-143 help, :224-309 commands, :104-117 how a prompt is composed): the
// conversation is a list of turns (user, assistant, user, ...); a prompt is the system text, the turns and the new line
// joined by newlines; /clear forgets the turns and keeps the system text; every turn takes the next seed.  Without a
// tokenizer a line is a list of token ids and stands alone (there is no text to join).
class Console {
public:
    Console(TextEngine& e, ChatArgs& a) : engine_(e), a_(a) {}

    // 1 = handled, 0 = leave the loop, -1 = not a command (a prompt)
    int command(const std::string& line) {
        auto starts = [&](const char* p) { return line.rfind(p, 0) == 0; };
        if (line == "/exit" || line == "/quit") { std::puts("Exiting..."); return 0; }
        if (line == "/help") {
            std::printf("Commands:\n"
                        "  /help               Show commands + current state.\n"
                        "  /temp <float>       Sampling temperature (0 = greedy). Current: %g\n"
                        "  /top_p <float>      Nucleus top-p threshold. Current: %g\n"
                        "  /max <int>          Max generated tokens per response. Current: %d\n"
                        "  /system <text>      Set/replace the system prompt prefix (no text: clear it).\n"
                        "  /clear              Clear conversation history (keeps system).\n"
                        "  /history            Show per-turn stats for the last response.\n"
                        "  /model              Show model info (path / config / device).\n"
                        "  /save <file>        Persist conversation history to file.\n"
                        "  /load <file>        Load conversation history from file.\n"
                        "  /exit, /quit        Exit.\n\n"
                        "Model path: %s\nTokenizer:  %s\nDevice:     %s\nSynthetic:  %s\n\n",
                        a_.temp, a_.top_p, a_.max_tokens, a_.model.c_str(), a_.tokenizer.c_str(), a_.device.c_str(), a_.synthetic ? "yes" : "no");
            return 1;
        }
        if (line == "/model") {
            const json::Value info = engine_.describe();
            for (const auto& m : info.as_object())
                std::printf("%-10s%s\n", (m.first + ":").c_str(), m.second.is_string() ? m.second.as_string().c_str() : m.second.dump().c_str());
            std::puts("");
            return 1;
        }
        if (line == "/history") {
            std::printf("Last response: %d tokens in %.2fs (%.1f tok/s)\nLast text: %s\n\n", last_.tokens, last_.seconds,
                        last_.seconds > 0 ? last_.tokens / last_.seconds : 0.0, last_.text.c_str());
            return 1;
        }
        if (line == "/clear") {
            turns_.clear();
            std::puts("Conversation cleared (system prompt retained).\n");
            return 1;
        }
        if (starts("/temp ") || starts("/top_p ")) {
            const bool is_temp = starts("/temp ");
            const std::string v = trimmed(line.substr(is_temp ? 6 : 7));
            char* end = nullptr;
            const float f = std::strtof(v.c_str(), &end);
            if (v.empty() || *end) std::printf("Invalid %s value\n\n", is_temp ? "temperature" : "top-p");
            else {
                (is_temp ? a_.temp : a_.top_p) = f;
                std::printf("%s set to %g\n\n", is_temp ? "Temperature" : "Top-P", f);
            }
            return 1;
        }
        if (starts("/max ")) {
            const std::string v = trimmed(line.substr(5));
            char* end = nullptr;
            const long n = std::strtol(v.c_str(), &end, 10);
            if (v.empty() || *end || n < 0) std::puts("Invalid max new tokens value\n");
            else {
                a_.max_tokens = static_cast<int>(n);
                std::printf("Max new tokens set to %ld\n\n", n);
            }
            return 1;
        }
        if (line == "/system" || starts("/system ")) {
            system_ = starts("/system ") ? line.substr(8) : "";
            if (system_.empty()) std::puts("System prompt cleared.\n");
            else std::printf("System prompt set (%zu chars).\n\n", system_.size());
            return 1;
        }
        if (starts("/save ")) {
            const std::string path = trimmed(line.substr(6));
            std::ofstream f(path);
            if (f && (f << snapshot())) std::printf("Saved to %s\n\n", path.c_str());
            else std::printf("Save failed: %s\n\n", path.c_str());
            return 1;
        }
        if (starts("/load ")) {
            const std::string path = trimmed(line.substr(6));
            std::ifstream f(path);
            if (!f) { std::printf("Load failed: %s\n\n", path.c_str()); return 1; }
            std::stringstream ss;
            ss << f.rdbuf();
            restore(ss.str());
            std::printf("Loaded from %s (%zu turns)\n\n", path.c_str(), turns_.size());
            return 1;
        }
        return -1;
    }

    // the conversation as a file: role lines (SYSTEM / USER / ASSISTANT), each followed by the text; # lines are comments
    std::string snapshot() const {
        std::string out = "# velomind_b200 conversation snapshot\n";
        if (!system_.empty()) out += "SYSTEM\n" + system_ + "\n";
        for (size_t i = 0; i < turns_.size(); ++i) out += std::string(i % 2 == 0 ? "USER" : "ASSISTANT") + "\n" + turns_[i] + "\n";
        return out;
    }

    void restore(const std::string& text) {
        system_.clear();
        turns_.clear();
        std::string role;
        std::vector<std::string> body;
        auto flush = [&]() {
            std::string joined;
            for (size_t i = 0; i < body.size(); ++i) joined += (i ? "\n" : "") + body[i];
            if (role == "SYSTEM") system_ = joined;
            else if (role == "USER" || role == "ASSISTANT") turns_.push_back(joined);
        };
        std::stringstream ss(text);
        std::string ln;
        while (std::getline(ss, ln)) {
            const bool comment = !ln.empty() && ln[0] == '#';
            if (comment || ln == "SYSTEM" || ln == "USER" || ln == "ASSISTANT") {
                flush();
                role = comment ? "" : ln;
                body.clear();
            } else body.push_back(ln);
        }
        flush();
    }

    std::string compose(const std::string& user_text) const {
        std::string out = system_;
        for (const std::string& t : turns_) out += (out.empty() ? "" : "\n") + t;
        return out + (out.empty() ? "" : "\n") + user_text;
    }

    void turn(const std::string& line) {
        std::vector<int> prompt;
        if (!engine_.tokenizer) {
            try {
                prompt = parse_ids(line);
            } catch (const Error&) {
                std::puts("no tokenizer.json: type token ids, e.g. 1 5 17");
                return;
            }
        } else prompt = engine_.encode(compose(line));
        last_ = run_turn(engine_, prompt, a_);
        ++a_.seed;
        if (engine_.tokenizer) {
            turns_.push_back(line);
            turns_.push_back(last_.text);
        }
    }

private:
    TextEngine& engine_;
    ChatArgs& a_;
    std::string system_;
    std::vector<std::string> turns_;
    Turn last_;
};

}  // namespace

int smollm2_chat_main(int argc, char** argv) {
    ChatArgs a;
    try {
        for (int i = 1; i < argc; ++i) {
            const std::string arg = argv[i];
            auto value = [&]() -> std::string {
                if (i + 1 >= argc) throw ArgumentError(arg + " needs a value");
                return argv[++i];
            };
            if (arg == "-h" || arg == "--help") { std::fputs(kUsage, stdout); return 0; }
            else if (arg == "--device") a.device = value();
            else if (arg == "--model") a.model = value();
            else if (arg == "--tokenizer") a.tokenizer = value();
            else if (arg == "--synthetic") a.synthetic = true;
            else if (arg == "--config") a.config = value();
            else if (arg == "--temp") a.temp = std::strtof(value().c_str(), nullptr);
            else if (arg == "--top-p") a.top_p = std::strtof(value().c_str(), nullptr);
            else if (arg == "--max-tokens") a.max_tokens = std::atoi(value().c_str());
            else if (arg == "--prompt") a.prompt = value();
            else if (arg == "--prompt-ids") a.prompt_ids = value();
            else if (arg == "--prompt-file") a.prompt_file = value();
            else if (arg == "--seed") a.seed = std::atoll(value().c_str());
            else if (arg == "--dtype") a.dtype = value();
            else if (arg == "--fp32") a.dtype = "float32";
            else if (arg == "--op-times") a.op_times = true;
            else throw ArgumentError("Unknown option: " + arg);
        }
        if (a.device == "cuda") a.device = "cuda:0";
        if (a.device.rfind("cuda", 0) != 0)
            throw ArgumentError("Unknown device: " + a.device + " (this library runs on cuda only; the reference's cpu and ispc backends are not built)");
        if (!a.synthetic && a.model.empty()) throw ArgumentError("give --model <folder> or --synthetic");
        EngineConfig cfg;
        cfg.model_path = a.model;
        cfg.tokenizer_path = a.tokenizer;
        cfg.device = a.device;
        cfg.use_synthetic = a.synthetic;
        if (!a.config.empty()) cfg.model_config = json::parse(read_file(a.config), a.config, false);
        cfg.seed = a.seed;
        cfg.dtype = a.dtype;
        if (a.op_times) cfg.use_graphs = 0;
        std::printf("Initializing engine on device [%s]...\n", cfg.device.c_str());
        std::fflush(stdout);
        TextEngine engine(cfg);
        engine.load();
        std::puts("Engine ready.");
        if (!a.prompt_file.empty()) {
            const std::string text = trimmed(read_file(a.prompt_file));
            if (engine.tokenizer) a.prompt = text;
            else a.prompt_ids = text;
        }
        if (!a.prompt_ids.empty()) {
            run_turn(engine, parse_ids(a.prompt_ids), a);
            return 0;
        }
        if (!a.prompt.empty()) {
            std::printf("Prompt: %s\n", a.prompt.c_str());
            // without a tokenizer the reference feeds the single token 1 (llama_engine.cpp:603-605)
            run_turn(engine, engine.tokenizer ? engine.encode(a.prompt) : std::vector<int>{1}, a);
            return 0;
        }
        Console console(engine, a);
        std::string line;
        while (true) {
            std::fputs(">>> ", stdout);
            std::fflush(stdout);
            if (!std::getline(std::cin, line)) break;
            line = trimmed(line);
            if (line.empty()) continue;
            const int handled = line[0] == '/' ? console.command(line) : -1;
            if (handled == 0) break;
            if (handled < 0) console.turn(line);
        }
    } catch (const std::exception& ex) {       // the reference prints "Error: <what>" and returns 1 (interactive_main.cpp:131-134)
        std::fprintf(stderr, "Error: %s\n", ex.what());
        return 1;
    }
    return 0;
}

}  // namespace vmb
