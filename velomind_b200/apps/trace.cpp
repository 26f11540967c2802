// Trace replay: feed given token ids through a model step by step and write logits.  Samples nothing.
//
// It drives the same model, step function, cache and kernels that generation uses.
//
//   trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--device cuda:0]
//
// Input, one JSON object per line on standard input:
//     {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
// For a step in which something is wanted, `<out>/<step>.f32` receives the logits at the wanted places in the order of the
// entries and of `want`, little-endian float32 [wanted, vocab].  After every step a line `done <step>` is printed and flushed.
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <sys/stat.h>

#include "velomind_b200/velomind.h"

namespace vmb {

namespace {
std::string id_text(const json::Value& v) { return v.is_string() ? v.as_string() : v.dump(); }

std::vector<int> int_list(const json::Value* v, const char* what) {
    std::vector<int> out;
    if (!v || v->is_null()) return out;
    if (!v->is_array()) throw ArgumentError(std::string(what) + " must be a list of integers");
    for (const auto& x : v->as_array()) {
        if (!x.is_integer()) throw ArgumentError(std::string(what) + " must be a list of integers");
        out.push_back(static_cast<int>(x.as_int()));
    }
    return out;
}

int trace_main(int argc, char** argv) {
    std::string model_dir, dtype, out_dir, device = "cuda:0";
    long long max_tokens = -1;
    for (int i = 1; i < argc; ++i) {
        const std::string arg = argv[i];
        auto value = [&]() -> std::string {
            if (i + 1 >= argc) throw ArgumentError(arg + " needs a value");
            return argv[++i];
        };
        if (arg == "--model") model_dir = value();
        else if (arg == "--dtype") dtype = value();
        else if (arg == "--out") out_dir = value();
        else if (arg == "--max-tokens") max_tokens = std::atoll(value().c_str());
        else if (arg == "--device") device = value();
        else if (arg == "-h" || arg == "--help") {
            std::puts("usage: trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--device cuda:0]\n"
                      "  reads steps from standard input, one JSON object a line:\n"
                      "  {\"step\": 0, \"entries\": [{\"id\": \"a\", \"tokens\": [5, 17, 3], \"want\": [0, 2]}], \"end\": []}\n"
                      "  writes <out>/<step>.f32 (float32 [wanted, vocab]) and prints `done <step>` after every step");
            return 0;
        } else throw ArgumentError("unknown option " + arg);
    }
    if (model_dir.empty() || dtype.empty() || out_dir.empty() || max_tokens < 0)
        throw ArgumentError("the options --model, --dtype, --out and --max-tokens are required");
    if (dtype != "bfloat16" && dtype != "float32") throw ArgumentError("--dtype is bfloat16 or float32");
    ::mkdir(out_dir.c_str(), 0777);
    auto model = load_model(model_dir, compute_dtype(dtype), device);
    EngineOptions o;
    o.max_tokens = max_tokens;
    Engine engine(model, o);
    std::map<std::string, int> slots;
    std::string line;
    std::vector<float> host;
    while (std::getline(std::cin, line)) {
        if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
        const json::Value rec = json::parse(line, "a line of the trace", false);
        const json::Value* step = rec.find("step");
        if (!step) throw ArgumentError("a line of the trace has no \"step\"");
        const std::string step_name = id_text(*step);
        std::vector<Entry> entries;
        if (const json::Value* es = rec.find("entries"))
            for (const auto& e : es->as_array()) {
                const json::Value* id = e.find("id");
                if (!id) throw ArgumentError("an entry of the trace has no \"id\"");
                const std::string rid = id_text(*id);
                auto it = slots.find(rid);
                if (it == slots.end()) it = slots.emplace(rid, engine.open()).first;
                entries.push_back(Entry{it->second, int_list(e.find("tokens"), "tokens"), int_list(e.find("want"), "want")});
            }
        if (!entries.empty()) {
            int rows = 0;
            const float* logits = engine.step(entries, &rows);
            if (rows > 0) {
                host.resize(static_cast<size_t>(rows) * engine.vocab);
                engine.copy_logits_to_host(logits, rows, host.data());      // synchronises
                const std::string path = out_dir + "/" + step_name + ".f32";
                FILE* f = std::fopen(path.c_str(), "wb");
                if (!f || std::fwrite(host.data(), sizeof(float), host.size(), f) != host.size() || std::fclose(f) != 0)
                    throw Error(path + ": cannot write");
            }
            engine.raise_if_error();
        }
        if (const json::Value* end = rec.find("end"))
            for (const auto& r : end->as_array()) {
                auto it = slots.find(id_text(r));
                if (it != slots.end()) {
                    engine.close(it->second);
                    slots.erase(it);
                }
            }
        std::printf("done %s\n", step_name.c_str());
        std::fflush(stdout);
    }
    return 0;
}
}  // namespace

// A failure is one line on stderr and exit code 1.
int trace_run_main(int argc, char** argv) {
    try {
        return trace_main(argc, argv);
    } catch (const std::exception& ex) {
        std::fprintf(stderr, "trace_run: error: %s\n", ex.what());
        return 1;
    }
}

}  // namespace vmb
