// Times the reference (Aiza-Lee/velo-mind) end to end through its own public engine API, unmodified:
// `SmolLM2Engine` with `use_synthetic` at its built-in 135M sizes (examples/smollm2/smollm2_engine.h:16-81), then
// `prefill(tokens)` and `forward_step(token, pos)` (examples/common/llama/llama_engine.h:94-106) exactly as its own
// generation loop calls them (llama_engine.cpp:633-653), with a greedy pick on the host from the logits each call returns.
// The reference runs ONE sequence at a time, so a batch of B requests is B sequences one after another.
//
//   reference_driver <cpu|cuda> <sequences> <prompt tokens> <decode steps> <warm-up steps> <prefill tokens>
//
// Prints one JSON object: wall-clock milliseconds of every timed call, host tokens in and host logits out.
// This file belongs to this repository (it is no part of the reference) and links nothing of this repository.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "smollm2_engine.h"

namespace {
using Clock = std::chrono::steady_clock;

double ms_since(Clock::time_point t0) {
    return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}

std::int32_t argmax(const std::vector<float>& v) {
    return static_cast<std::int32_t>(std::max_element(v.begin(), v.end()) - v.begin());
}

double median(std::vector<double> v) {
    if (v.empty()) return 0.0;
    std::sort(v.begin(), v.end());
    return v.size() % 2 ? v[v.size() / 2] : 0.5 * (v[v.size() / 2 - 1] + v[v.size() / 2]);
}
}  // namespace

int main(int argc, char** argv) {
    if (argc < 7) {
        std::fprintf(stderr, "usage: %s <cpu|cuda> <sequences> <prompt tokens> <decode steps> <warm-up steps> <prefill tokens>\n", argv[0]);
        return 2;
    }
    const std::string dev = argv[1];
    const int B = std::atoi(argv[2]), S = std::atoi(argv[3]), K = std::atoi(argv[4]), W = std::atoi(argv[5]), P = std::atoi(argv[6]);
    namespace sm = velomind::examples::smollm2;
    try {
        sm::EngineConfig cfg;
        cfg.device = dev == "cuda" ? velomind::DeviceType::CUDA : velomind::DeviceType::CPU;
        cfg.use_synthetic = true;
        sm::SmolLM2Engine engine(cfg);
        engine.load();
        const int V = static_cast<int>(engine.config().model_config.vocab_size);

        std::vector<double> step_ms, prompt_ms;
        std::uint32_t rng = 12345u;
        for (int b = 0; b < B; ++b) {
            std::vector<std::int32_t> prompt(S);
            for (auto& t : prompt) { rng = rng * 1664525u + 1013904223u; t = static_cast<std::int32_t>((rng >> 8) % V); }
            engine.reset_session();
            auto t0 = Clock::now();
            auto logits = engine.prefill(prompt);
            prompt_ms.push_back(ms_since(t0));
            std::int32_t tok = argmax(logits);
            for (int k = 0; k < W + K; ++k) {
                auto t1 = Clock::now();
                logits = engine.forward_step(tok, engine.session_seq_len());
                tok = argmax(logits);
                if (k >= W) step_ms.push_back(ms_since(t1));
            }
        }
        double total = 0.0;
        for (double x : step_ms) total += x;

        std::vector<double> long_ms;
        if (P > 0) {
            std::vector<std::int32_t> prompt(P);
            for (auto& t : prompt) { rng = rng * 1664525u + 1013904223u; t = static_cast<std::int32_t>((rng >> 8) % V); }
            for (int r = 0; r < 3; ++r) {
                engine.reset_session();
                auto t0 = Clock::now();
                auto logits = engine.prefill(prompt);
                long_ms.push_back(ms_since(t0));
                (void)argmax(logits);
            }
            engine.reset_session();
        }
        std::printf("{\"device\": \"%s\", \"sequences\": %d, \"prompt_tokens\": %d, \"decode_steps\": %d, \"warmup\": %d, "
                    "\"decode_ms_total\": %.4f, \"decode_ms_median\": %.4f, \"prompt_ms_median\": %.4f, "
                    "\"prefill_tokens\": %d, \"prefill_ms_median\": %.4f, \"logit_bytes_per_step\": %zu}\n",
                    dev.c_str(), B, S, K, W, total, median(step_ms), median(prompt_ms), P, median(long_ms),
                    static_cast<std::size_t>(V) * sizeof(float));
    } catch (const std::exception& ex) {
        std::printf("{\"error\": \"%s\"}\n", ex.what());
        return 1;
    }
    return 0;
}
