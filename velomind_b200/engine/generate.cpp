// The generation loop: batches of unequal prompts, stop tokens, sequences that end early, batch after batch.
//
// The reference generates one sequence: prefill, sample, then feed each token back until `max_new_tokens` or the
// end-of-sequence token, which is kept in the output and not fed (examples/common/llama/llama_engine.cpp:633-653;
// `max_new_tokens == 0` returns after the prompt, :635-637).  The same rules hold here for every sequence of a batch; a
// sequence that ends leaves the batch at once and its slot and pages go back to the cache; requests that did not fit into
// one batch run in the next.
//
// The loop only needs a Stepper (open / close / step_and_sample, optionally decode_many), so its decisions can be tested
// without a GPU.
#include <algorithm>
#include <chrono>
#include <set>

#include "velomind_b200/kernels.h"
#include "velomind_b200/velomind.h"

namespace vmb {

int pages_for(const Request& r) {
    const long long most = static_cast<long long>(r.prompt.size()) + std::max(r.params.max_tokens - 1, 0);
    return static_cast<int>((std::max<long long>(most, 1) + VM_PAGE_TOKENS - 1) / VM_PAGE_TOKENS);
}

std::vector<std::vector<int>> plan_batches(const std::vector<Request>& requests, int total_pages, int max_batch) {
    std::vector<std::vector<int>> batches;
    std::vector<int> cur;
    long long used = 0;
    for (int i = 0; i < static_cast<int>(requests.size()); ++i) {
        const int need = pages_for(requests[i]);
        if (need > total_pages)
            throw ArgumentError(format("request %d may reach %d cached tokens; the cache holds %d", i, need * VM_PAGE_TOKENS, total_pages * VM_PAGE_TOKENS));
        if (!cur.empty() && (used + need > total_pages || static_cast<int>(cur.size()) >= max_batch)) {
            batches.push_back(cur);
            cur.clear();
            used = 0;
        }
        cur.push_back(i);
        used += need;
    }
    if (!cur.empty()) batches.push_back(cur);
    return batches;
}

GenerationLoop::GenerationLoop(Stepper& stepper, int total_pages, int max_batch, std::vector<int> default_stop, int steps_per_sync)
    : stepper_(stepper), total_pages_(total_pages), max_batch_(max_batch), steps_per_sync_(std::max(1, steps_per_sync)), default_stop_(std::move(default_stop)) {}

std::vector<Result> GenerationLoop::run(const std::vector<Request>& requests, const TokenCallback& on_token) {
    std::vector<Result> results(requests.size());
    for (size_t i = 0; i < requests.size(); ++i) results[i].prompt_tokens = static_cast<int>(requests[i].prompt.size());
    timing = Timing();
    for (const auto& batch : plan_batches(requests, total_pages_, max_batch_)) run_batch(requests, batch, results, on_token);
    return results;
}

void GenerationLoop::run_batch(const std::vector<Request>& requests, const std::vector<int>& batch, std::vector<Result>& results, const TokenCallback& on_token) {
    using Clock = std::chrono::steady_clock;
    struct Live { int request, slot; };
    std::vector<Live> live;
    try {
        for (int i : batch) {
            const Request& r = requests[i];
            if (r.params.max_tokens <= 0) { results[i].finish_reason = "length"; continue; }     // llama_engine.cpp:635-637: nothing to generate
            if (r.prompt.empty()) { results[i].finish_reason = "empty"; continue; }
            live.push_back(Live{i, stepper_.open()});
        }
        std::map<int, std::vector<int>> feed;
        for (const Live& l : live) feed[l.request] = requests[l.request].prompt;
        auto t0 = Clock::now();
        long long step_no = 0;
        while (!live.empty()) {
            // how many decode steps to queue before looking at the tokens: 1 for the prompts' step, for steppers that cannot queue,
            // and when steps_per_sync is 1; never beyond what the sequence closest to its budget may still take
            int run = 1;
            if (step_no > 0 && steps_per_sync_ > 1 && stepper_.can_queue()) {
                int room = 1 << 30;
                for (const Live& l : live) room = std::min(room, requests[l.request].params.max_tokens - static_cast<int>(results[l.request].tokens.size()));
                run = std::max(1, std::min({steps_per_sync_, room, stepper_.max_run()}));
            }
            std::vector<SamplingParams> params;
            std::vector<long long> streams, drawn;
            for (const Live& l : live) {
                params.push_back(requests[l.request].params);
                streams.push_back(requests[l.request].stream);
                drawn.push_back(static_cast<long long>(results[l.request].tokens.size()));
            }
            std::vector<std::vector<int>> rows;
            if (run > 1) {
                std::vector<int> slots, last;
                for (const Live& l : live) { slots.push_back(l.slot); last.push_back(feed[l.request][0]); }
                rows = stepper_.decode_many(slots, last, params, streams, drawn, run);
            } else {
                std::vector<Entry> entries;
                for (const Live& l : live) {
                    const std::vector<int>& f = feed[l.request];
                    entries.push_back(Entry{l.slot, f, {static_cast<int>(f.size()) - 1}});
                }
                rows.push_back(stepper_.step_and_sample(entries, params, streams, drawn));
            }
            const auto now = Clock::now();
            const double dt = std::chrono::duration<double>(now - t0).count();
            if (step_no == 0) timing.prefill_seconds += dt;
            else { timing.decode_seconds += dt; timing.decode_steps += static_cast<long long>(rows.size()); }
            t0 = now;
            std::set<int> ended;
            for (const auto& tokens : rows) {              // one row of tokens per step of the run
                for (size_t j = 0; j < live.size(); ++j) {
                    const int i = live[j].request;
                    if (ended.count(i)) continue;          // the sequence ended earlier in this run: the rest is not its output
                    const int tok = tokens[j];
                    const SamplingParams& par = requests[i].params;
                    std::vector<int>& out = results[i].tokens;
                    out.push_back(tok);
                    ++timing.generated_tokens;
                    if (on_token) on_token(i, tok);
                    const std::vector<int>& stops = par.stop_tokens.empty() ? default_stop_ : par.stop_tokens;
                    std::string reason;
                    if (std::find(stops.begin(), stops.end(), tok) != stops.end()) reason = "stop";
                    else if (static_cast<int>(out.size()) >= par.max_tokens) reason = "length";
                    else if (tok < 0) reason = "error";
                    if (!reason.empty()) { results[i].finish_reason = reason; ended.insert(i); }
                    else feed[i] = {tok};
                }
            }
            if (!ended.empty()) {
                std::vector<Live> still;
                for (const Live& l : live) {
                    if (ended.count(l.request)) stepper_.close(l.slot);     // the slot and its pages are free for the next batch at once
                    else still.push_back(l);
                }
                live.swap(still);
            }
            step_no += static_cast<long long>(rows.size());
        }
    } catch (...) {
        for (const Live& l : live) {
            try { stepper_.close(l.slot); } catch (...) {}
        }
        throw;
    }
}

std::vector<int> EngineStepper::step_and_sample(const std::vector<Entry>& entries, const std::vector<SamplingParams>& params,
                                                const std::vector<long long>& streams, const std::vector<long long>& drawn) {
    int rows = 0;
    const float* logits = engine.step(entries, &rows);
    if (!sample_fn) return engine.sample(logits, rows, params, streams, drawn);
    // the reference's way of sampling (llama_engine.h:106-121): a host function of one row of float32 logits
    std::vector<float> host(static_cast<size_t>(rows) * engine.vocab);
    engine.copy_logits_to_host(logits, rows, host.data());
    std::vector<int> out;
    for (int r = 0; r < rows; ++r) out.push_back(sample_fn(host.data() + static_cast<size_t>(r) * engine.vocab, engine.vocab));
    return out;
}

}  // namespace vmb
