// Host-side tests of the library that need no GPU: the cache's bookkeeping (no slot or page lost, held twice or freed
// twice), the activation arena's plan, the generation loop's decisions (with a stand-in stepper), the streamer, the JSON
// reader.  Built and run by tests/test_host_cpp.py (and by ctest): `host_tests` runs every case and prints `ok <name>` or
// `FAILED <name>: <why>`; `host_tests --list` prints the names; `host_tests <name>` runs one.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <functional>
#include <random>
#include <set>

#include "velomind_b200/kernels.h"
#include "velomind_b200/velomind.h"

using namespace vmb;

namespace {

struct Failure : std::runtime_error { using std::runtime_error::runtime_error; };

#define CHECK(cond)                                                                                   \
    do {                                                                                              \
        if (!(cond)) throw Failure(format("%s:%d: %s", __FILE__, __LINE__, #cond));                    \
    } while (0)

template <class E, class F> void expect_throw(F&& f, const char* needle, const char* file, int line) {
    try {
        f();
    } catch (const E& e) {
        if (std::string(e.what()).find(needle) == std::string::npos)
            throw Failure(format("%s:%d: message '%s' lacks '%s'", file, line, e.what(), needle));
        return;
    }
    throw Failure(format("%s:%d: nothing was thrown (expected '%s')", file, line, needle));
}
#define THROWS(E, needle, ...) expect_throw<E>([&] { __VA_ARGS__; }, needle, __FILE__, __LINE__)

std::vector<std::pair<std::string, std::function<void()>>>& cases() {
    static std::vector<std::pair<std::string, std::function<void()>>> c;
    return c;
}
struct Case {
    Case(const char* name, std::function<void()> f) { cases().emplace_back(name, std::move(f)); }
};
#define TEST(name) \
    void name();   \
    Case case_##name(#name, name); \
    void name()

// ------------------------------------------------------------------------------------------------ free list
TEST(free_list_never_loses_or_doubles) {
    FreeList fl(5, "thing");
    for (int i = 0; i < 5; ++i) CHECK(fl.take() == i);
    CHECK(fl.free_count() == 0);
    THROWS(CacheError, "out of things", fl.take());
    fl.give(3);
    fl.give(1);
    THROWS(CacheError, "freed twice", fl.give(3));
    THROWS(CacheError, "does not exist", fl.give(9));
    CHECK(fl.take() == 1 && fl.take() == 3);          // lowest first: what a batch gave back is used again
    fl.check();
    std::mt19937 rnd(0);
    std::set<int> held{0, 1, 2, 3, 4};
    for (int it = 0; it < 2000; ++it) {
        if (!held.empty() && rnd() % 2) {
            auto pick = held.begin();
            std::advance(pick, rnd() % held.size());
            fl.give(*pick);
            held.erase(pick);
        } else if (held.size() < 5) {
            const int i = fl.take();
            CHECK(!held.count(i));
            held.insert(i);
        }
        fl.check();
        CHECK(fl.held_count() == static_cast<int>(held.size()));
    }
}

CacheNeed all_keys(int kv_heads, int dim) {
    CacheNeed n;
    n.kind = CacheNeed::All;
    n.kv_heads = kv_heads;
    n.key_dim = n.value_dim = dim;
    return n;
}

TEST(slots_and_pages_come_back) {
    CacheBook c({all_keys(2, 16), all_keys(2, 16)}, {-1, -1}, 64 * 8, 1024, 3);
    CHECK(c.groups.size() == 1 && c.layers_in_group[0] == 2 && c.n_pages == 8 && c.max_slots == 3);
    const int a = c.open(), b = c.open();
    c.reserve(a, 65); c.commit(a, 65);
    c.reserve(b, 64); c.commit(b, 64);
    CHECK(c.groups[0].pages.held_count() == 3 && c.tokens_held() == 192);
    c.reserve(a, 66); c.commit(a, 66);                          // same page
    CHECK(c.groups[0].pages.held_count() == 3);
    c.check();
    THROWS(CacheError, "out of cache pages", c.reserve(b, 64 * 7));
    CHECK(c.groups[0].pages.held_count() == 3);                 // a refused reservation changes nothing
    CHECK(!c.can_hold({{a, 66}, {b, 64 * 7}}) && c.can_hold({{a, 128}, {b, 64 * 6}}));
    c.close(a);
    THROWS(CacheError, "not open", c.close(a));
    THROWS(CacheError, "not open", c.reserve(a, 1));
    CHECK(c.groups[0].pages.held_count() == 1);
    const int a2 = c.open();
    CHECK(a2 == a && c.length[a2] == 0);                        // the slot is used again, empty
    c.reserve(a2, 1);
    const int page = c.groups[0].table_row(a2)[0];
    CHECK(page == 0 || page == 1);                              // and so are its pages
    c.close(a2);
    c.close(b);
    c.check();
    CHECK(c.slots.held_count() == 0 && c.tokens_held() == 0);
    const int s = c.open();
    THROWS(CacheError, "model's limit", c.reserve(s, 2000));
    THROWS(CacheError, "less than one page", CacheBook({all_keys(1, 16)}, {-1}, 10, 1024));
}

TEST(groups_with_different_needs_have_their_own_storage) {
    CacheNeed win;
    win.kind = CacheNeed::Window;
    win.kv_heads = 1;
    win.key_dim = win.value_dim = 32;
    win.window = 70;
    CacheNeed state_only;
    state_only.state_floats = 5;
    CacheBook c({all_keys(2, 16), win, all_keys(2, 16), CacheNeed{}, state_only}, {-1, -1, -1, 1, -1}, 64 * 16, 1024);
    CHECK(c.groups.size() == 2);
    CHECK(c.where(0) == std::make_pair(0, 0) && c.where(2) == std::make_pair(0, 1) && c.where(1) == std::make_pair(1, 0));
    CHECK(c.where(3) == std::make_pair(1, 0) && c.where(4).first < 0);        // run 3 reads run 1's cache; run 4 holds no keys
    CHECK(c.state_floats[4] == 5 && c.state_owner[4] == 4 && c.state_floats[0] == 0);
    const int s = c.open();
    c.reserve(s, 300);
    c.commit(s, 300);
    CHECK(c.groups[0].pages.held_count() == 5);
    // window 70: the next query (position 300) sees keys 231..300, so blocks 0..2 (keys < 192) are gone
    CHECK(c.groups[1].pages.held_count() == 2 && c.groups[1].blocks_begin[s] == 3);
    for (int b = 0; b < 3; ++b) CHECK(c.groups[1].table_row(s)[b] == -1);
    c.check();
    c.close(s);
    c.check();
    CacheNeed unequal = all_keys(2, 16);
    unequal.value_dim = 32;
    THROWS(CacheError, "keys of 16 and values of 32", CacheBook({unequal}, {-1}, 64 * 4, 256));
}

// ------------------------------------------------------------------------------------------------ arena
TEST(arena_plan_packs_by_liveness) {
    // a and b overlap in time, c lives after a died: c reuses a's bytes
    ArenaPlan plan = plan_arena({{1000, 1, 4}, {500, 2, 6}, {900, 5, 8}});
    CHECK(plan.peak_bytes == 1024 + 512 && plan.buffer_count == 3 && plan.reused_count >= 1);
    for (size_t o : plan.offsets) CHECK(o % 256 == 0);
    std::vector<Interval> ivs;
    for (int i = 0; i < 40; ++i) {
        std::mt19937 r1(i), r2(i + 7);
        ivs.push_back(Interval{static_cast<size_t>(1 + r1() % 4999), i, i + static_cast<int>(r2() % 6)});
    }
    plan = plan_arena(ivs);
    size_t total = 0;
    for (int i = 0; i < 40; ++i) {
        total += plan.sizes[i];
        for (int j = 0; j < i; ++j) {
            const bool overlap_t = !(ivs[i].death < ivs[j].birth || ivs[j].death < ivs[i].birth);
            const bool overlap_m = plan.offsets[i] < plan.offsets[j] + plan.sizes[j] && plan.offsets[j] < plan.offsets[i] + plan.sizes[i];
            CHECK(!(overlap_t && overlap_m));
        }
    }
    CHECK(plan.bytes_saved == static_cast<long long>(total) - static_cast<long long>(plan.peak_bytes) && plan.bytes_saved > 0);
}

// ------------------------------------------------------------------------------------------------ generation loop
// Next token = (last token + 1) % vocab; records what it is asked to do.
struct FakeStepper : Stepper {
    int vocab = 50;
    std::set<int> free_slots, open_slots;
    std::vector<std::vector<std::pair<int, std::vector<int>>>> log;
    std::vector<int> closed;
    std::vector<long long> last_streams, last_steps;
    int fail_at = -1;
    explicit FakeStepper(int slots = 4) {
        for (int i = 0; i < slots; ++i) free_slots.insert(i);
    }
    int open() override {
        if (free_slots.empty()) throw CacheError("out of slots");
        const int s = *free_slots.begin();
        free_slots.erase(free_slots.begin());
        open_slots.insert(s);
        return s;
    }
    void close(int slot) override {
        if (!open_slots.count(slot)) throw Failure("closed twice");
        open_slots.erase(slot);
        free_slots.insert(slot);
        closed.push_back(slot);
    }
    std::vector<int> step_and_sample(const std::vector<Entry>& entries, const std::vector<SamplingParams>&, const std::vector<long long>& streams,
                                     const std::vector<long long>& drawn) override {
        if (static_cast<int>(log.size()) == fail_at) throw Error("boom");
        std::vector<std::pair<int, std::vector<int>>> rec;
        std::vector<int> out;
        for (const Entry& e : entries) {
            if (!open_slots.count(e.slot) || e.want.size() != 1 || e.want[0] != static_cast<int>(e.tokens.size()) - 1) throw Failure("bad entry");
            rec.emplace_back(e.slot, e.tokens);
            out.push_back((e.tokens.back() + 1) % vocab);
        }
        log.push_back(rec);
        last_streams = streams;
        last_steps = drawn;
        return out;
    }
};

// the same, and it can queue several decode steps
struct FakeRunStepper : FakeStepper {
    struct Run { std::vector<int> slots, last; std::vector<long long> steps; int k; };
    std::vector<Run> runs;
    bool can_queue() const override { return true; }
    int max_run() const override { return 5; }
    std::vector<std::vector<int>> decode_many(const std::vector<int>& slots, const std::vector<int>& last, const std::vector<SamplingParams>&,
                                              const std::vector<long long>&, const std::vector<long long>& steps, int k) override {
        for (int s : slots)
            if (!open_slots.count(s)) throw Failure("a run on a closed slot");
        if (k < 1 || k > 5) throw Failure("run length");
        runs.push_back(Run{slots, last, steps, k});
        std::vector<std::vector<int>> rows;
        for (int j = 0; j < k; ++j) {
            std::vector<int> row;
            for (int t : last) row.push_back((t + 1 + j) % vocab);
            rows.push_back(row);
        }
        return rows;
    }
};

Request request(std::vector<int> prompt, int max_tokens, long long stream = 0) {
    Request r;
    r.prompt = std::move(prompt);
    r.params.temperature = 0.f;
    r.params.max_tokens = max_tokens;
    r.stream = stream;
    return r;
}

TEST(loop_unequal_prompts_stop_tokens_and_early_ends) {
    FakeStepper st;
    GenerationLoop loop(st, 100, 4, {13});
    const std::vector<Request> reqs = {request({1, 2, 3}, 5), request({10}, 9), request({40, 41}, 2), request({7}, 0), request({}, 4)};
    std::vector<std::pair<int, int>> seen;
    const std::vector<Result> res = loop.run(reqs, [&](int i, int t) { seen.emplace_back(i, t); });
    CHECK((res[0].tokens == std::vector<int>{4, 5, 6, 7, 8}) && res[0].finish_reason == "length");
    CHECK((res[1].tokens == std::vector<int>{11, 12, 13}) && res[1].finish_reason == "stop");     // the stop token is kept, not fed
    CHECK((res[2].tokens == std::vector<int>{42, 43}) && res[2].finish_reason == "length");
    CHECK(res[3].tokens.empty() && res[3].finish_reason == "length");                             // max_tokens 0: nothing to do
    CHECK(res[4].finish_reason == "empty");
    using Rec = std::vector<std::pair<int, std::vector<int>>>;
    CHECK((st.log[0] == Rec{{0, {1, 2, 3}}, {1, {10}}, {2, {40, 41}}}));                          // prompts whole, in one step
    CHECK((st.log[1] == Rec{{0, {4}}, {1, {11}}, {2, {42}}}));                                    // then one token each
    CHECK((st.log[2] == Rec{{0, {5}}, {1, {12}}}));                                               // request 2 ended earlier
    CHECK((st.log[3] == Rec{{0, {6}}}) && st.log.size() == 5);                                    // 13 was never fed
    std::vector<int> closed = st.closed;
    std::sort(closed.begin(), closed.end());
    CHECK(st.open_slots.empty() && (closed == std::vector<int>{0, 1, 2}));
    std::vector<int> of_one;
    for (auto& p : seen)
        if (p.first == 1) of_one.push_back(p.second);
    CHECK((of_one == std::vector<int>{11, 12, 13}));
    CHECK(loop.timing.generated_tokens == 10 && loop.timing.decode_steps == 4 && res[0].prompt_tokens == 3);
}

TEST(loop_runs_batch_after_batch_and_reuses_slots) {
    FakeStepper st(2);
    GenerationLoop loop(st, 100, 2);
    std::vector<Request> reqs;
    for (int i = 0; i < 5; ++i) reqs.push_back(request({i}, 2 + i, i));
    const std::vector<Result> res = loop.run(reqs);
    for (int i = 0; i < 5; ++i) {
        std::vector<int> want;
        for (int k = 0; k < 2 + i; ++k) want.push_back(i + 1 + k);
        CHECK(res[i].tokens == want);
    }
    std::vector<int> closed = st.closed;
    std::sort(closed.begin(), closed.end());
    CHECK((closed == std::vector<int>{0, 0, 0, 1, 1}) && st.open_slots.empty());
    CHECK(st.log[0][0].first == 0 && st.log[0][1].first == 1);
    CHECK((st.last_streams == std::vector<long long>{4}) && (st.last_steps == std::vector<long long>{5}));   // request 4's stream and its own step count
}

TEST(batches_are_cut_by_pages_and_slots) {
    const std::vector<Request> reqs = {request(std::vector<int>(100, 0), 29), request(std::vector<int>(10, 0), 1), request(std::vector<int>(64, 0), 2),
                                       request(std::vector<int>(300, 0), 1)};
    CHECK(pages_for(reqs[0]) == 2 && pages_for(reqs[1]) == 1 && pages_for(reqs[2]) == 2 && pages_for(reqs[3]) == 5);
    CHECK((plan_batches(reqs, 5, 8) == std::vector<std::vector<int>>{{0, 1, 2}, {3}}));
    CHECK((plan_batches(reqs, 100, 2) == std::vector<std::vector<int>>{{0, 1}, {2, 3}}));
    THROWS(ArgumentError, "request 3", plan_batches(reqs, 4, 8));
}

TEST(loop_closes_slots_when_a_step_fails) {
    FakeStepper st;
    st.fail_at = 1;
    GenerationLoop loop(st, 100, 4);
    THROWS(Error, "boom", loop.run({request({1}, 5), request({2}, 5)}));
    CHECK(st.open_slots.empty());
}

TEST(loop_with_queued_decode_runs_gives_the_same_tokens) {
    const std::vector<Request> reqs = {request({1, 2, 3}, 9), request({10}, 12), request({40, 41}, 2)};
    FakeStepper plain;
    const std::vector<Result> base = GenerationLoop(plain, 100, 4, {15}).run(reqs);
    FakeRunStepper st;
    GenerationLoop loop(st, 100, 4, {15}, 8);
    const std::vector<Result> got = loop.run(reqs);
    for (size_t i = 0; i < reqs.size(); ++i) CHECK(got[i].tokens == base[i].tokens && got[i].finish_reason == base[i].finish_reason);
    CHECK((got[1].tokens == std::vector<int>{11, 12, 13, 14, 15}) && got[1].finish_reason == "stop");   // ended inside a run; the rest is dropped
    // request 2 may take only one more token after the prompts' step, so that step is a single one; then a run of the stepper's
    // cap (5), inside which request 1 stops; then what request 0's budget leaves (2)
    CHECK(st.runs.size() == 2 && st.runs[0].k == 5 && st.runs[1].k == 2);
    CHECK((st.runs[0].slots == std::vector<int>{0, 1}) && (st.runs[0].steps == std::vector<long long>{2, 2}));
    CHECK((st.runs[1].slots == std::vector<int>{0}) && (st.runs[1].last == std::vector<int>{10}) && (st.runs[1].steps == std::vector<long long>{7}));
    CHECK(st.open_slots.empty());
    long long total = 0;
    for (const Result& r : got) total += static_cast<long long>(r.tokens.size());
    CHECK(loop.timing.generated_tokens == total);
}

// ------------------------------------------------------------------------------------------------ text
std::shared_ptr<Tokenizer> byte_tokenizer() {
    // a vocabulary of the 256 byte symbols plus two merges and the special tokens
    json::Value vocab;
    vocab.object();
    int id = 0, extra = 0;
    // the GPT-2 byte-to-unicode alphabet, in byte order: printable bytes stand for themselves, the others get U+0100 onwards
    for (int b = 0; b < 256; ++b) {
        const bool keep = (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
        const unsigned cp = keep ? static_cast<unsigned>(b) : 256u + static_cast<unsigned>(extra++);
        std::string s;
        if (cp < 0x80) s.push_back(static_cast<char>(cp));
        else { s.push_back(static_cast<char>(0xC0 | (cp >> 6))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
        vocab.set(s, id++);
    }
    vocab.set("he", id++);
    vocab.set("hel", id++);
    json::Value model;
    model.set("vocab", vocab);
    model.set("merges", json::Array{json::Value("h e"), json::Value(json::Array{json::Value("he"), json::Value("l")})});
    json::Value root;
    root.set("model", model);
    json::Array added;
    for (const char* t : {"<|endoftext|>", "<|im_end|>", "<pad>"}) {
        json::Value a;
        a.set("content", t);
        a.set("id", id++);
        added.push_back(a);
    }
    root.set("added_tokens", json::Value(std::move(added)));
    return Tokenizer::from_json(root, "test tokenizer");
}

TEST(pretokenizer_pieces) {
    using V = std::vector<std::string>;
    CHECK((Tokenizer::pretokenize("Hello world") == V{"Hello", "\xC4\xA0world"}));                  // a leading space joins the word
    CHECK((Tokenizer::pretokenize("it's 12") == V{"it", "'s", "\xC4\xA0", "1", "2"}));               // contractions; digits stand alone
    CHECK((Tokenizer::pretokenize("a,, b") == V{"a", ",,", "\xC4\xA0" "b"}));
    CHECK(Tokenizer::pretokenize("").empty());
}

TEST(bpe_round_trip_and_special_ids) {
    auto tok = byte_tokenizer();
    CHECK(tok->bos_id == 258 && tok->eos_id == 259 && tok->pad_id == 260 && tok->unk_id < 0);
    const std::vector<int> ids = tok->encode("hello h\xC3\xA9!");
    CHECK(ids[0] == 257);                                                       // "hel" by the two merges, lowest rank first
    CHECK(tok->decode(ids) == "hello h\xC3\xA9!");
    std::vector<int> with_special = ids;
    with_special.insert(with_special.begin(), tok->bos_id);
    with_special.push_back(tok->eos_id);
    CHECK(tok->decode(with_special) == "hello h\xC3\xA9!");                     // begin/end/pad ids are skipped
    CHECK(tok->decode({9999, -1}).empty());
}

TEST(streamer_emits_deltas_and_waits_for_whole_characters) {
    auto tok = byte_tokenizer();
    const std::vector<int> ids = tok->encode("h\xC3\xA9y \xE2\x82\xAC");        // é is two bytes, the euro sign three
    TextStreamer s(tok);
    std::string all;
    std::vector<std::string> pieces;
    for (int id : ids) {
        pieces.push_back(s.put(id));
        all += pieces.back();
    }
    CHECK(all == "h\xC3\xA9y \xE2\x82\xAC");
    CHECK(pieces[0] == "h" && pieces[1].empty() && pieces[2] == "\xC3\xA9");     // the first byte of é is held back
    CHECK(s.flush().empty());
    // a sequence that ENDS inside a character: nothing is emitted for the tail until flush
    TextStreamer cut(tok);
    std::string got;
    for (size_t i = 0; i + 1 < ids.size(); ++i) got += cut.put(ids[i]);
    CHECK(got == "h\xC3\xA9y ");
    CHECK(cut.flush() == "\xEF\xBF\xBD");                                        // the incomplete character, as a replacement mark
    TextStreamer none;
    CHECK(none.put(17) == "[17]" && none.flush().empty());                       // without a tokenizer a token prints as "[id]"
}

TEST(json_reads_and_writes) {
    const json::Value v = json::parse("{\"a\": [1, 2.5, -3e2, true, null, \"x\\u00e9\\n\"], \"b\": {\"c\": 1e5}}", "t");
    CHECK(v.find("a")->as_array()[0].is_integer() && v.find("a")->as_array()[0].as_int() == 1);
    CHECK(!v.find("a")->as_array()[1].is_integer() && v.find("a")->as_array()[1].as_double() == 2.5);
    CHECK(v.find("a")->as_array()[2].as_int() == -300 && v.find("a")->as_array()[3].as_bool() && v.find("a")->as_array()[4].is_null());
    CHECK(v.find("a")->as_array()[5].as_string() == "x\xC3\xA9\n");
    CHECK(v.find("b")->find("c")->is_integer() && v.find("b")->find("c")->as_int() == 100000);
    CHECK(json::parse(v.dump(), "again") == v && json::parse(v.dump(2), "again") == v);
    THROWS(Error, "duplicate key", json::parse("{\"a\": 1, \"a\": 2}", "t"));
    THROWS(Error, "not valid JSON", json::parse("{\"a\": ", "t"));
    THROWS(Error, "nesting too deep", json::parse(std::string(1000, '['), "t"));
    THROWS(Error, "text after the value", json::parse("1 2", "t"));
}

TEST(parts_and_architectures_are_looked_up_by_name) {
    THROWS(ConfigError, "no norm of kind 'layernorm' is registered; registered: rmsnorm", build_part("norm", PartSpec{"layernorm", json::Value()}));
    THROWS(ConfigError, "unknown role", register_part("gadget", "x", nullptr));
    const std::vector<std::string> positions = registered_parts("position");
    CHECK(std::find(positions.begin(), positions.end(), "rotary_interleaved") != positions.end());
    CHECK(error_word_meaning(VM_ERRWORD_CACHE_READ).find("cache read") != std::string::npos && error_word_meaning(77) == "code 77");
    register_error_word(77, "a toy kernel's own fault");
    CHECK(error_word_meaning(77) == "a toy kernel's own fault");
    ModelPlan plan = llama_plan(LlamaConfig::from_json(json::parse(SMOLLM2_135M_CONFIG, "built-in")));
    CHECK(plan.blocks.size() == 30 && plan.hidden_size == 576 && plan.max_positions == 8192);
    plan.schedule = {ScheduleEntry{0, 1}, ScheduleEntry{1, -1}};
    THROWS(ConfigError, "does not come before", plan.validate());
    const WeightTable table = weight_table(llama_plan(LlamaConfig::from_json(json::parse(SMOLLM2_135M_CONFIG, "built-in"))));
    CHECK(table.size() == 30 * 9 + 3 && table.at("lm_head.weight").alias_of == "model.embed_tokens.weight");
}

}  // namespace

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "--list") == 0) {
        for (const auto& c : cases()) std::printf("%s\n", c.first.c_str());
        return 0;
    }
    int failed = 0;
    for (const auto& c : cases()) {
        if (argc > 1 && c.first != argv[1]) continue;
        try {
            c.second();
            std::printf("ok %s\n", c.first.c_str());
        } catch (const std::exception& e) {
            std::printf("FAILED %s: %s\n", c.first.c_str(), e.what());
            ++failed;
        }
        std::fflush(stdout);
    }
    return failed ? 1 : 0;
}
