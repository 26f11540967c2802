// The step function: a batch of sequences, each bringing its next tokens; one pass from the cache.
//
// The reference has two entry points for one sequence, `prefill(tokens)` and `forward_step(token, pos)`, each of which
// builds, compiles and allocates a new graph (examples/common/llama/llama_engine.cpp:333-393, :395-455).  Here one function
// serves any batch: whole prompts of unequal lengths in one step, then one token per sequence, or any other cut.  It runs
// only the tokens it is given, packed without padding, reads and extends the cache in place, and returns float32 logits at
// the wanted places.
//
// A step costs one host-to-device copy (all its integers lie in one pinned buffer), takes its activations from the arena
// plan of its capacity bucket, and is replayed from a CUDA graph where its shape was seen before: decode steps always, any
// other shape from its second appearance on.  Everything that changes from step to step (tokens, positions, lengths, block
// tables) lies in the descriptor buffer, which the recorded kernels read.
#include <algorithm>
#include <cstring>
#include <numeric>

#include "ops.h"

namespace vmb {

namespace {

// Capacity a count is rounded up to, so that few distinct buffer plans exist.
int bucket(int n, int floor = 8, int fine_from = 512, int fine_step = 512) {
    n = std::max(n, 1);
    if (n <= fine_from) {
        int b = floor;
        while (b < n) b *= 2;
        return b;
    }
    return (n + fine_step - 1) / fine_step * fine_step;
}

struct Chunk { int entry, first, last; };      // tokens [first, last) of an entry

}  // namespace

// The integers that describe one step, laid out in one pinned host buffer and one device buffer of the same layout.
class Descriptors {
public:
    Descriptors(int T, int B, int R, const std::vector<int>& widths) : T_cap(T), B_cap(B), R_cap(R), table_widths(widths) {
        auto field = [&](int n) {
            const int off = total;
            total += (n + 3) / 4 * 4;          // 16-byte aligned fields
            return off;
        };
        tokens = field(T); positions = field(T); seq_of_token = field(T); cu_tokens = field(B + 1); slots = field(B);
        ctx_len = field(B); logit_rows = field(std::max(R, 1));
        for (int w : widths) tables.push_back(field(B * w));
        host = std::make_unique<PinnedBuffer>(static_cast<size_t>(total) * sizeof(int));
        dev = std::make_unique<DeviceBuffer>(static_cast<size_t>(total) * sizeof(int), true);
        copied = vm_event_create();
        if (!copied) throw KernelError("could not create a CUDA event");
    }
    ~Descriptors() {
        if (copied) vm_event_destroy(copied);
    }
    int* h(int off) const { return static_cast<int*>(host->ptr) + off; }
    const int* d(int off) const { return static_cast<const int*>(dev->ptr) + off; }
    int* d_mut(int off) const { return static_cast<int*>(dev->ptr) + off; }
    void upload(cudaStream_t stream) {
        ops::check(vm_upload_record(dev->ptr, host->ptr, static_cast<long long>(total) * sizeof(int), copied, stream), "upload", stream);
        --ops::counters().own_launches;        // a copy, not a kernel
        ops::counters().h2d_bytes += static_cast<long long>(total) * sizeof(int);
        used = true;
    }
    void wait_reusable() {
        if (used && vm_event_synchronize(copied) != 0) throw KernelError("waiting for a step's descriptors to leave the host failed");
    }
    int T_cap, B_cap, R_cap;
    std::vector<int> table_widths;
    int total = 0;
    int tokens, positions, seq_of_token, cu_tokens, slots, ctx_len, logit_rows;
    std::vector<int> tables;
    std::unique_ptr<PinnedBuffer> host;
    std::unique_ptr<DeviceBuffer> dev;
    void* copied = nullptr;
    bool used = false;
};

struct Engine::Impl {
    struct Graph {
        cudaGraphExec_t exec = nullptr;
        long long own_launches = 0, library_calls = 0, tc_attention_calls = 0;
    };
    std::map<std::string, std::unique_ptr<Descriptors>> descs;
    std::unique_ptr<DeviceBuffer> logits;
    int logits_cap = 0;
    std::unique_ptr<DeviceBuffer> reordered;       // rows in the asked-for order, for the rare step that produces them in another
    std::unique_ptr<DeviceBuffer> err;
    std::map<std::string, Graph> graphs;
    std::map<std::string, int> shape_seen;

    // the device sampler's parameter block: int64 seed, stream, step [3, cap], then float32 temperature, top_p [2, cap]
    int sampler_cap = 0;
    std::unique_ptr<PinnedBuffer> sampler_host, sampled_host;
    std::unique_ptr<DeviceBuffer> sampler_dev, sampled_dev;
    int* sampled_direct = nullptr;                 // where kernels reach `sampled_host` themselves (no copy follows the sampler)
    std::vector<SamplingParams> uploaded_params;
    std::vector<long long> uploaded_streams, uploaded_steps;
    bool uploaded = false;

    // queued decode runs: token feedback on the device
    int run_cap = 0;
    std::unique_ptr<DeviceBuffer> run_history, run_iteration;
    std::unique_ptr<PinnedBuffer> run_history_host;

    ~Impl() {
        for (auto& kv : graphs)
            if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    }
    void drop_graphs() {
        for (auto& kv : graphs)
            if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
        graphs.clear();
    }
};

Engine::Engine(std::shared_ptr<DecoderModel> m, const EngineOptions& o) : model(std::move(m)), ws(o.poison_freed), options(o), impl_(new Impl) {
    if (!model || model->device < 0) throw Error("the model has no weights bound; use load_model()");
    ops::cuda_check(cudaSetDevice(model->device), "selecting the model's device");
    dtype = model->dtype;
    vocab = model->plan.vocab_size;
    ops::cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "creating the engine's stream");
    // pages are whole: round the budget up
    const long long max_tokens = (std::max<long long>(o.max_tokens, 1) + VM_PAGE_TOKENS - 1) / VM_PAGE_TOKENS * VM_PAGE_TOKENS;
    cache = std::make_unique<SequenceCache>(model->cache_needs(), model->cache_shares(), max_tokens, model->plan.max_positions, dtype, stream, o.max_slots);
    impl_->err = std::make_unique<DeviceBuffer>(sizeof(int), true);
    // (waiting for the device after every launch, a debugging switch of the launch wrappers, cannot be recorded)
    use_graphs = (o.use_graphs != 0) && model->graph_safe() && !ops::sync_every_op();
}

Engine::~Engine() {
    if (stream) cudaStreamSynchronize(stream);
    impl_.reset();
    cache.reset();
    if (stream) cudaStreamDestroy(stream);
}

void Engine::synchronize() { ops::cuda_check(cudaStreamSynchronize(stream), "waiting for the engine's stream"); }

void Engine::raise_if_error() {
    int code = 0;
    ops::cuda_check(cudaMemcpyAsync(&code, impl_->err->ptr, sizeof(int), cudaMemcpyDeviceToHost, stream), "reading the error word");
    synchronize();
    if (code) {
        ops::cuda_check(cudaMemsetAsync(impl_->err->ptr, 0, sizeof(int), stream), "clearing the error word");
        throw CacheError("a kernel reported " + error_word_meaning(code));
    }
}

void Engine::copy_logits_to_host(const float* dev, int rows, float* host) {
    if (rows <= 0) return;
    const size_t bytes = static_cast<size_t>(rows) * vocab * sizeof(float);
    ops::cuda_check(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, stream), "copying logits to the host");
    synchronize();
    counters.d2h_bytes += static_cast<long long>(bytes);
}

namespace {

void validate(const Engine& e, const std::vector<Entry>& entries, int extra) {
    const CacheBook& book = e.cache->book;
    std::vector<char> seen(static_cast<size_t>(book.max_slots), 0);
    std::vector<std::pair<int, int>> need;
    for (const Entry& en : entries) {
        if (!book.slots.is_held(en.slot)) throw CacheError(format("slot %d is not open", en.slot));
        if (seen[en.slot]) throw ArgumentError(format("slot %d appears twice in one step", en.slot));
        seen[en.slot] = 1;
        const int n = static_cast<int>(en.tokens.size());
        if (n == 0 && !en.want.empty()) throw ArgumentError(format("slot %d: logits wanted but no tokens given", en.slot));
        for (int t : en.tokens)
            if (t < 0 || t >= e.vocab)     // the reference checks ids on the host before its embedding kernel too (src/executable.cpp:54-72)
                throw ArgumentError(format("slot %d: token id %d outside the vocabulary of %d", en.slot, t, e.vocab));
        for (int w : en.want)
            if (w < 0 || w >= n) throw ArgumentError(format("slot %d: wanted place %d outside the %d tokens of this step", en.slot, w, n));
        const int new_len = book.length[en.slot] + n + extra;
        if (new_len > book.max_positions)
            throw CacheError(format("slot %d would reach %d tokens; the model's limit is %d", en.slot, new_len, book.max_positions));
        need.emplace_back(en.slot, new_len);
    }
    if (!book.can_hold(need)) throw CacheError("out of cache pages for this step: the live sequences and the new tokens exceed max_tokens");
}

// Cut a step that brings more than max_step_tokens into pieces, in order.
std::vector<std::vector<Chunk>> cut(const std::vector<Entry>& entries, int max_step_tokens) {
    std::vector<std::vector<Chunk>> chunks;
    std::vector<Chunk> cur;
    int room = max_step_tokens;
    for (int i = 0; i < static_cast<int>(entries.size()); ++i) {
        int a = 0;
        const int n = static_cast<int>(entries[i].tokens.size());
        while (a < n) {
            const int take = std::min(n - a, room);
            cur.push_back(Chunk{i, a, a + take});
            a += take;
            room -= take;
            if (room == 0) {
                chunks.push_back(cur);
                cur.clear();
                room = max_step_tokens;
            }
        }
    }
    if (!cur.empty()) chunks.push_back(cur);
    return chunks;
}

// Per cache group, how wide the block tables of a batch of these slots are: the most blocks any of them holds, rounded up to
// a power of two (few distinct step shapes), at most the table's own width.
std::vector<int> table_widths(const CacheBook& book, const std::vector<int>& slots) {
    std::vector<int> widths;
    for (const PageBook& g : book.groups) {
        int need = 1;
        for (int s : slots) need = std::max(need, g.blocks_end[s]);
        int w = 1;
        while (w < need) w *= 2;
        widths.push_back(std::min(w, g.max_blocks));
    }
    return widths;
}

std::string widths_text(const std::vector<int>& w) {
    std::string s;
    for (int x : w) s += std::to_string(x) + ",";
    return s;
}

struct Described {
    Descriptors* desc = nullptr;
    int T = 0, B = 0, R = 0;
    std::vector<int> widths, new_len;
    std::vector<std::pair<int, int>> wanted;       // (entry, place) of the rows this piece produces, in order
    std::string lens;                              // new tokens per sequence, as part of a recorded step's shape
};

}  // namespace

// ------------------------------------------------------------------------------------------------ internals that need Impl
namespace {

float* logits_buffer(Engine& e, Engine::Impl& im, int rows) {
    const int cap = bucket(std::max(rows, 1));
    if (!im.logits || im.logits_cap < cap) {
        e.synchronize();                           // a step in flight may still write the old buffer
        im.logits.reset();
        im.logits = std::make_unique<DeviceBuffer>(static_cast<size_t>(cap) * e.vocab * sizeof(float));
        im.logits_cap = cap;
    }
    return static_cast<float*>(im.logits->ptr);
}

Descriptors& descriptors(Engine::Impl& im, int T, int B, int R, const std::vector<int>& widths) {
    const int Tc = bucket(T), Bc = bucket(B, 1), Rc = R > 0 ? bucket(R) : 0;
    const std::string key = format("%d/%d/%d/", Tc, Bc, Rc) + widths_text(widths);
    auto it = im.descs.find(key);
    if (it == im.descs.end()) it = im.descs.emplace(key, std::make_unique<Descriptors>(Tc, Bc, Rc, widths)).first;
    return *it->second;
}

// Reserve cache room for a piece of a step and write its descriptors.  `reserve_extra` tokens of room are reserved beyond
// the piece's own (decode runs that queue several steps).
Described describe(Engine& e, Engine::Impl& im, const std::vector<Entry>& entries, const std::vector<Chunk>& chunk, int reserve_extra) {
    CacheBook& book = e.cache->book;
    Described out;
    out.B = static_cast<int>(chunk.size());
    std::vector<int> slots;
    for (const Chunk& c : chunk) {
        const Entry& en = entries[c.entry];
        out.T += c.last - c.first;
        book.reserve(en.slot, book.length[en.slot] + (c.last - c.first) + reserve_extra);
        slots.push_back(en.slot);
    }
    out.widths = table_widths(book, slots);
    for (const Chunk& c : chunk)
        for (int w : entries[c.entry].want)
            if (c.first <= w && w < c.last) out.wanted.emplace_back(c.entry, w);
    out.R = static_cast<int>(out.wanted.size());
    Descriptors& d = descriptors(im, out.T, out.B, out.R, out.widths);
    d.wait_reusable();
    out.desc = &d;
    int *tok = d.h(d.tokens), *pos = d.h(d.positions), *sot = d.h(d.seq_of_token), *cu = d.h(d.cu_tokens), *sl = d.h(d.slots),
        *cl = d.h(d.ctx_len), *lr = d.h(d.logit_rows);
    int t0 = 0;
    cu[0] = 0;
    std::vector<int> start_of(entries.size(), 0);
    for (int s = 0; s < out.B; ++s) {
        const Chunk& c = chunk[s];
        const Entry& en = entries[c.entry];
        const int n = c.last - c.first, base = book.length[en.slot];
        for (int j = 0; j < n; ++j) {
            tok[t0 + j] = en.tokens[c.first + j];
            pos[t0 + j] = base + j;
            sot[t0 + j] = s;
        }
        sl[s] = en.slot;
        cl[s] = base + n;
        out.new_len.push_back(base + n);
        start_of[c.entry] = t0 - c.first;
        t0 += n;
        cu[s + 1] = t0;
        if (out.T != out.B) out.lens += std::to_string(n) + ",";
    }
    for (int r = 0; r < out.R; ++r) lr[r] = start_of[out.wanted[r].first] + out.wanted[r].second;
    for (size_t g = 0; g < book.groups.size(); ++g) {
        const int w = out.widths[g];
        int* tab = d.h(d.tables[g]);
        for (int s = 0; s < out.B; ++s) std::memcpy(tab + static_cast<size_t>(s) * w, book.groups[g].table_row(sl[s]), static_cast<size_t>(w) * sizeof(int));
    }
    d.upload(e.stream);
    return out;
}

StepContext make_context(Engine& e, Engine::Impl& im, const Described& ds, float* logits) {
    const Descriptors& d = *ds.desc;
    StepContext ctx;
    ctx.T = ds.T; ctx.B = ds.B; ctx.R = ds.R;
    ctx.T_cap = d.T_cap; ctx.B_cap = d.B_cap; ctx.R_cap = d.R_cap;
    ctx.hidden = e.model->plan.hidden_size;
    ctx.tokens = d.d(d.tokens); ctx.positions = d.d(d.positions); ctx.seq_of_token = d.d(d.seq_of_token); ctx.cu_tokens = d.d(d.cu_tokens);
    ctx.slots = d.d(d.slots); ctx.ctx_len = d.d(d.ctx_len); ctx.logit_rows = d.d(d.logit_rows);
    ctx.host_positions = d.h(d.positions); ctx.host_cu_tokens = d.h(d.cu_tokens); ctx.host_ctx_len = d.h(d.ctx_len); ctx.host_slots = d.h(d.slots);
    for (size_t g = 0; g < d.tables.size(); ++g) ctx.tables.push_back(d.d(d.tables[g]));
    ctx.table_widths = ds.widths;
    for (int b = 0; b < ds.B; ++b) {
        ctx.max_ctx_len = std::max(ctx.max_ctx_len, ctx.host_ctx_len[b]);
        ctx.max_new = std::max(ctx.max_new, ctx.host_cu_tokens[b + 1] - ctx.host_cu_tokens[b]);
    }
    ctx.one_token_each = ctx.max_new == 1 && ds.T == ds.B;
    ctx.logits = logits;
    ctx.act_dtype = e.dtype;
    ctx.err = static_cast<int*>(im.err->ptr);
    ctx.stream = e.stream;
    ctx.ws = &e.ws;
    ctx.cache = e.cache.get();
    ctx.schedule = &e.model->plan.schedule;
    ctx.fused_prefill_rows = e.options.fused_prefill_rows;
    ctx.sm_count = ops::sm_count();
    return ctx;
}

std::string bucket_of(const Engine& e, const StepContext& ctx) {
    return format("%d/%d/%d/%d/%d", ctx.T_cap, ctx.B_cap, ctx.R_cap, ctx.one_token_each ? 1 : 0, e.options.fused_prefill_rows);   // decode steps take other scratch
}

template <class Body> void run_eager(Engine& e, const std::string& bkt, Body&& body) {
    e.ws.begin(bkt, e.stream);
    try {
        body();
    } catch (...) {
        e.ws.abort();
        throw;
    }
    e.ws.end();
}

// Record `body()` (the launches of one step) into a CUDA graph and keep it under `key`.
template <class Body> Engine::Impl::Graph& record(Engine& e, Engine::Impl& im, StepContext& ctx, const std::string& bkt, const std::string& key, Body&& body) {
    if (im.graphs.size() >= 256) im.drop_graphs();
    ctx.capturing = true;
    e.synchronize();
    const ops::Counters before = ops::counters();
    e.ws.begin(bkt, e.stream);
    cudaGraph_t graph = nullptr;
    ops::cuda_check(cudaStreamBeginCapture(e.stream, cudaStreamCaptureModeRelaxed), "beginning to record a step");
    try {
        body();
    } catch (...) {
        cudaStreamEndCapture(e.stream, &graph);
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        e.ws.abort();
        ctx.capturing = false;
        throw;
    }
    const cudaError_t ended = cudaStreamEndCapture(e.stream, &graph);
    e.ws.end();
    ctx.capturing = false;
    ops::cuda_check(ended, "recording a step");
    Engine::Impl::Graph g;
    const cudaError_t made = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    ops::cuda_check(made, "instantiating a recorded step");
    // what a replay launches: counted once here, added to the counters at every replay
    ops::Counters& now = ops::counters();
    g.own_launches = now.own_launches - before.own_launches;
    g.library_calls = now.library_calls - before.library_calls;
    g.tc_attention_calls = now.tc_attention_calls - before.tc_attention_calls;
    now.own_launches = before.own_launches;
    now.library_calls = before.library_calls;
    now.tc_attention_calls = before.tc_attention_calls;
    ++e.counters.graphs_recorded;
    return im.graphs[key] = g;
}

void replay(Engine& e, const Engine::Impl::Graph& g) {
    ops::cuda_check(cudaGraphLaunch(g.exec, e.stream), "replaying a recorded step");
    ops::Counters& c = ops::counters();
    c.own_launches += g.own_launches;
    c.library_calls += g.library_calls;
    c.tc_attention_calls += g.tc_attention_calls;
}

// Run the model on a described step: from its CUDA graph where there is one, else part by part.
void execute(Engine& e, Engine::Impl& im, const Described& ds, float* logits) {
    StepContext ctx = make_context(e, im, ds, logits);
    const std::string bkt = bucket_of(e, ctx);
    bool graphed = e.use_graphs && e.ws.planned(bkt) && !ops::op_times_active();
    const std::string shape = bkt + format("|%d/%d/%d/%p/%llu|", ds.T, ds.B, ds.R, static_cast<void*>(logits), static_cast<unsigned long long>(e.ws.generation)) +
                              widths_text(ds.widths) + "|" + ds.lens;
    if (graphed && !ctx.one_token_each) {
        // other steps (prompts) are recorded only when the very same shape comes a second time
        if (im.shape_seen.size() > 4096) im.shape_seen.clear();
        graphed = ++im.shape_seen[shape] >= 2;
    }
    if (graphed) {
        auto it = im.graphs.find(shape);
        if (it == im.graphs.end()) {
            Engine::Impl::Graph& g = record(e, im, ctx, bkt, shape, [&] { e.model->forward(ctx); });
            replay(e, g);
        } else {
            replay(e, it->second);
        }
        return;
    }
    run_eager(e, bkt, [&] { e.model->forward(ctx); });
}

}  // namespace

// ------------------------------------------------------------------------------------------------ one step
const float* Engine::step(const std::vector<Entry>& entries, int* rows_out) {
    Impl& im = *impl_;
    validate(*this, entries, 0);
    int n_rows = 0, total = 0;
    for (const Entry& en : entries) {
        n_rows += static_cast<int>(en.want.size());
        total += static_cast<int>(en.tokens.size());
    }
    if (rows_out) *rows_out = n_rows;
    float* logits = logits_buffer(*this, im, n_rows);
    std::vector<std::vector<Chunk>> chunks;
    if (total <= options.max_step_tokens) {
        std::vector<Chunk> all;
        for (int i = 0; i < static_cast<int>(entries.size()); ++i)
            if (!entries[i].tokens.empty()) all.push_back(Chunk{i, 0, static_cast<int>(entries[i].tokens.size())});
        if (!all.empty()) chunks.push_back(all);
    } else {
        chunks = cut(entries, options.max_step_tokens);
    }
    // rows come out in processing order; `produced` is compared with the asked-for order below
    std::vector<std::pair<int, int>> produced;
    int row0 = 0;
    const ops::Counters before = ops::counters();
    for (const auto& chunk : chunks) {
        const Described ds = describe(*this, im, entries, chunk, 0);
        execute(*this, im, ds, logits + static_cast<size_t>(row0) * vocab);
        for (int s = 0; s < ds.B; ++s) cache->book.commit(entries[chunk[s].entry].slot, ds.new_len[s]);
        produced.insert(produced.end(), ds.wanted.begin(), ds.wanted.end());
        row0 += ds.R;
    }
    const ops::Counters& now = ops::counters();
    counters.own_launches += now.own_launches - before.own_launches;
    counters.library_calls += now.library_calls - before.library_calls;
    counters.h2d_bytes += now.h2d_bytes - before.h2d_bytes;
    counters.tc_attention_calls += now.tc_attention_calls - before.tc_attention_calls;
    ++counters.steps;
    std::vector<std::pair<int, int>> asked;
    for (int i = 0; i < static_cast<int>(entries.size()); ++i)
        for (int w : entries[i].want) asked.emplace_back(i, w);
    if (produced != asked) {
        // a piece produces an entry's rows in the order of `want`, but an entry cut over several pieces with its places asked out
        // of order produces them piece by piece: copy the rows into the asked-for order
        const size_t row_bytes = static_cast<size_t>(vocab) * sizeof(float);
        if (!im.reordered || im.reordered->bytes < row_bytes * n_rows) im.reordered = std::make_unique<DeviceBuffer>(row_bytes * n_rows);
        for (int r = 0; r < n_rows; ++r) {
            const auto at = std::find(produced.begin(), produced.end(), asked[r]);
            const size_t from = static_cast<size_t>(at - produced.begin());
            ops::cuda_check(cudaMemcpyAsync(static_cast<char*>(im.reordered->ptr) + row_bytes * r, reinterpret_cast<const char*>(logits) + row_bytes * from,
                                            row_bytes, cudaMemcpyDeviceToDevice, stream),
                            "reordering logits");
        }
        return static_cast<const float*>(im.reordered->ptr);
    }
    return logits;
}

// ------------------------------------------------------------------------------------------------ the device sampler
namespace {
void sampler_room(Engine::Impl& im, int rows) {
    if (rows <= im.sampler_cap) return;
    const int cap = bucket(std::max(rows, 2 * im.sampler_cap), 64);
    const size_t bytes = static_cast<size_t>(cap) * (3 * 8 + 2 * 4);
    im.sampler_host = std::make_unique<PinnedBuffer>(bytes);
    im.sampler_dev = std::make_unique<DeviceBuffer>(bytes, true);
    im.sampled_host = std::make_unique<PinnedBuffer>(static_cast<size_t>(cap) * sizeof(int));
    im.sampled_dev = std::make_unique<DeviceBuffer>(static_cast<size_t>(cap) * sizeof(int));
    im.sampled_direct = static_cast<int*>(vm_host_device_pointer(im.sampled_host->ptr));
    im.sampler_cap = cap;
    im.uploaded = false;
}

struct SamplerBlock {
    long long *seed, *stream_id, *step;
    float *temperature, *top_p;
};
SamplerBlock block_at(void* base, int cap) {
    SamplerBlock b;
    long long* i64 = static_cast<long long*>(base);
    b.seed = i64; b.stream_id = i64 + cap; b.step = i64 + 2 * cap;
    float* f32 = reinterpret_cast<float*>(i64 + 3 * cap);
    b.temperature = f32; b.top_p = f32 + cap;
    return b;
}
}  // namespace

std::vector<int> Engine::sample(const float* logits, int R, const std::vector<SamplingParams>& params, const std::vector<long long>& streams,
                                const std::vector<long long>& steps) {
    Impl& im = *impl_;
    if (R <= 0) return {};
    if (static_cast<int>(params.size()) < R || static_cast<int>(streams.size()) < R || static_cast<int>(steps.size()) < R)
        throw ArgumentError("sample: one set of parameters, one stream and one step per row");
    sampler_room(im, R);
    // the same requests as at the last upload, all moved on by the same number of draws: the block on the device still serves,
    // and that number goes to the kernel as an argument
    long long step_add = 0;
    bool reuse = im.uploaded && static_cast<int>(im.uploaded_params.size()) == R;
    if (reuse) {
        step_add = steps[0] - im.uploaded_steps[0];
        for (int r = 0; r < R && reuse; ++r)
            reuse = params[r].same_draw(im.uploaded_params[r]) && streams[r] == im.uploaded_streams[r] && steps[r] - im.uploaded_steps[r] == step_add;
    }
    if (!reuse) {
        SamplerBlock h = block_at(im.sampler_host->ptr, im.sampler_cap);
        for (int r = 0; r < R; ++r) {
            h.temperature[r] = params[r].temperature; h.top_p[r] = params[r].top_p;
            h.seed[r] = params[r].seed; h.stream_id[r] = streams[r]; h.step[r] = steps[r];
        }
        ops::cuda_check(cudaMemcpyAsync(im.sampler_dev->ptr, im.sampler_host->ptr, im.sampler_host->bytes, cudaMemcpyHostToDevice, stream),
                        "uploading sampling parameters");
        counters.h2d_bytes += static_cast<long long>(im.sampler_host->bytes);
        im.uploaded_params.assign(params.begin(), params.begin() + R);
        im.uploaded_streams.assign(streams.begin(), streams.begin() + R);
        im.uploaded_steps.assign(steps.begin(), steps.begin() + R);
        im.uploaded = true;
        step_add = 0;
    }
    SamplerBlock d = block_at(im.sampler_dev->ptr, im.sampler_cap);
    const long long before = ops::counters().own_launches;
    if (im.sampled_direct) {
        ops::sample(logits, vocab, R, vocab, d.temperature, d.top_p, d.seed, d.stream_id, d.step, step_add, im.sampled_direct, stream);
    } else {
        int* out = static_cast<int*>(im.sampled_dev->ptr);
        ops::sample(logits, vocab, R, vocab, d.temperature, d.top_p, d.seed, d.stream_id, d.step, step_add, out, stream);
        ops::cuda_check(cudaMemcpyAsync(im.sampled_host->ptr, out, static_cast<size_t>(R) * sizeof(int), cudaMemcpyDeviceToHost, stream), "copying tokens");
    }
    counters.own_launches += ops::counters().own_launches - before;
    synchronize();
    counters.d2h_bytes += 4ll * R;
    const int* got = static_cast<const int*>(im.sampled_host->ptr);
    return std::vector<int>(got, got + R);
}

// ------------------------------------------------------------------------------------------------ several decode steps without the host
std::vector<std::vector<int>> Engine::decode_many(const std::vector<int>& slots, const std::vector<int>& last_tokens,
                                                  const std::vector<SamplingParams>& params, const std::vector<long long>& streams,
                                                  const std::vector<long long>& draw_steps, int k) {
    Impl& im = *impl_;
    const int B = static_cast<int>(slots.size());
    if (k < 1 || k > MAX_DECODE_RUN) throw ArgumentError(format("decode_many: k must be in 1..%d", MAX_DECODE_RUN));
    if (B == 0) return std::vector<std::vector<int>>(static_cast<size_t>(k));
    if (static_cast<int>(last_tokens.size()) != B || static_cast<int>(params.size()) != B || static_cast<int>(streams.size()) != B ||
        static_cast<int>(draw_steps.size()) != B)
        throw ArgumentError("decode_many: one token, one set of parameters, one stream and one step per slot");
    std::vector<Entry> entries;
    std::vector<Chunk> chunk;
    for (int i = 0; i < B; ++i) {
        entries.push_back(Entry{slots[i], {last_tokens[i]}, {0}});
        chunk.push_back(Chunk{i, 0, 1});
    }
    validate(*this, entries, k - 1);
    sampler_room(im, B);
    if (im.run_cap < B) {
        const int cap = bucket(B);
        im.run_history = std::make_unique<DeviceBuffer>(static_cast<size_t>(MAX_DECODE_RUN) * cap * sizeof(int));
        im.run_history_host = std::make_unique<PinnedBuffer>(static_cast<size_t>(MAX_DECODE_RUN) * cap * sizeof(int));
        im.run_iteration = std::make_unique<DeviceBuffer>(sizeof(int), true);
        im.run_cap = cap;
    }
    float* logits = logits_buffer(*this, im, B);
    const ops::Counters before = ops::counters();
    const Described ds = describe(*this, im, entries, chunk, k - 1);
    SamplerBlock h = block_at(im.sampler_host->ptr, im.sampler_cap);
    for (int r = 0; r < B; ++r) {
        h.temperature[r] = params[r].temperature; h.top_p[r] = params[r].top_p;
        h.seed[r] = params[r].seed; h.stream_id[r] = streams[r]; h.step[r] = draw_steps[r];
    }
    ops::cuda_check(cudaMemcpyAsync(im.sampler_dev->ptr, im.sampler_host->ptr, im.sampler_host->bytes, cudaMemcpyHostToDevice, stream),
                    "uploading sampling parameters");
    ops::counters().h2d_bytes += static_cast<long long>(im.sampler_host->bytes);
    im.uploaded = false;                           // the run advances the steps on the device: the block no longer matches a host copy
    ops::cuda_check(cudaMemsetAsync(im.run_iteration->ptr, 0, sizeof(int), stream), "clearing the run's step counter");
    StepContext ctx = make_context(*this, im, ds, logits);
    const std::string bkt = bucket_of(*this, ctx);
    SamplerBlock d = block_at(im.sampler_dev->ptr, im.sampler_cap);
    int* sampled = static_cast<int*>(im.sampled_dev->ptr);
    Descriptors& desc = *ds.desc;
    auto one_step = [&] {
        model->forward(ctx);
        ops::sample(logits, vocab, B, vocab, d.temperature, d.top_p, d.seed, d.stream_id, d.step, 0, sampled, stream);
        ops::decode_advance(sampled, desc.d_mut(desc.tokens), desc.d_mut(desc.positions), desc.d_mut(desc.ctx_len), d.step,
                            static_cast<int*>(im.run_history->ptr), static_cast<int*>(im.run_iteration->ptr), B, stream);
    };
    if (use_graphs && ws.planned(bkt) && !ops::op_times_active()) {
        const std::string key = "run|" + bkt + format("|%d/%p/%p/%llu|", B, static_cast<void*>(logits), static_cast<void*>(sampled),
                                                      static_cast<unsigned long long>(ws.generation)) + widths_text(ds.widths);
        auto it = im.graphs.find(key);
        const Impl::Graph* g = it == im.graphs.end() ? &record(*this, im, ctx, bkt, key, one_step) : &it->second;
        for (int i = 0; i < k; ++i) replay(*this, *g);
    } else {
        for (int i = 0; i < k; ++i) run_eager(*this, bkt, one_step);
    }
    const size_t bytes = static_cast<size_t>(k) * B * sizeof(int);
    ops::cuda_check(cudaMemcpyAsync(im.run_history_host->ptr, im.run_history->ptr, bytes, cudaMemcpyDeviceToHost, stream), "copying the run's tokens");
    synchronize();
    for (int i = 0; i < B; ++i) cache->book.commit(slots[i], ds.new_len[i] + k - 1);
    const ops::Counters& now = ops::counters();
    counters.own_launches += now.own_launches - before.own_launches;
    counters.library_calls += now.library_calls - before.library_calls;
    counters.h2d_bytes += now.h2d_bytes - before.h2d_bytes;
    counters.d2h_bytes += static_cast<long long>(bytes);
    counters.steps += k;
    const int* got = static_cast<const int*>(im.run_history_host->ptr);
    std::vector<std::vector<int>> rows(static_cast<size_t>(k));
    for (int i = 0; i < k; ++i) rows[i].assign(got + static_cast<size_t>(i) * B, got + static_cast<size_t>(i + 1) * B);
    return rows;
}

}  // namespace vmb
