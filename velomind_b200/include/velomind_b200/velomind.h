// velomind.h — the C++ API of velomind_b200: a small generation library for one NVIDIA B200 (sm_100a).
//
// Everything between a request's tokens and its next token: a typed configuration read from config.json, a
// registry from the architecture's name to its model, weights from safetensors bound by name, layers built from
// parts (norm, position encoding, mixer, feed-forward, arrangement), a paged cache with a slot per sequence, ONE
// step function for batches of unequal sequences, a generation loop, device samplers, a tokenizer and a console.
//
// The counterpart of the reference's engine facade (examples/smollm2/smollm2_engine.h:28-81,
// examples/common/llama/llama_engine.h:59-155): `TextEngine` keeps its method names (`load`, `generate`, `prefill`,
// `forward_step`, `forward_logits`, `forward_full_logits`, `reset_session`).  Unlike the reference, `generate` takes a
// batch of prompts, config.json chooses the model class, and nothing is rebuilt or allocated per token.
//
// Threading: an Engine and everything it owns belong to one host thread at a time.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace vmb {

// ------------------------------------------------------------------------------------------------ errors
struct Error : std::runtime_error { using std::runtime_error::runtime_error; };
struct ConfigError : Error { using Error::Error; };        // config.json: a key is missing, of the wrong kind, or unsupported
struct WeightError : Error { using Error::Error; };        // the tensors of a folder do not match the model
struct CacheError : Error { using Error::Error; };         // the cache was asked for more than it holds, or was misused
struct KernelError : Error { using Error::Error; };        // a launcher refused its arguments or CUDA reported an error
struct ArgumentError : Error { using Error::Error; };      // a caller's argument is wrong (a bad token id, a slot twice)

std::string format(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

// ------------------------------------------------------------------------------------------------ JSON
namespace json {
class Value;
using Array = std::vector<Value>;
using Member = std::pair<std::string, Value>;
using Object = std::vector<Member>;          // keeps the file's order; keys are unique (the parser refuses duplicates)

class Value {
public:
    enum Kind { Null, Bool, Number, String, ArrayKind, ObjectKind };
    Value() = default;
    Value(std::nullptr_t) {}
    Value(bool b) : kind_(Bool), b_(b) {}
    Value(int v) : kind_(Number), num_(v), int_(v), is_int_(true) {}
    Value(long long v) : kind_(Number), num_(static_cast<double>(v)), int_(v), is_int_(true) {}
    Value(double v) : kind_(Number), num_(v) {}
    Value(const char* s) : kind_(String), str_(s) {}
    Value(std::string s) : kind_(String), str_(std::move(s)) {}
    Value(Array a);
    Value(Object o);

    Kind kind() const { return kind_; }
    bool is_null() const { return kind_ == Null; }
    bool is_bool() const { return kind_ == Bool; }
    bool is_number() const { return kind_ == Number; }
    bool is_integer() const { return kind_ == Number && is_int_; }   // written without fraction or exponent, or a whole double
    bool is_string() const { return kind_ == String; }
    bool is_array() const { return kind_ == ArrayKind; }
    bool is_object() const { return kind_ == ObjectKind; }
    bool as_bool() const { return b_; }
    double as_double() const { return num_; }
    long long as_int() const { return int_; }
    const std::string& as_string() const { return str_; }
    const Array& as_array() const;
    const Object& as_object() const;
    Array& array();
    Object& object();
    const Value* find(const std::string& key) const;     // member of an object, or nullptr
    void set(const std::string& key, Value v);           // add or replace a member (makes this an object if null)
    bool operator==(const Value& o) const;
    std::string dump(int indent = -1) const;             // -1: one line

private:
    Kind kind_ = Null;
    bool b_ = false;
    double num_ = 0.0;
    long long int_ = 0;
    bool is_int_ = false;
    std::string str_;
    std::shared_ptr<Array> arr_;
    std::shared_ptr<Object> obj_;
};

// Throws Error("<where>: not valid JSON: <what> at byte N").  `no_duplicate_keys`: an object that names a key twice is refused.
Value parse(const std::string& text, const std::string& where = "JSON", bool no_duplicate_keys = true);
}  // namespace json

// ------------------------------------------------------------------------------------------------ dtypes
enum class DType { F32, BF16, F16, I32, I64, I16, I8, U8, BOOL };
size_t dtype_size(DType t);
const char* dtype_name(DType t);                 // the safetensors name ("F32", "BF16", ...)
std::optional<DType> dtype_from_name(const std::string& name);
bool dtype_is_float(DType t);
uint16_t float_to_bf16(float x);                 // round to nearest even
float bf16_to_float(uint16_t x);
float f16_to_float(uint16_t x);

// ------------------------------------------------------------------------------------------------ configuration
// Typed reading of config.json keys; every getter checks type and range and names the key on failure.
class KeyReader {
public:
    KeyReader(const json::Value& data, std::string where);
    long long integer(const std::string& key, long long minimum = 1) const;
    long long integer_or(const std::string& key, long long fallback, long long minimum = 1) const;
    double number(const std::string& key, bool positive = true) const;
    double number_or(const std::string& key, double fallback, bool positive = true) const;
    bool boolean_or(const std::string& key, bool fallback) const;
    std::string string_or(const std::string& key, const std::string& fallback) const;
    std::vector<int> int_or_list(const std::string& key) const;      // absent/null -> {}, an int -> {int}, a list -> list
    bool has(const std::string& key) const;                          // present and not null
    // reject an option this library does not implement instead of ignoring it
    void absent_or(const std::string& key, const std::vector<json::Value>& allowed, const std::string& why) const;
    const std::string& where() const { return where_; }
    const json::Value& data() const { return data_; }

private:
    const json::Value* get(const std::string& key) const;
    const json::Value& data_;
    std::string where_;
};

json::Value read_config_json(const std::string& folder_or_file);

// The Llama dense decoder's configuration.  Required keys follow the reference's parser
// (examples/smollm2/config_parser.cpp:205-213) and its `llama::Config` (examples/common/llama/llama_config.h:7-24).
struct LlamaConfig {
    int vocab_size = 0, hidden_size = 0, intermediate_size = 0, num_hidden_layers = 0;
    int num_attention_heads = 0, num_key_value_heads = 0, head_dim = 0;
    double rms_norm_eps = 0.0, rope_theta = 0.0;
    bool tie_word_embeddings = true;
    int max_position_embeddings = 0;
    std::vector<int> eos_token_ids;
    std::optional<int> bos_token_id;

    static LlamaConfig from_json(const json::Value& data, const std::string& where = "config.json");
    json::Value to_json() const;
};

// ------------------------------------------------------------------------------------------------ the plan of a model
// One part: the registry kind and the arguments of its constructor (sizes, eps, theta ...), a JSON object.
struct PartSpec {
    std::string kind;
    json::Value args;
};

// One layer: an arrangement (how norms, mixer, feed-forward and residual are wired) and its parts.
struct BlockSpec {
    std::string arrangement;                  // registry kind of the wiring, e.g. "prenorm"
    std::string prefix;                       // weight-name prefix of this layer in the checkpoint
    PartSpec mixer, feed_forward, mixer_norm, feed_forward_norm;
    std::map<std::string, std::string> names; // part -> sub-prefix, e.g. {"mixer": "self_attn."}
};

// One run of a layer.  `layer` indexes ModelPlan::blocks (a layer may appear several times); `cache_of` names the
// schedule position whose cache this run reads instead of writing its own (-1: the run owns a cache of its own).
struct ScheduleEntry {
    int layer = 0;
    int cache_of = -1;
};

struct ModelPlan {
    int hidden_size = 0, vocab_size = 0;
    PartSpec embedding;
    std::string embedding_prefix;
    std::vector<BlockSpec> blocks;
    std::vector<ScheduleEntry> schedule;
    PartSpec final_norm;
    std::string final_norm_prefix;
    PartSpec head;
    std::string head_prefix;
    int max_positions = 0;
    std::vector<int> stop_tokens;
    std::optional<int> bos_token;
    json::Value describe;                     // what a console's /model shows (sizes by name), filled by the architecture
    void validate() const;
};

// The registry from an architecture's name (config.json `architectures[0]`) to its model: a function that reads the
// typed configuration from the config.json object and returns the plan the engine builds parts from.
using PlanFunction = std::function<ModelPlan(const json::Value& config, const std::string& where)>;
void register_architecture(const std::string& name, PlanFunction plan);
void unregister_architecture(const std::string& name);
std::vector<std::string> registered_architectures();
std::string architecture_name(const json::Value& config, const std::string& where = "config.json");
const PlanFunction& resolve_architecture(const json::Value& config, const std::string& where = "config.json");
ModelPlan llama_plan(const LlamaConfig& cfg);

// ------------------------------------------------------------------------------------------------ weights
struct WeightSpec {
    std::vector<long long> shape;
    bool is_float = true;                     // false: an integer table
    bool init_ones = false;                   // random-weights mode: 1 + U(-jitter, jitter) instead of N(0, std)
    std::string alias_of;                     // if the file lacks this tensor, the named tensor stands in (tied head)
};
using WeightTable = std::map<std::string, WeightSpec>;

// A tensor in host memory, dtype as stored.  `data` points into `owner` (a mapped file or a byte vector).
struct HostTensor {
    DType dtype = DType::F32;
    std::vector<long long> shape;
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
    std::shared_ptr<void> owner;
    long long numel() const;
};
using HostTensors = std::map<std::string, HostTensor>;

// The safetensors container (8-byte header length, JSON header, raw bytes).  The checks follow the reference's reader
// (src/safetensors.cpp:253-377, 412-452, 508-546).  Errors are WeightError.
HostTensors load_safetensors(const std::string& path);
void save_safetensors(const HostTensors& tensors, const std::string& path, const std::map<std::string, std::string>& metadata = {});
// Validates a header blob against `data_bytes` bytes of payload; returns name -> (dtype, shape, begin, end).
struct TensorEntry { DType dtype; std::vector<long long> shape; long long begin = 0, end = 0; };
std::map<std::string, TensorEntry> parse_safetensors_header(const std::string& blob, long long data_bytes);

// Reads `folder/model.safetensors` and checks it against the model's table; ONE WeightError lists missing and
// unexpected tensors, wrong shapes and wrong kinds of dtype.  (The reference checks presence and dtype only,
// examples/smollm2/model_loader.cpp:115-119,31-34.)
HostTensors load_weights(const std::string& folder, const WeightTable& specs);
HostTensors check_and_bind(const HostTensors& found, const WeightTable& specs, const std::string& where);

struct RandomInit { double std = 0.02, norm_jitter = 0.1; std::string dtype = "bfloat16"; };
// Random-weights mode: writes `folder/config.json` and `folder/model.safetensors` for the architecture that `config` names.
// Each tensor's values depend on (seed, tensor name, index) only.
std::string write_random_model(const std::string& folder, const json::Value& config, uint64_t seed = 0, const RandomInit& init = {});

// ------------------------------------------------------------------------------------------------ device memory
struct DeviceBuffer {                          // owns cudaMalloc'd memory
    void* ptr = nullptr;
    size_t bytes = 0;
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t n, bool zero = false);
    ~DeviceBuffer();
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
};
struct PinnedBuffer {                          // page-locked host memory
    void* ptr = nullptr;
    size_t bytes = 0;
    PinnedBuffer() = default;
    explicit PinnedBuffer(size_t n);
    ~PinnedBuffer();
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
};
struct DeviceTensor {                          // a weight on the device
    void* ptr = nullptr;
    DType dtype = DType::F32;
    std::vector<long long> shape;
    std::shared_ptr<DeviceBuffer> owner;
    long long rows() const { return shape.empty() ? 0 : shape[0]; }
    long long cols() const { return shape.size() < 2 ? 1 : shape[1]; }
};

int require_cuda(const std::string& device);   // "cuda" / "cuda:N" -> N, made current; anything else, or no GPU: KernelError

// Where and in which dtype a model is being put on the device.  Host tensors that several parts share (a tied head
// and the embedding table) become one device tensor too.
class BindContext {
public:
    BindContext(DType dtype, cudaStream_t stream) : dtype(dtype), stream(stream) {}
    DType dtype;                               // the engine's activation dtype: F32 or BF16
    cudaStream_t stream;
    DeviceTensor upload(const HostTensor& t, DType as);
    DeviceTensor upload_stacked(const std::vector<const HostTensor*>& parts, DType as);   // rows of several matrices, one tensor
    DeviceTensor upload_floats(const std::vector<float>& values);
    // dtype a weight matrix is kept in: the compute dtype, except that a tensor stored in 32-bit stays 32-bit
    DType matrix_dtype(const std::vector<const HostTensor*>& stored) const;

private:
    std::map<std::pair<const uint8_t*, int>, DeviceTensor> uploads_;
};

// ------------------------------------------------------------------------------------------------ the cache
class CacheError;
// Hands out integers 0..n-1, lowest free id first; refuses misuse (an id freed twice or never handed out).
class FreeList {
public:
    FreeList(int n, std::string what);
    int take();
    std::vector<int> take_many(int k);
    void give(int i);
    bool is_held(int i) const { return i >= 0 && i < n_ && held_[i]; }
    int free_count() const { return static_cast<int>(free_.size()); }
    int held_count() const { return n_ - static_cast<int>(free_.size()); }
    int size() const { return n_; }
    void check() const;                        // every id is either held or exactly once on the free list

private:
    int n_;
    std::string what_;
    std::vector<int> free_;                    // sorted descending: back() is the lowest
    std::vector<char> held_;
};

// What one run of a mixer keeps per sequence.
struct CacheNeed {
    enum Kind { None, All, Window } kind = None;   // every earlier key/value; the last `window`; nothing
    int kv_heads = 0;
    int key_dim = 0, value_dim = 0;                // per head; the paged storage of this library wants them equal
    int window = 0;
    int state_floats = 0;                          // fixed-size float32 state per sequence (0: none)
    bool same_group(const CacheNeed& o) const {
        return kind == o.kind && kv_heads == o.kv_heads && key_dim == o.key_dim && value_dim == o.value_dim && window == o.window;
    }
};

// Host bookkeeping of the pages and block tables of the layers that share one CacheNeed (no device memory here).
class PageBook {
public:
    PageBook(const CacheNeed& need, int n_pages, int max_slots, int max_blocks);
    int pages_needed(int slot, int new_len) const;
    void ensure(int slot, int new_len);            // give `slot` pages so that tokens [0, new_len) have a place
    void trim(int slot, int length);               // a window group gives back the pages no later query can reach
    void release(int slot);
    const int* table_row(int slot) const { return &table_[static_cast<size_t>(slot) * max_blocks]; }
    CacheNeed need;
    int n_pages, max_slots, max_blocks;
    FreeList pages;
    std::vector<int> blocks_begin, blocks_end;     // logical blocks [begin, end) of a slot hold a page
    uint64_t version = 0;                          // grows whenever an entry of the block table changes

private:
    std::vector<int> table_;                       // [max_slots, max_blocks], -1 where none
    friend class CacheBook;
};

// Slots for sequences; for each slot its length and its pages in every group.  Host only.
class CacheBook {
public:
    // needs[i]: the CacheNeed of schedule position i; shares[i] >= 0: the run reads that position's cache instead.
    CacheBook(const std::vector<CacheNeed>& needs, const std::vector<int>& shares, long long max_tokens, int max_positions, int max_slots = 0);
    int open();
    void close(int slot);
    bool can_hold(const std::vector<std::pair<int, int>>& slot_new_len) const;
    void reserve(int slot, int new_len);           // room for tokens [length, new_len) in every group, or CacheError and no change
    void commit(int slot, int new_len);
    long long tokens_held() const;                 // tokens of live sequences, each rounded up to whole pages
    void check() const;                            // no slot or page lost, held twice or owned by a closed slot
    std::pair<int, int> where(int run) const { return where_[run]; }   // (group, layer in group) or (-1, -1)
    int n_pages, max_positions, max_blocks, max_slots;
    FreeList slots;
    std::vector<int> length;
    std::vector<PageBook> groups;
    std::vector<int> layers_in_group;
    std::vector<int> state_floats;                 // per schedule position (0: none); shared runs name their owner's
    std::vector<int> state_owner;                  // schedule position whose state area a run uses (-1: none)

private:
    std::vector<std::pair<int, int>> where_;
};

// The book plus the device storage: k/v[layer, page, kv_head, VM_PAGE_TOKENS, head_dim] per group, and a float32 state area
// [max_slots, n] for every run that asks for one (zeroed when a slot is opened).  Keys are stored after the position
// encoding, as the reference caches them (examples/common/llama/llama_graph.cpp:210-215).
class SequenceCache {
public:
    SequenceCache(const std::vector<CacheNeed>& needs, const std::vector<int>& shares, long long max_tokens, int max_positions,
                  DType dtype, cudaStream_t stream, int max_slots = 0);
    int open();
    void close(int slot) { book.close(slot); }
    CacheBook book;
    DType dtype;
    struct GroupStorage { std::unique_ptr<DeviceBuffer> k, v; size_t layer_bytes = 0; };
    std::vector<GroupStorage> storage;
    std::vector<std::shared_ptr<DeviceBuffer>> state;   // per schedule position (null: none)
    void* k_pages(int group, int layer) const;
    void* v_pages(int group, int layer) const;

private:
    cudaStream_t stream_;
};

// ------------------------------------------------------------------------------------------------ activation memory
// Liveness intervals packed into one arena: best-fit-decreasing with 256-byte alignment, in the reference's manner
// (src/internal/graph_compiler.cpp:147-191 liveness, :286-398 placement; statistics as include/velomind/graph.h:40-46).
struct ArenaPlan {
    std::vector<size_t> offsets, sizes;
    size_t peak_bytes = 0;
    int buffer_count = 0, reused_count = 0;
    long long bytes_saved = 0;
};
struct Interval { size_t bytes; int birth, death; };      // alive over [birth, death] inclusive
ArenaPlan plan_arena(const std::vector<Interval>& intervals);

// Hands out step buffers.  The first step of a capacity bucket records the sequence of requests (with ordinary
// allocations); the plan made from it serves every later step of the bucket from one arena without allocating.
class Workspace {
public:
    explicit Workspace(bool poison = false);
    ~Workspace();
    void begin(const std::string& bucket, cudaStream_t stream);
    void* take(size_t bytes);
    void give(void* p);                         // nullptr is ignored
    void end();
    void abort();
    bool planned(const std::string& bucket) const;
    const ArenaPlan* plan(const std::string& bucket) const;
    uint64_t generation = 0;                    // bumped when the arena moves (recorded graphs must be dropped)
    bool poison;                                // debugging aid: a buffer that is given back is filled with NaN bytes
    long long fail_after = -1;                  // host-side fault injection: the N-th buffer of a step is refused (-1: off)
    size_t arena_bytes() const { return arena_ ? arena_->bytes : 0; }

private:
    struct Live { int index; size_t bytes; };
    std::unique_ptr<DeviceBuffer> arena_;
    std::vector<std::unique_ptr<DeviceBuffer>> loose_;     // the recording step's ordinary allocations, freed at end()
    std::map<std::string, ArenaPlan> plans_;
    std::string key_;
    bool open_ = false, recording_ = false;
    std::vector<Interval> log_;
    std::unordered_map<void*, Live> live_;
    int clock_ = 0, next_ = 0;
    cudaStream_t stream_ = nullptr;
};

// ------------------------------------------------------------------------------------------------ a step, as the parts see it
class Norm;
struct RotaryTable {                            // what a position encoding hands to the mixer's kernels
    const float* inv_freq = nullptr;            // device float32 [rotary_dim / 2], or null: no rotation
    int rotary_dim = 0;
    int pairing = 0;                            // VM_PAIR_HALF_SPLIT or VM_PAIR_INTERLEAVED
};

struct KVView {
    void* k_pages = nullptr;                    // [n_pages, kv_heads, VM_PAGE_TOKENS, head_dim]
    void* v_pages = nullptr;
    const int* block_table = nullptr;           // device int32 [B, table_width]
    int table_width = 0, n_pages = 0;
    bool owns = true;                           // false: the run reads another run's cache and must not write it
};

// Packed tokens and their places, the cache, scratch buffers.  Device arrays (int32): tokens [T], positions [T] (place of
// each token in its sequence), seq_of_token [T] (index into the batch), cu_tokens [B+1], slots [B], ctx_len [B] (length
// after this step), logit_rows [R].  Host copies of the same live in host_*.
struct StepContext {
    int T = 0, B = 0, R = 0, T_cap = 0, B_cap = 0, R_cap = 0;
    int hidden = 0;                             // width of the residual stream
    const int *tokens = nullptr, *positions = nullptr, *seq_of_token = nullptr, *cu_tokens = nullptr, *slots = nullptr,
              *ctx_len = nullptr, *logit_rows = nullptr;
    const int *host_positions = nullptr, *host_cu_tokens = nullptr, *host_ctx_len = nullptr, *host_slots = nullptr;
    std::vector<const int*> tables;             // per cache group: device block table of the batch
    std::vector<int> table_widths;
    int max_ctx_len = 0, max_new = 0;
    bool one_token_each = false;
    bool capturing = false;                     // the step is being recorded: no choice may depend on lengths, only on shape
    int run = -1;                               // the schedule position that is running
    float* logits = nullptr;                    // [R, vocab]
    DType act_dtype = DType::BF16;
    int* err = nullptr;                         // device error word
    cudaStream_t stream = nullptr;
    Workspace* ws = nullptr;
    SequenceCache* cache = nullptr;
    const std::vector<ScheduleEntry>* schedule = nullptr;
    int fused_prefill_rows = 0;                 // steps with at least this many tokens use the fused tcgen05 products (0: never)
    int sm_count = 0;

    void* take_tokens(long long cols, DType dtype);     // [T, cols], backed by T_cap rows so that a bucket's plan fits every step
    void* take(long long elements, DType dtype);
    void give(void* p) { ws->give(p); }
    KVView kv() const;                          // the cache of the running schedule position
    float* state() const;                       // its float32 state [max_slots, n] (index with `slots`), or null
    int state_floats() const;
};

// ------------------------------------------------------------------------------------------------ parts
// None knows which model it is in; each gets its sizes and constants from a PartSpec.  Roles: "norm", "position",
// "mixer", "feed_forward", "arrangement", "embedding", "head".
using Weights = std::map<std::string, HostTensor>;

class Part {
public:
    virtual ~Part() = default;
    virtual WeightTable weight_specs() const { return {}; }
    virtual void bind(const Weights&, BindContext&) {}
    // True only for parts whose forward launches the same work for every step of the same SHAPE (token, sequence and row
    // counts, table widths) and reads everything else from device memory: such a step can be recorded into a CUDA graph.
    virtual bool graph_safe() const { return false; }
};

class Norm : public Part {
public:
    // h float32 [T, hid] residual; delta (activation dtype, may be null) is added to h first; out (activation dtype)
    // receives norm(h) for all T rows, or for the n_rows rows named by `rows` (then h is not written).
    virtual void forward(StepContext& ctx, float* h, const void* delta, void* out, const int* rows, int n_rows) = 0;
    // (weight, eps) if this is a root-mean-square norm that a product kernel may fuse; false otherwise
    virtual bool as_rms(const float** weight, float* eps) const { (void)weight; (void)eps; return false; }
};

class Position : public Part {
public:
    virtual RotaryTable tables(BindContext& bc) = 0;
};

class Mixer : public Part {
public:
    virtual CacheNeed cache_need() const { return {}; }
    virtual void forward(StepContext& ctx, const void* x, void* out) = 0;       // x, out [T, hid] activation dtype
    // optional: take the norm before the part and the residual sum after it into the part's own kernels
    virtual bool can_fuse(const StepContext&, const Norm&) const { return false; }
    virtual void forward_fused(StepContext&, float* /*h*/, Norm&) {}
};

class FeedForward : public Part {
public:
    virtual void forward(StepContext& ctx, const void* x, void* out) = 0;
    virtual bool can_fuse(const StepContext&, const Norm&) const { return false; }
    virtual void forward_fused(StepContext&, float* /*h*/, Norm&) {}
};

struct BlockParts {
    std::shared_ptr<Mixer> mixer;
    std::shared_ptr<FeedForward> feed_forward;
    std::shared_ptr<Norm> mixer_norm, feed_forward_norm;
};

class Arrangement : public Part {
public:
    // wires norms, parts and the residual; `pending` is a delta (activation dtype) not yet added to h, or null;
    // returns the delta this layer leaves pending (a workspace buffer the caller gives back), or null
    virtual void* forward(StepContext& ctx, float* h, void* pending) = 0;
};

class Embedding : public Part {
public:
    virtual void forward(StepContext& ctx, const int* tokens, float* h) = 0;
};

class Head : public Part {
public:
    virtual void forward(StepContext& ctx, const void* x_rows, float* logits) = 0;   // x_rows [R, hid] activation dtype
};

// Registries of part kinds: `factory(args)` returns the part.  Registering a kind needs no change to this library.
using PartFactory = std::function<std::shared_ptr<Part>(const json::Value& args)>;
using ArrangementFactory = std::function<std::shared_ptr<Arrangement>(const json::Value& args, const BlockParts& parts)>;
void register_part(const std::string& role, const std::string& kind, PartFactory factory);
void register_arrangement(const std::string& kind, ArrangementFactory factory);
void unregister_part(const std::string& role, const std::string& kind);
std::vector<std::string> registered_parts(const std::string& role);
std::shared_ptr<Part> build_part(const std::string& role, const PartSpec& spec);
template <class T> std::shared_ptr<T> build_part_as(const std::string& role, const PartSpec& spec) {
    auto p = std::dynamic_pointer_cast<T>(build_part(role, spec));
    if (!p) throw ConfigError(format("the %s of kind '%s' does not have the interface of its role", role.c_str(), spec.kind.c_str()));
    return p;
}
std::shared_ptr<Arrangement> build_arrangement(const std::string& kind, const json::Value& args, const BlockParts& parts);
PartSpec part_spec_from_json(const json::Value& v, const std::string& what);     // {"kind": ..., "args": {...}}

// Error words of kernels, registered by the part that may raise them; Engine::raise_if_error looks them up.
void register_error_word(int code, const std::string& meaning);
std::string error_word_meaning(int code);

// ------------------------------------------------------------------------------------------------ the model
class Layer {
public:
    explicit Layer(const BlockSpec& spec);
    BlockSpec spec;
    BlockParts parts;
    std::shared_ptr<Arrangement> block;
    std::vector<std::pair<std::string, Part*>> named_parts() const;
};

// A decoder built from a plan: embedding, layers run in the plan's order, final norm, head.  Nothing here names an architecture.
class DecoderModel {
public:
    explicit DecoderModel(ModelPlan plan);
    WeightTable weight_table() const;
    void bind(const HostTensors& tensors, DType dtype, int device, cudaStream_t stream);
    bool graph_safe() const;
    std::vector<CacheNeed> cache_needs() const;    // one per schedule position (kind None where the run shares a cache)
    std::vector<int> cache_shares() const;
    void forward(StepContext& ctx);                // logits [R, vocab] at ctx.logit_rows into ctx.logits
    ModelPlan plan;
    std::shared_ptr<Embedding> embedding;
    std::vector<Layer> layers;
    std::shared_ptr<Norm> final_norm;
    std::shared_ptr<Head> head;
    DType dtype = DType::BF16;
    int device = -1;                               // -1: no weights bound
    json::Value config;

private:
    std::vector<std::pair<std::string, Part*>> named_parts() const;
};

WeightTable weight_table(const ModelPlan& plan);
DType compute_dtype(const std::string& name);      // "bfloat16"/"bf16" or "float32"/"fp32"
// Read config.json, choose the architecture by its name, build the parts, load and bind the weights.
std::shared_ptr<DecoderModel> load_model(const std::string& folder, DType dtype, const std::string& device = "cuda:0");

// ------------------------------------------------------------------------------------------------ sampling
// Option names and defaults follow the reference's command line (examples/smollm2/interactive_main.cpp:23-25,39-41):
// temperature 0.7 (0 or less: greedy), top-p 0.9 (0 or less: greedy), 32 tokens; its fixed seed is 42 (:113).
struct SamplingParams {
    float temperature = 0.7f, top_p = 0.9f;
    int max_tokens = 32;
    long long seed = 42;
    std::vector<int> stop_tokens;
    bool greedy() const { return temperature <= 0 || top_p <= 0; }
    bool same_draw(const SamplingParams& o) const { return temperature == o.temperature && top_p == o.top_p && seed == o.seed; }
};

// ------------------------------------------------------------------------------------------------ the engine
// One sequence's share of a step: its slot, its next tokens, and the places among these tokens whose logits are wanted.
struct Entry {
    int slot = 0;
    std::vector<int> tokens;
    std::vector<int> want;
};

struct EngineOptions {
    long long max_tokens = 65536;                  // cached tokens of live sequences (rounded up to whole pages)
    int max_slots = 0;                             // 0: as many as pages, at most 4,096
    int max_step_tokens = 8192;                    // a step that brings more is cut into pieces
    int use_graphs = -1;                           // -1: the default (on where the model allows it); 0 / 1
    int fused_prefill_rows = 0;                    // steps with at least this many tokens use the fused tcgen05 products (0: never)
    bool poison_freed = false;                     // debugging aid: scratch buffers are filled with NaN when given back
};

struct EngineCounters {                            // what ran since the engine was made
    long long own_launches = 0, library_calls = 0, h2d_bytes = 0, d2h_bytes = 0, steps = 0, graphs_recorded = 0, tc_attention_calls = 0;
};

class Descriptors;
class Engine {
public:
    Engine(std::shared_ptr<DecoderModel> model, const EngineOptions& options = {});
    ~Engine();
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    int open() { return cache->open(); }
    void close(int slot) { cache->close(slot); }
    int length(int slot) const { return cache->book.length[slot]; }

    // Run the entries' tokens as one batch from the cache; float32 logits [wanted, vocab] on the device, in the order of
    // the entries and of each entry's `want`.  Valid until the next step.  `rows` receives the number of rows.
    const float* step(const std::vector<Entry>& entries, int* rows = nullptr);

    // Feed `last_tokens` (one per slot) and decode `k` tokens for every slot: each step's sampled tokens are fed back on the
    // device.  Returns [k][B]: the tokens sampled after each step.  Every slot's length has grown by k.
    static constexpr int MAX_DECODE_RUN = 64;
    std::vector<std::vector<int>> decode_many(const std::vector<int>& slots, const std::vector<int>& last_tokens,
                                              const std::vector<SamplingParams>& params, const std::vector<long long>& streams,
                                              const std::vector<long long>& draw_steps, int k);

    // One token per row of device logits [R, vocab]: row r uses params[r] and the Philox counter (steps[r], streams[r]).
    std::vector<int> sample(const float* logits, int R, const std::vector<SamplingParams>& params,
                            const std::vector<long long>& streams, const std::vector<long long>& steps);

    void synchronize();
    void raise_if_error();                         // synchronise and throw if a kernel left an error word
    void copy_logits_to_host(const float* dev, int rows, float* host);

    std::shared_ptr<DecoderModel> model;
    std::unique_ptr<SequenceCache> cache;
    Workspace ws;
    EngineOptions options;
    EngineCounters counters;
    DType dtype;
    int vocab;
    cudaStream_t stream = nullptr;
    bool use_graphs = false;

    struct Impl;                                   // descriptors, recorded graphs, sampler buffers (engine/step.cpp)
    std::unique_ptr<Impl> impl_;
};

// ------------------------------------------------------------------------------------------------ the generation loop
struct Request {
    std::vector<int> prompt;
    SamplingParams params;
    long long stream = 0;                          // Philox stream of this request (its index, by default)
};

// What the reference returns per call (llama_engine.h:32-38), per sequence.
struct Result {
    std::vector<int> tokens;
    std::string finish_reason;                     // "stop" (a stop token, kept in `tokens`), "length", "empty", "error"
    int prompt_tokens = 0;
    std::string text;
    double elapsed_seconds = 0.0, tokens_per_second = 0.0;
};

struct Timing {
    double prefill_seconds = 0.0, decode_seconds = 0.0;
    long long decode_steps = 0, generated_tokens = 0;
    double tokens_per_second() const {
        const double t = prefill_seconds + decode_seconds;
        return t > 0 ? generated_tokens / t : 0.0;
    }
};

// What the loop needs of an engine, so that its decisions can be tested without a GPU.
class Stepper {
public:
    virtual ~Stepper() = default;
    virtual int open() = 0;
    virtual void close(int slot) = 0;
    // one step; returns one sampled token per entry (the logits wanted at each entry's last token)
    virtual std::vector<int> step_and_sample(const std::vector<Entry>& entries, const std::vector<SamplingParams>& params,
                                             const std::vector<long long>& streams, const std::vector<long long>& drawn) = 0;
    virtual bool can_queue() const { return false; }
    virtual int max_run() const { return 1; }
    virtual std::vector<std::vector<int>> decode_many(const std::vector<int>&, const std::vector<int>&, const std::vector<SamplingParams>&,
                                                      const std::vector<long long>&, const std::vector<long long>&, int) {
        throw Error("this stepper cannot queue decode steps");
    }
};

int pages_for(const Request& r);                   // pages a request may come to hold: prompt plus every token it may feed back
// Cut the request list, in order, into batches that fit the cache (by pages) and `max_batch` slots.
std::vector<std::vector<int>> plan_batches(const std::vector<Request>& requests, int total_pages, int max_batch);

using TokenCallback = std::function<void(int request_index, int token)>;

// Batches of unequal prompts, stop tokens (kept in the output, not fed: llama_engine.cpp:633-653), sequences that end
// early and free their slot at once, batch after batch.  `max_tokens == 0` returns after nothing (:635-637).
class GenerationLoop {
public:
    GenerationLoop(Stepper& stepper, int total_pages, int max_batch, std::vector<int> default_stop = {}, int steps_per_sync = 1);
    std::vector<Result> run(const std::vector<Request>& requests, const TokenCallback& on_token = nullptr);
    Timing timing;

private:
    void run_batch(const std::vector<Request>& requests, const std::vector<int>& batch, std::vector<Result>& results, const TokenCallback& on_token);
    Stepper& stepper_;
    int total_pages_, max_batch_, steps_per_sync_;
    std::vector<int> default_stop_;
};

// An Engine as the loop's stepper: the step function and the device sampler.
class EngineStepper : public Stepper {
public:
    explicit EngineStepper(Engine& e) : engine(e) {}
    int open() override { return engine.open(); }
    void close(int slot) override { engine.close(slot); }
    std::vector<int> step_and_sample(const std::vector<Entry>& entries, const std::vector<SamplingParams>& params,
                                     const std::vector<long long>& streams, const std::vector<long long>& drawn) override;
    bool can_queue() const override { return true; }
    int max_run() const override { return Engine::MAX_DECODE_RUN; }
    std::vector<std::vector<int>> decode_many(const std::vector<int>& slots, const std::vector<int>& last, const std::vector<SamplingParams>& params,
                                              const std::vector<long long>& streams, const std::vector<long long>& drawn, int k) override {
        return engine.decode_many(slots, last, params, streams, drawn, k);
    }
    // optional: a host function of one row of float32 logits instead of the device sampler (the reference's `sample_fn`)
    std::function<int(const float* row, int vocab)> sample_fn;
    Engine& engine;
};

// ------------------------------------------------------------------------------------------------ text
// Byte-level BPE read from a Hugging Face tokenizer.json, as the reference's tokenizer (examples/smollm2/tokenizer.cpp).
class Tokenizer {
public:
    static std::shared_ptr<Tokenizer> from_file(const std::string& path);
    static std::shared_ptr<Tokenizer> from_json(const json::Value& root, const std::string& where);
    std::vector<int> encode(const std::string& text) const;
    std::string decode(const std::vector<int>& ids) const;        // skips the begin/end/pad ids; invalid UTF-8 becomes U+FFFD
    static std::vector<std::string> pretokenize(const std::string& text);   // pieces in the byte-to-unicode alphabet
    int bos_id = -1, eos_id = -1, pad_id = -1, unk_id = -1;

private:
    std::vector<std::string> bpe(const std::string& word) const;
    std::unordered_map<std::string, int> token_to_id_;
    std::vector<std::string> id_to_token_;
    std::unordered_map<std::string, int> rank_;                   // "a b" -> rank
};

// Turns a growing token list into text pieces: decode everything so far and emit what is new, holding back an incomplete
// multi-byte character (examples/common/llama/llama_engine.cpp:43-112).  Without a tokenizer a token prints as "[id]".
class TextStreamer {
public:
    explicit TextStreamer(std::shared_ptr<const Tokenizer> tokenizer = nullptr) : tokenizer_(std::move(tokenizer)) {}
    std::string put(int token);
    std::string flush();                                          // what was held back

private:
    std::shared_ptr<const Tokenizer> tokenizer_;
    std::vector<int> tokens_;
    size_t emitted_ = 0;                                          // bytes of the decoded text already given out
};

// ------------------------------------------------------------------------------------------------ the entry point
extern const char* const SMOLLM2_135M_CONFIG;      // examples/smollm2/model.h:11-22 as a config.json object

struct EngineConfig {
    std::string model_path;                        // a folder with config.json and model.safetensors (or the path of model.safetensors)
    std::string tokenizer_path;                    // tokenizer.json; default: the one in model_path, if any
    std::string device = "cuda:0";
    bool use_synthetic = false;                    // random weights: `model_config` (a config.json object) and `seed`
    json::Value model_config;
    long long seed = 42;
    std::string dtype = "bfloat16";
    long long max_tokens = 65536;
    int max_batch = 64;
    int use_graphs = -1;
};

struct GenerateOptions {
    float temperature = 0.7f, top_p = 0.9f;
    int max_tokens = 32;
    long long seed = 42;
    std::optional<std::vector<int>> stop_tokens;   // absent: the model's (or the tokenizer's) end-of-sequence ids
    int steps_per_sync = 1;                        // decode steps queued on the GPU before the host reads their tokens
    std::function<void(int index, int token, const std::string& piece)> on_token;   // token -1: the held-back rest of the text
    std::function<int(const float* row, int vocab)> sample_fn;
};

class TextEngine {
public:
    explicit TextEngine(EngineConfig config);
    ~TextEngine();
    TextEngine& load();
    bool is_loaded() const { return engine != nullptr; }
    std::vector<int> encode(const std::string& prompt) const;     // with the begin-of-sequence token in front (llama_engine.cpp:596-602)
    std::vector<Result> generate(const std::vector<std::vector<int>>& prompts, const GenerateOptions& options = {});
    std::vector<Result> generate_text(const std::vector<std::string>& prompts, const GenerateOptions& options = {});
    std::vector<int> default_stop_tokens() const;
    json::Value describe() const;
    // the reference's single-session calls; logits are host float32
    void reset_session();
    int session_length() const;
    std::vector<float> prefill(const std::vector<int>& tokens);
    std::vector<float> forward_step(int token, long long pos = -1);
    std::vector<float> forward_logits(const std::vector<int>& tokens);
    std::vector<float> forward_full_logits(const std::vector<int>& tokens);

    EngineConfig config;
    std::shared_ptr<DecoderModel> model;
    std::unique_ptr<Engine> engine;
    std::shared_ptr<Tokenizer> tokenizer;
    Timing last_timing;

private:
    int session_slot_ = -1;
};

// ------------------------------------------------------------------------------------------------ programs
int smollm2_chat_main(int argc, char** argv);      // the command line in the manner of examples/smollm2/interactive_main.cpp
int trace_run_main(int argc, char** argv);         // replay: feeds given token ids step by step and writes logits

}  // namespace vmb
