// c_api.h — the C ABI of velomind_b200, for bindings (the Python package loads it through ctypes).
//
// Every function that can fail returns a negative status (or a null pointer) and leaves a message: vmb_last_error() gives
// its text, vmb_last_error_kind() which family it belongs to.  Handles are opaque pointers; each *_free takes what the
// matching *_create / *_load returned.  Texts that functions return (JSON, decoded strings) stay valid until the next call
// of this API on the same thread.  An engine and everything made from it belong to one host thread at a time.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

enum { VMB_ERROR_OTHER = 0, VMB_ERROR_CONFIG = 1, VMB_ERROR_WEIGHT = 2, VMB_ERROR_CACHE = 3, VMB_ERROR_KERNEL = 4, VMB_ERROR_ARGUMENT = 5 };
const char* vmb_last_error(void);
int vmb_last_error_kind(void);

// ---- configuration and weights (host only: these run without a GPU)
// The typed configuration of a config.json object, as JSON, with the architecture's plan summary; null on a ConfigError.
const char* vmb_config_describe(const char* config_json);
// name -> {"shape": [...], "float": bool, "ones": bool, "alias_of": name} of the model that `config_json` names; null on error
const char* vmb_weight_table(const char* config_json);
// Reads folder/config.json and folder/model.safetensors and checks the tensors against the model; 0 if they fit.
int vmb_check_model_folder(const char* folder);
// Random-weights mode: writes folder/config.json and folder/model.safetensors.  dtype "bfloat16" or "float32".
int vmb_write_random_model(const char* folder, const char* config_json, unsigned long long seed, double std, double norm_jitter, const char* dtype);
// Validates a safetensors header blob of `n` bytes against `data_bytes` bytes of payload; the tensor count, or negative.
int vmb_safetensors_check_header(const char* blob, long long n, long long data_bytes);
// name -> {"dtype", "shape"} of a safetensors file as stored (nothing is cast); null on error
const char* vmb_safetensors_info(const char* path);
const char* vmb_registered_architectures(void);       // JSON list
const char* vmb_smollm2_135m_config(void);            // the reference's built-in sizes as a config.json object

// ---- tokenizer (host only)
void* vmb_tokenizer_load(const char* path);
void* vmb_tokenizer_from_json(const char* tokenizer_json);
void vmb_tokenizer_free(void* tokenizer);
int vmb_tokenizer_encode(void* tokenizer, const char* text, int* out, int capacity);    // returns the count (may exceed capacity)
const char* vmb_tokenizer_decode(void* tokenizer, const int* ids, int n);
const char* vmb_pretokenize(const char* text);        // JSON list of pieces in the byte-to-unicode alphabet
int vmb_tokenizer_special(void* tokenizer, int which);  // 0 bos, 1 eos, 2 pad, 3 unk; -1 if none

// ---- model and engine
void* vmb_model_load(const char* folder, const char* dtype, const char* device);
void vmb_model_free(void* model);
const char* vmb_model_info(void* model);              // JSON: vocab, hidden, max_positions, stop_tokens, bos_token, runs, graph_safe, dtype

void* vmb_engine_create(void* model, long long max_tokens, int max_slots, int max_step_tokens, int use_graphs, int fused_prefill_rows, int poison_freed);
void vmb_engine_free(void* engine);
int vmb_engine_open(void* engine);                    // a slot, or negative
int vmb_engine_close(void* engine, int slot);
int vmb_engine_length(void* engine, int slot);
// One step.  Entry i has slot slots[i], n_tokens[i] tokens (concatenated in `tokens`) and n_want[i] wanted places (in `want`).
// *logits receives a DEVICE pointer to float32 [*rows, vocab], valid until the engine's next step; the work is queued on the
// engine's stream (vmb_engine_synchronize waits for it).
int vmb_engine_step(void* engine, int n_entries, const int* slots, const int* n_tokens, const int* tokens, const int* n_want, const int* want,
                    const float** logits, int* rows);
int vmb_engine_sample(void* engine, const float* logits, int rows, const float* temperature, const float* top_p, const long long* seed,
                      const long long* streams, const long long* steps, int* out_tokens);
int vmb_engine_decode_many(void* engine, int n, const int* slots, const int* last_tokens, const float* temperature, const float* top_p,
                           const long long* seed, const long long* streams, const long long* steps, int k, int* out_tokens /* [k, n] */);
int vmb_engine_synchronize(void* engine);
int vmb_engine_raise_if_error(void* engine);
int vmb_engine_logits_to_host(void* engine, const float* device_logits, int rows, float* host);
int vmb_engine_cache_check(void* engine);             // 0 if no slot or page is lost, held twice or owned by a closed slot
int vmb_engine_set_fail_after(void* engine, long long n_buffers);   // host-side fault injection; -1 switches it off
const char* vmb_engine_stats(void* engine);           // JSON: counters, cache, arena plans, vocab, dtype, graphs
unsigned long long vmb_engine_stream(void* engine);   // the engine's CUDA stream handle

// Generation loop over an engine.  Request i: prompt_lens[i] tokens of `prompts`, its own sampling parameters and Philox stream;
// n_stop[i] stop tokens of `stops` (n_stop[i] < 0: the `default_stop` list).  `on_token(user, request, token)` may be null.
// Returns JSON: {"results": [{"tokens", "finish_reason", "prompt_tokens"}], "timing": {...}}; null on error.
typedef void (*vmb_token_callback)(void* user, int request, int token);
const char* vmb_engine_generate(void* engine, int n, const int* prompt_lens, const int* prompts, const float* temperature, const float* top_p,
                                const int* max_tokens, const long long* seed, const long long* streams, const int* n_stop, const int* stops,
                                int n_default_stop, const int* default_stop, int max_batch, int steps_per_sync, vmb_token_callback on_token, void* user);

// ---- the text engine (the reference's facade)
typedef void (*vmb_piece_callback)(void* user, int request, int token, const char* piece);
typedef int (*vmb_sample_callback)(void* user, const float* row, int vocab);
void* vmb_text_create(const char* engine_config_json);
void vmb_text_free(void* text_engine);
int vmb_text_load(void* text_engine);
void* vmb_text_engine(void* text_engine);             // the Engine inside (owned by the text engine)
void* vmb_text_model(void* text_engine);
void* vmb_text_tokenizer(void* text_engine);          // null if the model folder has none
const char* vmb_text_describe(void* text_engine);
// options_json: temperature, top_p, max_tokens, seed, stop_tokens (absent: the model's), steps_per_sync.  Returns JSON as
// vmb_engine_generate plus "text", "elapsed_seconds", "tokens_per_second" per result.
const char* vmb_text_generate(void* text_engine, int n, const int* prompt_lens, const int* prompts, const char* options_json,
                              vmb_piece_callback on_token, vmb_sample_callback sample_fn, void* user);
int vmb_text_reset_session(void* text_engine);
int vmb_text_session_length(void* text_engine);
int vmb_text_prefill(void* text_engine, const int* tokens, int n, float* logits /* [vocab] */);
int vmb_text_forward_step(void* text_engine, int token, long long pos, float* logits /* [vocab] */);
int vmb_text_forward_logits(void* text_engine, const int* tokens, int n, float* logits /* [vocab] */);
int vmb_text_forward_full_logits(void* text_engine, const int* tokens, int n, float* logits /* [n, vocab] */);

// ---- debugging aids
void* vmb_op_times_begin(void);                       // device time per kind of operation from here on (CUDA graphs are off meanwhile)
const char* vmb_op_times_table(void* handle);
void vmb_op_times_end(void* handle);

#ifdef __cplusplus
}
#endif
