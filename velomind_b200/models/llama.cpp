// The Llama dense decoder as a plan of parts: pre-norm layers of grouped-query attention with rotary positions and a
// SwiGLU feed-forward, RMSNorm everywhere, an optional tied head.
//
// Layer wiring: examples/common/llama/llama_graph.cpp:165-248.  Tensor names:
// examples/smollm2/model_loader.cpp:130,168-233,266,271.
#include "velomind_b200/velomind.h"

namespace vmb {

// examples/smollm2/model.h:11-22: the sizes the reference's `--synthetic` switch uses
const char* const SMOLLM2_135M_CONFIG =
    "{\"architectures\": [\"LlamaForCausalLM\"], \"model_type\": \"llama\", \"vocab_size\": 49152, \"hidden_size\": 576, "
    "\"intermediate_size\": 1536, \"num_hidden_layers\": 30, \"num_attention_heads\": 9, \"num_key_value_heads\": 3, "
    "\"rms_norm_eps\": 1e-05, \"rope_theta\": 100000.0, \"max_position_embeddings\": 8192, \"tie_word_embeddings\": true, "
    "\"hidden_act\": \"silu\"}";

ModelPlan llama_plan(const LlamaConfig& cfg) {
    static const char* kEmbed = "model.embed_tokens.";
    json::Value pos_args;
    pos_args.set("head_dim", cfg.head_dim);
    pos_args.set("theta", cfg.rope_theta);
    json::Value position;
    position.set("kind", "rotary_half_split");
    position.set("args", pos_args);
    json::Value norm_args;
    norm_args.set("size", cfg.hidden_size);
    norm_args.set("eps", cfg.rms_norm_eps);
    const PartSpec norm{"rmsnorm", norm_args};

    ModelPlan plan;
    plan.hidden_size = cfg.hidden_size;
    plan.vocab_size = cfg.vocab_size;
    for (int l = 0; l < cfg.num_hidden_layers; ++l) {
        BlockSpec b;
        b.arrangement = "prenorm";
        b.prefix = format("model.layers.%d.", l);
        json::Value m;
        m.set("hidden", cfg.hidden_size);
        m.set("heads", cfg.num_attention_heads);
        m.set("kv_heads", cfg.num_key_value_heads);
        m.set("head_dim", cfg.head_dim);
        m.set("position", position);
        b.mixer = PartSpec{"grouped_query_attention", m};
        json::Value f;
        f.set("hidden", cfg.hidden_size);
        f.set("intermediate", cfg.intermediate_size);
        b.feed_forward = PartSpec{"swiglu", f};
        b.mixer_norm = norm;
        b.feed_forward_norm = norm;
        b.names = {{"mixer", "self_attn."}, {"feed_forward", "mlp."}, {"mixer_norm", "input_layernorm."},
                   {"feed_forward_norm", "post_attention_layernorm."}};
        plan.blocks.push_back(std::move(b));
        plan.schedule.push_back(ScheduleEntry{l, -1});
    }
    json::Value e;
    e.set("vocab", cfg.vocab_size);
    e.set("hidden", cfg.hidden_size);
    plan.embedding = PartSpec{"token_table", e};
    plan.embedding_prefix = kEmbed;
    plan.final_norm = norm;
    plan.final_norm_prefix = "model.norm.";
    json::Value h;
    h.set("vocab", cfg.vocab_size);
    h.set("hidden", cfg.hidden_size);
    if (cfg.tie_word_embeddings) h.set("tied_to", std::string(kEmbed) + "weight");
    plan.head = PartSpec{"linear", h};
    plan.head_prefix = "lm_head.";
    plan.max_positions = cfg.max_position_embeddings;
    plan.stop_tokens = cfg.eos_token_ids;
    plan.bos_token = cfg.bos_token_id;
    // what the reference console's /model prints (llama_interactive_console.cpp:145-158)
    json::Value d;
    d.set("Vocab", format("%d tokens", cfg.vocab_size));
    d.set("Hidden", cfg.hidden_size);
    d.set("Layers", cfg.num_hidden_layers);
    d.set("Heads", format("%d (kv=%d)", cfg.num_attention_heads, cfg.num_key_value_heads));
    d.set("HeadDim", cfg.head_dim);
    d.set("Intermed", cfg.intermediate_size);
    plan.describe = d;
    return plan;
}

namespace {
struct RegisterLlama {
    RegisterLlama() {
        register_architecture("LlamaForCausalLM", [](const json::Value& config, const std::string& where) {
            return llama_plan(LlamaConfig::from_json(config, where));
        });
    }
} register_llama;
}  // namespace

}  // namespace vmb
