"""The Llama dense decoder as a plan of parts: pre-norm layers of grouped-query attention with rotary
positions and a SwiGLU feed-forward, RMSNorm everywhere, an optional tied head.

Layer wiring: examples/common/llama/llama_graph.cpp:165-248.  Tensor names:
examples/smollm2/model_loader.cpp:130,168-233,266,271.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import BlockSpec, ModelPlan, PartSpec, ScheduleEntry

EMBED = "model.embed_tokens."


def llama_plan(cfg: LlamaConfig) -> ModelPlan:
    position = PartSpec("rotary_half_split", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    blocks = []
    for l in range(cfg.num_hidden_layers):
        blocks.append(BlockSpec(
            arrangement="prenorm",
            prefix=f"model.layers.{l}.",
            mixer=PartSpec("grouped_query_attention", {
                "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "position": position}),
            feed_forward=PartSpec("swiglu", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size}),
            mixer_norm=norm,
            feed_forward_norm=norm,
            names={"mixer": "self_attn.", "feed_forward": "mlp.", "mixer_norm": "input_layernorm.",
                   "feed_forward_norm": "post_attention_layernorm."},
        ))
    return ModelPlan(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size}),
        embedding_prefix=EMBED,
        blocks=tuple(blocks),
        schedule=tuple(ScheduleEntry(l) for l in range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_prefix="model.norm.",
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size,
                                 "tied_to": EMBED + "weight" if cfg.tie_word_embeddings else None}),
        head_prefix="lm_head.",
        max_positions=cfg.max_position_embeddings,
        stop_tokens=tuple(cfg.eos_token_ids),
        bos_token=cfg.bos_token_id,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_plan)
