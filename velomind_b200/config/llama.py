"""Typed configuration of the Llama dense decoder, read from the keys of its config.json.

Required keys and their meaning follow the reference's parser
(examples/smollm2/config_parser.cpp:205-213) and its `llama::Config`
(examples/common/llama/llama_config.h:7-24).  Keys the reference never reads
but which change the arithmetic (rope scaling, biases, another activation)
are rejected instead of ignored.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader

# llama_config.h:22 — what the reference's struct holds when config.json gives no context limit.
_DEFAULT_MAX_POSITIONS = 2048


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    @property
    def queries_per_kv_head(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @staticmethod
    def from_dict(data: Dict[str, Any], where: str = "config.json") -> "LlamaConfig":
        r = KeyReader(data, where)
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        # llama_config.h:14-16: zero kv heads means "as many as heads".
        kv = r.integer("num_key_value_heads", minimum=0)
        if kv == 0:
            kv = heads
        if heads % kv != 0:
            # llama_graph.cpp:179-182
            raise ConfigError(f"{where}: num_attention_heads ({heads}) must be divisible by num_key_value_heads ({kv})")
        if "head_dim" in data and data["head_dim"] is not None:
            head_dim = r.integer("head_dim")
        else:
            if hidden % heads != 0:
                # llama_graph.cpp:172-174
                raise ConfigError(f"{where}: hidden_size ({hidden}) must be divisible by num_attention_heads ({heads})")
            head_dim = hidden // heads  # llama_config.h:17-19
        if head_dim % 2 != 0:
            raise ConfigError(f"{where}: head size {head_dim} is odd; rotary pairs need an even size")
        r.absent_or("rope_scaling", [], "scaled rotary positions are not implemented")
        r.absent_or("attention_bias", [False], "projection biases are not implemented")
        r.absent_or("mlp_bias", [False], "feed-forward biases are not implemented")
        r.absent_or("hidden_act", ["silu"], "the feed-forward gate is SiLU")
        r.absent_or("sliding_window", [], "this architecture attends to all earlier tokens")
        bos = data.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError(f"{where}: key 'bos_token_id' must be an integer, found {bos!r}")
        cfg = LlamaConfig(
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=r.integer("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps"),
            rope_theta=r.number("rope_theta"),
            # config_parser.cpp:213 falls back to the tied constant of examples/smollm2/model.h:21
            tie_word_embeddings=r.boolean("tie_word_embeddings", True),
            max_position_embeddings=r.integer("max_position_embeddings", _DEFAULT_MAX_POSITIONS),
            eos_token_ids=r.int_or_list("eos_token_id"),
            bos_token_id=bos,
        )
        for t in cfg.eos_token_ids + ((cfg.bos_token_id,) if cfg.bos_token_id is not None else ()):
            if not 0 <= t < cfg.vocab_size:
                raise ConfigError(f"{where}: special token id {t} lies outside the vocabulary of {cfg.vocab_size}")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        """The config.json object that reads back as this configuration."""
        d: Dict[str, Any] = {
            "architectures": ["LlamaForCausalLM"],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu",
        }
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d
