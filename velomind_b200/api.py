"""The Python entry point: load a model folder (or make a random one) and generate.

Names follow the reference's engine facade (examples/smollm2/smollm2_engine.h:16-81,
examples/common/llama/llama_engine.h:59-155): an `EngineConfig` with
`model_path`, `tokenizer_path`, `device`, `use_synthetic`, `model_config`; `load()`;
`generate(...)`; and the single-session calls `prefill`, `forward_step`,
`forward_logits`, `forward_full_logits`, `reset_session`.  Unlike the
reference, `generate` takes a batch of prompts, and config.json chooses the
model class.
"""
from __future__ import annotations

import os
import tempfile
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import torch

from . import models  # noqa: F401  (registers the architectures)
from .cache.pages import PAGE_TOKENS
from .engine.generate import GenerationLoop, Request, Result
from .engine.model import load_model
from .engine.step import Engine, Entry
from .sampling.sampler import DeviceSampler, SamplingParams
from .weights.synthetic import write_random_model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}

# examples/smollm2/model.h:11-22: the sizes the reference's `--synthetic` switch uses
SMOLLM2_135M: Dict[str, Any] = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 49152, "hidden_size": 576,
    "intermediate_size": 1536, "num_hidden_layers": 30, "num_attention_heads": 9, "num_key_value_heads": 3,
    "rms_norm_eps": 1e-5, "rope_theta": 100000.0, "max_position_embeddings": 8192, "tie_word_embeddings": True,
    "hidden_act": "silu",
}


@dataclass
class EngineConfig:
    model_path: str = ""                 # a folder with config.json and model.safetensors
    tokenizer_path: str = ""             # tokenizer.json; default: the one in model_path, if any
    device: str = "cuda:0"
    use_synthetic: bool = False          # random weights: `model_config` (a config.json object) and `seed`
    model_config: Optional[Dict[str, Any]] = None
    seed: int = 42
    dtype: str = "bfloat16"
    max_tokens: int = 65536              # cached tokens of live sequences (whole pages of 64)
    max_batch: int = 64
    use_graphs: Optional[bool] = None    # None: the engine's default (decode steps replayed from CUDA graphs)


class TextEngine:
    """Model + cache + sampler behind one object."""

    def __init__(self, config: EngineConfig):
        self.config = config
        self.engine: Optional[Engine] = None
        self.model = None
        self.tokenizer = None
        self.sampler: Optional[DeviceSampler] = None
        self._session_slot: Optional[int] = None
        self._tmp = None

    # ---- loading
    def load(self) -> "TextEngine":
        cfg = self.config
        if cfg.dtype not in DTYPES:
            raise ValueError(f"dtype {cfg.dtype!r}: choose bfloat16 or float32")
        folder = cfg.model_path
        if cfg.use_synthetic:
            self._tmp = tempfile.TemporaryDirectory(prefix="velomind_b200_synthetic_")
            folder = write_random_model(self._tmp.name, cfg.model_config or SMOLLM2_135M, seed=cfg.seed)
        elif not folder:
            raise ValueError("EngineConfig.model_path is empty (or set use_synthetic)")
        if os.path.isfile(folder):               # the reference takes the path of model.safetensors itself
            folder = os.path.dirname(folder) or "."
        self.model = load_model(folder, DTYPES[cfg.dtype], cfg.device)
        self.engine = Engine(self.model, cfg.max_tokens, use_graphs=cfg.use_graphs)
        self.sampler = DeviceSampler(self.engine.device, cfg.max_batch)
        tok_path = cfg.tokenizer_path or os.path.join(folder, "tokenizer.json")
        if os.path.isfile(tok_path):
            from .tokenizer import ByteLevelBPETokenizer
            self.tokenizer = ByteLevelBPETokenizer.from_file(tok_path)
        if self._tmp is not None:
            self._tmp.cleanup()
            self._tmp = None
        return self

    @property
    def is_loaded(self) -> bool:
        return self.engine is not None

    def _need(self) -> Engine:
        if self.engine is None:
            raise RuntimeError("call load() first")
        return self.engine

    # ---- generation
    def encode(self, prompt: Union[str, Sequence[int]]) -> List[int]:
        """Token ids of a prompt.  Text needs a tokenizer and gets the begin-of-sequence token in front if the
        tokenizer has one and the text does not start with it (examples/common/llama/llama_engine.cpp:596-602)."""
        if not isinstance(prompt, str):
            return [int(t) for t in prompt]
        if self.tokenizer is None:
            raise ValueError("a text prompt needs tokenizer.json; pass token ids instead")
        ids = self.tokenizer.encode(prompt)
        bos = self.tokenizer.bos_id
        if bos is not None and bos >= 0 and (not ids or ids[0] != bos):
            ids = [bos] + ids
        return ids

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]], temperature: float = 0.7, top_p: float = 0.9,
                 max_tokens: int = 32, seed: int = 42, stop_tokens: Optional[Sequence[int]] = None,
                 on_token: Optional[Callable[[int, int, str], None]] = None, steps_per_sync: int = 1,
                 sample_fn: Optional[Callable[[Any], int]] = None) -> List[Result]:
        """Generate for a batch of prompts (token id lists, or text if a tokenizer is loaded).
        `on_token(index, token, piece)` is called for every new token; `piece` is its text (or "[id]").
        `steps_per_sync`: decode steps queued on the GPU before the host reads their tokens.  1 (the default): every
        step, each token reaches `on_token` as it is made, and on a host that keeps up this is also the faster way;
        more: the host is out of the loop for that many steps, at the price of steps computed past a stop token.
        `sample_fn(logits) -> token`: the reference's way of sampling (llama_engine.h:106-121): a function of one row of
        float32 logits (a numpy array on the host) instead of temperature and top-p; every step's logits then come to
        the host."""
        engine = self._need()
        stops = tuple(stop_tokens) if stop_tokens is not None else self.default_stop_tokens()
        requests = [Request(self.encode(p), SamplingParams(temperature, top_p, max_tokens, seed, stops), stream=i)
                    for i, p in enumerate(prompts)]
        sampler = self.sampler if sample_fn is None else FunctionSampler(sample_fn)
        if sample_fn is not None:
            steps_per_sync = 1                   # (the function runs on the host after every step)
        loop = GenerationLoop(engine, sampler, engine.cache.n_pages, self.config.max_batch, stops, steps_per_sync)
        streamers = [TextStreamer(self.tokenizer) for _ in requests]
        callback = None
        if on_token is not None:
            def callback(i, tok):
                on_token(i, tok, streamers[i].put(tok))
        t0 = time.perf_counter()
        results = loop.run(requests, callback)
        elapsed = time.perf_counter() - t0
        self.last_timing = loop.timing
        engine.raise_if_error()
        for res in results:                      # the reference's result fields (llama_engine.h:32-38)
            res.text = (self.tokenizer.decode(res.tokens) if self.tokenizer is not None
                        else "".join(f"[{t}]" for t in res.tokens))
            res.elapsed_seconds = elapsed
            res.tokens_per_second = len(res.tokens) / elapsed if elapsed > 0 else 0.0
        return results

    def describe(self) -> Dict[str, Any]:
        """What the reference console's /model prints (llama_interactive_console.cpp:145-158): device, mode and the
        model's sizes, read from the plan's parts."""
        plan = self.model.plan
        first = plan.blocks[plan.schedule[0].layer] if plan.schedule else None
        mixer = first.mixer.args if first is not None else {}
        ff = first.feed_forward.args if first is not None else {}
        return {"Backend": self.config.device, "Mode": "Synthetic" if self.config.use_synthetic else "Real model",
                "Vocab": f"{plan.vocab_size} tokens", "Hidden": plan.hidden_size, "Layers": len(plan.schedule),
                "Heads": f"{mixer.get('heads', '?')} (kv={mixer.get('kv_heads', '?')})", "HeadDim": mixer.get("head_dim", "?"),
                "Intermed": ff.get("intermediate", "?"), "Dtype": self.config.dtype}

    def default_stop_tokens(self):
        if self.tokenizer is not None and self.tokenizer.eos_id is not None and self.tokenizer.eos_id >= 0:
            return (self.tokenizer.eos_id,)
        return tuple(self.model.plan.stop_tokens)

    # ---- the reference's single-session calls
    def reset_session(self) -> None:
        if self._session_slot is not None:
            self._need().close(self._session_slot)
            self._session_slot = None

    @property
    def session_length(self) -> int:
        return 0 if self._session_slot is None else self._need().length(self._session_slot)

    def prefill(self, tokens: Sequence[int]) -> torch.Tensor:
        """Start a session with `tokens`; float32 logits [vocab] of the last one (llama_engine.cpp:333-393)."""
        engine = self._need()
        self.reset_session()
        self._session_slot = engine.open()
        return engine.step([Entry(self._session_slot, list(tokens), [len(tokens) - 1])])[0].clone()

    def forward_step(self, token: int, pos: Optional[int] = None) -> torch.Tensor:
        """Feed one more token to the session; logits [vocab] (llama_engine.cpp:395-455).  `pos`, the reference's second
        argument, is the token's place in the session: it can only be the session's length, and is checked when given."""
        if self._session_slot is None:
            raise RuntimeError("forward_step needs a session: call prefill first")
        if pos is not None and int(pos) != self.session_length:
            raise ValueError(f"forward_step: pos {pos} is not the session's length {self.session_length}")
        return self._need().step([Entry(self._session_slot, [int(token)], [0])])[0].clone()

    def forward_full_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """Stateless: logits [len, vocab] of a whole sequence (llama_engine.cpp:523-585)."""
        engine = self._need()
        slot = engine.open()
        try:
            return engine.step([Entry(slot, list(tokens), list(range(len(tokens))))]).clone()
        finally:
            engine.close(slot)

    def forward_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """Stateless: logits [vocab] of the last token (llama_engine.cpp:457-521)."""
        engine = self._need()
        slot = engine.open()
        try:
            return engine.step([Entry(slot, list(tokens), [len(tokens) - 1])])[0].clone()
        finally:
            engine.close(slot)


class FunctionSampler:
    """A host function of one row of logits as the loop's sampler (the reference's `sample_fn`)."""

    def __init__(self, fn: Callable[[Any], int]):
        self.fn = fn

    def sample(self, logits, params, streams, steps):
        import numpy as np
        rows = logits.float().cpu().numpy()
        return np.array([int(self.fn(rows[r])) for r in range(rows.shape[0])], dtype=np.int32)


class TextStreamer:
    """Turns a growing token list into text pieces: decode everything so far and emit what is new, holding
    back an incomplete multi-byte character (examples/common/llama/llama_engine.cpp:43-112).  Without a
    tokenizer a token prints as "[id]" (:64-69)."""

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer
        self.tokens: List[int] = []
        self.emitted = ""

    def put(self, token: int) -> str:
        if self.tokenizer is None:
            return f"[{token}]"
        self.tokens.append(int(token))
        text = self.tokenizer.decode(self.tokens)
        if text.endswith("�"):      # the bytes so far end inside a character: wait for the rest
            return ""
        piece = text[len(self.emitted):]
        self.emitted = text
        return piece

    def flush(self) -> str:
        if self.tokenizer is None:
            return ""
        text = self.tokenizer.decode(self.tokens)
        piece = text[len(self.emitted):]
        self.emitted = text
        return piece


def load(model_path: str, dtype: str = "bfloat16", device: str = "cuda:0", max_tokens: int = 65536,
         max_batch: int = 64) -> TextEngine:
    """Shorthand: a loaded TextEngine for the model folder `model_path`."""
    return TextEngine(EngineConfig(model_path=model_path, dtype=dtype, device=device, max_tokens=max_tokens,
                                   max_batch=max_batch)).load()
