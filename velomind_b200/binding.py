"""The Python binding: thin classes over the C ABI of the library (include/velomind_b200/c_api.h), loaded through ctypes.

Nothing is computed here.  The model, the cache, the step function, the generation loop, the samplers and the tokenizer
are the C++ library's; this file turns Python lists into C arrays and device pointers into torch tensors.

Names follow the reference's engine facade where it has them (examples/smollm2/smollm2_engine.h:16-81): `EngineConfig`
with `model_path`, `tokenizer_path`, `device`, `use_synthetic`, `model_config`; `TextEngine.load()`, `generate`, `prefill`,
`forward_step`, `forward_logits`, `forward_full_logits`, `reset_session`.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .kernels.library import KernelLibraryError, library

_c_int, _c_ll, _c_f, _c_d, _c_p, _c_s = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double, ctypes.c_void_p, ctypes.c_char_p


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong kind, or asks for something unsupported."""


class WeightError(ValueError):
    """The tensors of a model folder do not match what the model expects."""


class CacheError(RuntimeError):
    """The cache was asked for more than it holds, or was misused."""


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


_KINDS = {1: ConfigError, 2: WeightError, 3: CacheError, 4: KernelError, 5: ValueError}
_declared = False


def _lib():
    global _declared
    lib = library()
    if not _declared:
        for name in ("vmb_last_error", "vmb_config_describe", "vmb_weight_table", "vmb_registered_architectures", "vmb_smollm2_135m_config",
                     "vmb_tokenizer_decode", "vmb_pretokenize", "vmb_safetensors_info", "vmb_model_info", "vmb_engine_stats", "vmb_engine_generate",
                     "vmb_text_describe", "vmb_text_generate", "vmb_op_times_table"):
            getattr(lib, name).restype = _c_s
        for name in ("vmb_tokenizer_load", "vmb_tokenizer_from_json", "vmb_model_load", "vmb_engine_create", "vmb_text_create",
                     "vmb_text_engine", "vmb_text_model", "vmb_text_tokenizer", "vmb_op_times_begin"):
            getattr(lib, name).restype = _c_p
        lib.vmb_engine_stream.restype = ctypes.c_ulonglong
        for name in ("vmb_tokenizer_free", "vmb_model_free", "vmb_engine_free", "vmb_text_free", "vmb_op_times_end"):
            getattr(lib, name).restype = None
            getattr(lib, name).argtypes = [_c_p]
        _declared = True
    return lib


def _raise():
    lib = _lib()
    text = (lib.vmb_last_error() or b"unknown error").decode("utf-8", "replace")
    raise _KINDS.get(lib.vmb_last_error_kind(), RuntimeError)(text)


def _ok(status: int) -> int:
    if status < 0:
        _raise()
    return status


def _text(value) -> str:
    if value is None:
        _raise()
    return value.decode("utf-8", "replace")


def _ints(values, ctype=ctypes.c_int):
    arr = (ctype * max(len(values), 1))()
    for i, v in enumerate(values):
        arr[i] = int(v)
    return arr


def _floats(values):
    arr = (ctypes.c_float * max(len(values), 1))()
    for i, v in enumerate(values):
        arr[i] = float(v)
    return arr


def _dtype_name(dtype) -> str:
    name = str(dtype).replace("torch.", "")
    if name in ("bfloat16", "bf16"):
        return "bfloat16"
    if name in ("float32", "fp32", "float"):
        return "float32"
    raise ValueError(f"dtype {dtype!r}: choose bfloat16 or float32")


# ------------------------------------------------------------------------------------------------ configuration and weights
def smollm2_135m_config() -> Dict[str, Any]:
    """examples/smollm2/model.h:11-22: the sizes the reference's `--synthetic` switch uses, as a config.json object."""
    return json.loads(_lib().vmb_smollm2_135m_config().decode())


def describe_config(config: Dict[str, Any]) -> Dict[str, Any]:
    """The typed configuration and the plan's summary of a config.json object (raises ConfigError)."""
    return json.loads(_text(_lib().vmb_config_describe(json.dumps(config).encode())))


def weight_table(config: Dict[str, Any]) -> Dict[str, Dict[str, Any]]:
    """name -> {"shape", "float", "ones", "alias_of"} of the model that `config` names."""
    return json.loads(_text(_lib().vmb_weight_table(json.dumps(config).encode())))


def check_model_folder(folder: str) -> None:
    """Reads config.json and model.safetensors of `folder` and checks the tensors against the model (no GPU needed)."""
    _ok(_lib().vmb_check_model_folder(str(folder).encode()))


def check_safetensors_header(blob: bytes, data_bytes: int) -> int:
    """Validates a safetensors header against `data_bytes` bytes of payload (raises WeightError); returns the tensor count."""
    return _ok(_lib().vmb_safetensors_check_header(blob, _c_ll(len(blob)), _c_ll(int(data_bytes))))


def safetensors_info(path: str) -> Dict[str, Dict[str, Any]]:
    """name -> {"dtype", "shape"} of a safetensors file, as stored."""
    return json.loads(_text(_lib().vmb_safetensors_info(str(path).encode())))


def registered_architectures() -> List[str]:
    return json.loads(_text(_lib().vmb_registered_architectures()))


def write_random_model(folder: str, config: Dict[str, Any], seed: int = 0, std: float = 0.02, norm_jitter: float = 0.1,
                       dtype: str = "bfloat16") -> str:
    """Random-weights mode: create `folder` with config.json and model.safetensors for the architecture that `config` names."""
    _ok(_lib().vmb_write_random_model(str(folder).encode(), json.dumps(config).encode(), ctypes.c_ulonglong(int(seed)), _c_d(std),
                                      _c_d(norm_jitter), dtype.encode()))
    return str(folder)


# ------------------------------------------------------------------------------------------------ tokenizer
class Tokenizer:
    """Byte-level BPE read from a Hugging Face tokenizer.json (the library's C++ tokenizer)."""

    def __init__(self, handle, owned: bool = True):
        self._h, self._owned = _c_p(handle), owned

    @classmethod
    def from_file(cls, path: str) -> "Tokenizer":
        h = _lib().vmb_tokenizer_load(str(path).encode())
        if not h:
            _raise()
        return cls(h)

    @classmethod
    def from_dict(cls, root: Dict[str, Any]) -> "Tokenizer":
        h = _lib().vmb_tokenizer_from_json(json.dumps(root).encode())
        if not h:
            _raise()
        return cls(h)

    def __del__(self):
        try:
            if self._owned and self._h:
                _lib().vmb_tokenizer_free(self._h)
        except Exception:
            pass

    def encode(self, text: str) -> List[int]:
        cap = 4 * len(text.encode()) + 16
        out = (ctypes.c_int * cap)()
        n = _ok(_lib().vmb_tokenizer_encode(self._h, text.encode(), out, cap))
        return list(out[:n])

    def decode(self, ids: Sequence[int]) -> str:
        return _text(_lib().vmb_tokenizer_decode(self._h, _ints(ids), len(ids)))

    def _special(self, which: int) -> Optional[int]:
        v = _lib().vmb_tokenizer_special(self._h, which)
        return v if v >= 0 else None

    bos_id = property(lambda self: self._special(0))
    eos_id = property(lambda self: self._special(1))
    pad_id = property(lambda self: self._special(2))
    unk_id = property(lambda self: self._special(3))


def pretokenize(text: str) -> List[str]:
    return json.loads(_text(_lib().vmb_pretokenize(text.encode())))


# ------------------------------------------------------------------------------------------------ model and engine
@dataclass
class Entry:
    """One sequence's share of a step: its slot, its next tokens, and the places among these tokens (0-based) whose
    logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass(frozen=True)
class SamplingParams:
    """Option names and defaults of the reference's command line (examples/smollm2/interactive_main.cpp:23-25,39-41)."""
    temperature: float = 0.7
    top_p: float = 0.9
    max_tokens: int = 32
    seed: int = 42
    stop_tokens: Tuple[int, ...] = ()


@dataclass
class Request:
    prompt: Sequence[int]
    params: SamplingParams = SamplingParams()
    stream: int = 0


@dataclass
class Result:
    """What the reference returns per call (llama_engine.h:32-38), per sequence."""
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""
    prompt_tokens: int = 0
    text: str = ""
    elapsed_seconds: float = 0.0
    tokens_per_second: float = 0.0


@dataclass
class Timing:
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    generated_tokens: int = 0

    @property
    def tokens_per_second(self) -> float:
        total = self.prefill_seconds + self.decode_seconds
        return self.generated_tokens / total if total > 0 else 0.0


class Model:
    """A model with its weights on the device (C++ `DecoderModel`)."""

    def __init__(self, handle):
        self._h = _c_p(handle)
        self.info = json.loads(_text(_lib().vmb_model_info(self._h)))
        self.vocab_size = self.info["vocab_size"]
        self.stop_tokens = tuple(self.info["stop_tokens"])

    def __del__(self):
        try:
            if self._h:
                _lib().vmb_model_free(self._h)
        except Exception:
            pass


def load_model(folder: str, dtype="bfloat16", device: str = "cuda:0") -> Model:
    """Read config.json, choose the architecture by its name, build the parts, load and bind the weights."""
    h = _lib().vmb_model_load(str(folder).encode(), _dtype_name(dtype).encode(), str(device).encode())
    if not h:
        _raise()
    return Model(h)


class _DevicePointer:
    """Device memory as an object torch can wrap without copying."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"data": (int(ptr), False), "shape": tuple(shape), "typestr": typestr, "version": 2}


def _device_tensor(ptr: int, rows: int, cols: int, device):
    import torch
    if rows == 0:
        return torch.empty((0, cols), dtype=torch.float32, device=device)
    return torch.as_tensor(_DevicePointer(ptr, (rows, cols), "<f4"), device=device)


class _CacheView:
    """The cache's bookkeeping as the engine reports it."""

    def __init__(self, engine: "Engine"):
        self._e = engine

    def _stats(self):
        return self._e.stats()["cache"]

    n_pages = property(lambda self: self._stats()["n_pages"])
    max_slots = property(lambda self: self._stats()["max_slots"])
    groups = property(lambda self: self._stats()["groups"])

    @property
    def slots(self):
        held = self._stats()["slots_held"]
        return type("Slots", (), {"held_count": held})

    def tokens_held(self) -> int:
        return self._stats()["tokens_held"]

    def check(self) -> None:
        _ok(_lib().vmb_engine_cache_check(self._e._h))


class _WorkspaceView:
    def __init__(self, engine: "Engine"):
        self._e = engine
        self._fail_after = None

    @property
    def fail_after(self):
        return self._fail_after

    @fail_after.setter
    def fail_after(self, n):
        self._fail_after = n
        _ok(_lib().vmb_engine_set_fail_after(self._e._h, _c_ll(-1 if n is None else int(n))))


class Engine:
    """A model on one GPU with its cache: open/close sequence slots and step batches through the model."""

    MAX_DECODE_RUN = 64

    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None, max_step_tokens: int = 8192,
                 use_graphs: Optional[bool] = None, fused_prefill_rows: Optional[int] = None, poison_freed: bool = False, _borrowed=None):
        self.model = model
        if _borrowed is not None:
            self._h, self._owned = _c_p(_borrowed), False
        else:
            h = _lib().vmb_engine_create(model._h, _c_ll(int(max_tokens)), int(max_slots or 0), int(max_step_tokens),
                                         -1 if use_graphs is None else int(bool(use_graphs)), int(fused_prefill_rows or 0), int(bool(poison_freed)))
            if not h:
                _raise()
            self._h, self._owned = _c_p(h), True
        st = self.stats()
        self.vocab = st["vocab"]
        self.dtype_name = st["dtype"]
        self.use_graphs = st["use_graphs"]
        self.device = "cuda"
        self.cache = _CacheView(self)
        self.ws = _WorkspaceView(self)

    def __del__(self):
        try:
            if self._owned and self._h:
                _lib().vmb_engine_free(self._h)
        except Exception:
            pass

    # ---- slots
    def open(self) -> int:
        return _ok(_lib().vmb_engine_open(self._h))

    def close(self, slot: int) -> None:
        _ok(_lib().vmb_engine_close(self._h, int(slot)))

    def length(self, slot: int) -> int:
        return _ok(_lib().vmb_engine_length(self._h, int(slot)))

    # ---- one step
    def step(self, entries: Sequence[Entry], synchronize: bool = True):
        """Run the entries' tokens as one batch from the cache; float32 logits [wanted, vocab] as a torch CUDA tensor that views
        the engine's own buffer (valid until the next step), in the order of the entries and of each entry's `want`.
        The work runs on the engine's stream; with `synchronize` the call returns when it is done, so that the tensor can be
        used from torch's streams at once."""
        entries = list(entries)
        slots = _ints([e.slot for e in entries])
        n_tok = _ints([len(e.tokens) for e in entries])
        n_want = _ints([len(e.want) for e in entries])
        toks = np.ascontiguousarray(np.concatenate([np.asarray(e.tokens, dtype=np.int64).reshape(-1) for e in entries]) if entries else np.zeros(0))
        if toks.size and (toks.min() < -2**31 or toks.max() >= 2**31):
            raise ValueError("a token id does not fit 32 bits")
        toks = toks.astype(np.int32)
        want = np.ascontiguousarray(np.concatenate([np.asarray(e.want, dtype=np.int32).reshape(-1) for e in entries]) if entries else np.zeros(0),
                                    dtype=np.int32)
        logits, rows = ctypes.c_void_p(), ctypes.c_int()
        _ok(_lib().vmb_engine_step(self._h, len(entries), slots, n_tok, toks.ctypes.data_as(_c_p), n_want, want.ctypes.data_as(_c_p),
                                   ctypes.byref(logits), ctypes.byref(rows)))
        if synchronize:
            self.synchronize()
        return _device_tensor(logits.value or 0, rows.value, self.vocab, self.device)

    def sample(self, logits, params: Sequence[SamplingParams], streams: Sequence[int], steps: Sequence[int]) -> np.ndarray:
        """One token per row of `logits` (a tensor `step` returned): row r uses params[r] and the Philox counter (steps[r], streams[r])."""
        R = int(logits.shape[0])
        out = (ctypes.c_int * max(R, 1))()
        _ok(_lib().vmb_engine_sample(self._h, _c_p(logits.data_ptr()), R, _floats([p.temperature for p in params]), _floats([p.top_p for p in params]),
                                     _ints([p.seed for p in params], ctypes.c_longlong), _ints(streams, ctypes.c_longlong),
                                     _ints(steps, ctypes.c_longlong), out))
        return np.array(out[:R], dtype=np.int32)

    def decode_many(self, slots: Sequence[int], last_tokens: Sequence[int], params: Sequence[SamplingParams], streams: Sequence[int],
                    draw_steps: Sequence[int], k: int) -> np.ndarray:
        """Feed `last_tokens` (one per slot) and decode `k` tokens for every slot without the host in between; int32 [k, B]."""
        B = len(slots)
        out = (ctypes.c_int * max(int(k) * B, 1))()
        _ok(_lib().vmb_engine_decode_many(self._h, B, _ints(slots), _ints(last_tokens), _floats([p.temperature for p in params]),
                                          _floats([p.top_p for p in params]), _ints([p.seed for p in params], ctypes.c_longlong),
                                          _ints(streams, ctypes.c_longlong), _ints(draw_steps, ctypes.c_longlong), int(k), out))
        return np.array(out[: int(k) * B], dtype=np.int32).reshape(int(k), B)

    def generate(self, requests: Sequence[Request], max_batch: int = 64, default_stop: Sequence[int] = (), steps_per_sync: int = 1,
                 on_token: Optional[Callable[[int, int], None]] = None) -> Tuple[List[Result], Timing]:
        """The generation loop over this engine: batches of unequal prompts, stop tokens, early ends, batch after batch."""
        requests = list(requests)
        flat = [int(t) for r in requests for t in r.prompt]
        stops = [int(t) for r in requests for t in r.params.stop_tokens]
        cb_type = ctypes.CFUNCTYPE(None, _c_p, _c_int, _c_int)
        failure = []

        def _cb(user, i, tok):
            try:
                on_token(i, tok)
            except BaseException as ex:       # an exception cannot cross the C frames: keep it and raise it afterwards
                failure.append(ex)

        cb = cb_type(_cb) if on_token is not None else ctypes.cast(None, cb_type)
        text = _lib().vmb_engine_generate(
            self._h, len(requests), _ints([len(r.prompt) for r in requests]), _ints(flat), _floats([r.params.temperature for r in requests]),
            _floats([r.params.top_p for r in requests]), _ints([r.params.max_tokens for r in requests]),
            _ints([r.params.seed for r in requests], ctypes.c_longlong), _ints([r.stream for r in requests], ctypes.c_longlong),
            _ints([len(r.params.stop_tokens) for r in requests]), _ints(stops), len(default_stop), _ints(list(default_stop)), int(max_batch),
            int(steps_per_sync), cb, None)
        if failure:
            raise failure[0]
        data = json.loads(_text(text))
        return [Result(**r) for r in data["results"]], Timing(**data["timing"])

    def synchronize(self) -> None:
        _ok(_lib().vmb_engine_synchronize(self._h))

    @property
    def stream(self):
        """The engine's CUDA stream as a torch stream (to record events on, or to order torch work behind the engine's)."""
        import torch
        return torch.cuda.ExternalStream(int(_lib().vmb_engine_stream(self._h)))

    def raise_if_error(self) -> None:
        """Synchronise and raise if a kernel reported a fault of the step's descriptors (no page, bad id)."""
        _ok(_lib().vmb_engine_raise_if_error(self._h))

    def stats(self) -> Dict[str, Any]:
        return json.loads(_text(_lib().vmb_engine_stats(self._h)))

    @property
    def counters(self) -> Dict[str, int]:
        return self.stats()["counters"]

    @property
    def graphs_captured(self) -> int:
        return self.stats()["counters"]["graphs_recorded"]


class GenerationLoop:
    """The library's generation loop over an engine (kept as a class for symmetry with the C++ API)."""

    def __init__(self, engine: Engine, max_batch: int = 64, default_stop: Sequence[int] = (), steps_per_sync: int = 1):
        self.engine, self.max_batch, self.default_stop, self.steps_per_sync = engine, int(max_batch), tuple(default_stop), int(steps_per_sync)
        self.timing = Timing()

    def run(self, requests: Sequence[Request], on_token: Optional[Callable[[int, int], None]] = None) -> List[Result]:
        results, self.timing = self.engine.generate(requests, self.max_batch, self.default_stop, self.steps_per_sync, on_token)
        return results


# ------------------------------------------------------------------------------------------------ the text engine
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
    """Model + cache + sampler + tokenizer behind one object (the C++ `TextEngine`)."""

    def __init__(self, config: EngineConfig):
        self.config = config
        self._h = None
        self.engine: Optional[Engine] = None
        self.model: Optional[Model] = None
        self.tokenizer: Optional[Tokenizer] = None
        self.last_timing = Timing()

    def load(self) -> "TextEngine":
        c = self.config
        cfg = {"model_path": c.model_path, "tokenizer_path": c.tokenizer_path, "device": c.device, "use_synthetic": bool(c.use_synthetic),
               "seed": int(c.seed), "dtype": _dtype_name(c.dtype), "max_tokens": int(c.max_tokens), "max_batch": int(c.max_batch),
               "use_graphs": -1 if c.use_graphs is None else int(bool(c.use_graphs))}
        if c.model_config is not None:
            cfg["model_config"] = c.model_config
        lib = _lib()
        h = lib.vmb_text_create(json.dumps(cfg).encode())
        if not h:
            _raise()
        self._h = _c_p(h)
        _ok(lib.vmb_text_load(self._h))
        mh = lib.vmb_text_model(self._h)
        if not mh:
            _raise()
        self.model = Model(mh)
        self.engine = Engine(self.model, 0, _borrowed=lib.vmb_text_engine(self._h))
        th = lib.vmb_text_tokenizer(self._h)
        self.tokenizer = Tokenizer(th) if th else None
        return self

    def __del__(self):
        try:
            self.engine = None
            if self._h:
                _lib().vmb_text_free(self._h)
        except Exception:
            pass

    @property
    def is_loaded(self) -> bool:
        return self.engine is not None

    def _need(self):
        if self._h is None or self.engine is None:
            raise RuntimeError("call load() first")
        return self._h

    def encode(self, prompt: Union[str, Sequence[int]]) -> List[int]:
        """Token ids of a prompt.  Text needs a tokenizer and gets the begin-of-sequence token in front if the tokenizer has
        one and the text does not start with it (examples/common/llama/llama_engine.cpp:596-602)."""
        if not isinstance(prompt, str):
            return [int(t) for t in prompt]
        if self.tokenizer is None:
            raise ValueError("a text prompt needs tokenizer.json; pass token ids instead")
        ids = self.tokenizer.encode(prompt)
        bos = self.tokenizer.bos_id
        if bos is not None and (not ids or ids[0] != bos):
            ids = [bos] + ids
        return ids

    def default_stop_tokens(self):
        if self.tokenizer is not None and self.tokenizer.eos_id is not None:
            return (self.tokenizer.eos_id,)
        return tuple(self.model.stop_tokens)

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]], temperature: float = 0.7, top_p: float = 0.9, max_tokens: int = 32,
                 seed: int = 42, stop_tokens: Optional[Sequence[int]] = None, on_token: Optional[Callable[[int, int, str], None]] = None,
                 steps_per_sync: int = 1, sample_fn: Optional[Callable[[Any], int]] = None) -> List[Result]:
        """Generate for a batch of prompts (token id lists, or text if a tokenizer is loaded).
        `on_token(index, token, piece)` is called for every new token; `piece` is its text (or "[id]"); after the last token of a
        sequence whose text ends inside a multi-byte character, the held-back rest comes with token -1.
        `steps_per_sync`: decode steps queued on the GPU before the host reads their tokens (1: every step).
        `sample_fn(logits) -> token`: the reference's way of sampling (llama_engine.h:106-121): a function of one row of float32
        logits (a numpy array on the host) instead of temperature and top-p; every step's logits then come to the host."""
        h = self._need()
        ids = [self.encode(p) for p in prompts]
        options = {"temperature": float(temperature), "top_p": float(top_p), "max_tokens": int(max_tokens), "seed": int(seed),
                   "steps_per_sync": int(steps_per_sync)}
        if stop_tokens is not None:
            options["stop_tokens"] = [int(t) for t in stop_tokens]
        piece_type = ctypes.CFUNCTYPE(None, _c_p, _c_int, _c_int, _c_s)
        sample_type = ctypes.CFUNCTYPE(_c_int, _c_p, ctypes.POINTER(ctypes.c_float), _c_int)
        failure = []

        def _piece(user, i, tok, piece):
            try:
                on_token(i, tok, (piece or b"").decode("utf-8", "replace"))
            except BaseException as ex:
                failure.append(ex)

        def _sample(user, row, vocab):
            try:
                return int(sample_fn(np.ctypeslib.as_array(row, shape=(vocab,)).copy()))
            except BaseException as ex:
                failure.append(ex)
                return -1

        pc = piece_type(_piece) if on_token is not None else ctypes.cast(None, piece_type)
        sc = sample_type(_sample) if sample_fn is not None else ctypes.cast(None, sample_type)
        text = _lib().vmb_text_generate(h, len(ids), _ints([len(p) for p in ids]), _ints([t for p in ids for t in p]),
                                        json.dumps(options).encode(), pc, sc, None)
        if failure:
            raise failure[0]
        data = json.loads(_text(text))
        self.last_timing = Timing(**data["timing"])
        return [Result(**r) for r in data["results"]]

    def describe(self) -> Dict[str, Any]:
        return json.loads(_text(_lib().vmb_text_describe(self._need())))

    # ---- the reference's single-session calls (float32 logits as torch tensors on the host)
    def reset_session(self) -> None:
        _ok(_lib().vmb_text_reset_session(self._need()))

    @property
    def session_length(self) -> int:
        return _ok(_lib().vmb_text_session_length(self._need()))

    def _rows(self, fn, tokens, rows: int):
        import torch
        out = np.empty((rows, self.engine.vocab), dtype=np.float32)
        _ok(fn(self._need(), _ints(tokens), len(tokens), out.ctypes.data_as(_c_p)))
        return torch.from_numpy(out)

    def prefill(self, tokens: Sequence[int]):
        """Start a session with `tokens`; float32 logits [vocab] of the last one (llama_engine.cpp:333-393)."""
        return self._rows(_lib().vmb_text_prefill, list(tokens), 1)[0]

    def forward_step(self, token: int, pos: Optional[int] = None):
        """Feed one more token to the session; logits [vocab] (llama_engine.cpp:395-455).  `pos`, the reference's second argument,
        is the token's place in the session: it can only be the session's length, and is checked when given."""
        import torch
        out = np.empty(self.engine.vocab, dtype=np.float32)
        _ok(_lib().vmb_text_forward_step(self._need(), int(token), _c_ll(-1 if pos is None else int(pos)), out.ctypes.data_as(_c_p)))
        return torch.from_numpy(out)

    def forward_full_logits(self, tokens: Sequence[int]):
        """Stateless: logits [len, vocab] of a whole sequence (llama_engine.cpp:523-585)."""
        return self._rows(_lib().vmb_text_forward_full_logits, list(tokens), len(tokens))

    def forward_logits(self, tokens: Sequence[int]):
        """Stateless: logits [vocab] of the last token (llama_engine.cpp:457-521)."""
        return self._rows(_lib().vmb_text_forward_logits, list(tokens), 1)[0]


def load(model_path: str, dtype: str = "bfloat16", device: str = "cuda:0", max_tokens: int = 65536, max_batch: int = 64) -> TextEngine:
    """Shorthand: a loaded TextEngine for the model folder `model_path`."""
    return TextEngine(EngineConfig(model_path=model_path, dtype=dtype, device=device, max_tokens=max_tokens, max_batch=max_batch)).load()


class OpTimes:
    """Device time per kind of operation while the block runs (two CUDA events around every launch; CUDA graphs are off
    meanwhile): `with OpTimes() as t: ...; print(t.table())`."""

    def __enter__(self):
        h = _lib().vmb_op_times_begin()
        if not h:
            _raise()
        self._h = _c_p(h)
        self._table = ""
        return self

    def table(self) -> str:
        if self._h:
            self._table = _text(_lib().vmb_op_times_table(self._h))
        return self._table

    def __exit__(self, *exc):
        self.table()
        _lib().vmb_op_times_end(self._h)
        self._h = None
        return False


__all__ = ["ConfigError", "WeightError", "CacheError", "KernelError", "KernelLibraryError", "Entry", "SamplingParams", "Request", "Result",
           "Timing", "Model", "Engine", "GenerationLoop", "EngineConfig", "TextEngine", "Tokenizer", "OpTimes", "load", "load_model",
           "write_random_model", "weight_table", "describe_config", "check_model_folder", "check_safetensors_header", "safetensors_info", "registered_architectures", "smollm2_135m_config",
           "pretokenize"]
