"""Zero-dependency reader and writer for the safetensors container.

File layout: 8 bytes little-endian header length N, N bytes of JSON
(`name -> {"dtype", "shape", "data_offsets": [begin, end]}` plus an optional
`__metadata__` object), then the raw tensor bytes.  The checks follow the
reference's reader (src/safetensors.cpp:253-377, 412-452, 508-546): header
length bounds, duplicate keys, known dtype, shape x dtype == byte span,
spans inside the file and not overlapping.

Tensors come back as torch tensors that keep the STORED dtype (BF16 stays
bfloat16, F32 stays float32, integer types become int32); nothing is cast
here.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024  # src/safetensors.cpp:22-23 keeps a header limit too

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorEntry:
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate key {k!r} in safetensors header")
        out[k] = v
    return out


def parse_header(blob: bytes, data_bytes: int) -> Dict[str, TensorEntry]:
    """Validate the JSON header against `data_bytes` bytes of payload."""
    try:
        root = json.loads(blob.decode("utf-8"), object_pairs_hook=_no_duplicates)
    except SafetensorsError:
        raise
    except (UnicodeDecodeError, json.JSONDecodeError, RecursionError) as e:
        raise SafetensorsError(f"malformed safetensors header: {e}") from None
    if not isinstance(root, dict):
        raise SafetensorsError("safetensors header is not a JSON object")
    entries: Dict[str, TensorEntry] = {}
    for name, desc in root.items():
        if name == "__metadata__":
            continue
        if not isinstance(desc, dict):
            raise SafetensorsError(f"tensor {name!r}: entry is not an object")
        dt = desc.get("dtype")
        if dt not in _DTYPES:
            raise SafetensorsError(f"tensor {name!r}: unsupported dtype {dt!r}")
        shape = desc.get("shape")
        if not isinstance(shape, list) or any((not isinstance(d, int)) or isinstance(d, bool) or d < 0 for d in shape):
            raise SafetensorsError(f"tensor {name!r}: bad shape {shape!r}")
        offs = desc.get("data_offsets")
        if (not isinstance(offs, list) or len(offs) != 2
                or any((not isinstance(o, int)) or isinstance(o, bool) or o < 0 for o in offs)):
            raise SafetensorsError(f"tensor {name!r}: bad data_offsets {offs!r}")
        begin, end = offs
        numel = 1
        for d in shape:
            numel *= d
        want = numel * _DTYPES[dt][1]
        if end < begin or end - begin != want:
            raise SafetensorsError(
                f"tensor {name!r}: shape {shape} of {dt} needs {want} bytes, data_offsets span {end - begin}")
        if end > data_bytes:
            raise SafetensorsError(
                f"tensor {name!r}: data_offsets end {end} beyond the payload ({data_bytes} bytes): truncated file?")
        entries[name] = TensorEntry(dt, tuple(shape), begin, end)
    spans = sorted((e.begin, e.end, n) for n, e in entries.items() if e.end > e.begin)
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise SafetensorsError(f"tensors {n0!r} and {n1!r} overlap in the payload")
    return entries


def read_header(path: str) -> Tuple[Dict[str, TensorEntry], int]:
    """Return (entries, payload offset) of the file at `path`."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte length prefix")
        (n,) = struct.unpack("<Q", head)
        if n == 0 or n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} is not plausible for a file of {size} bytes")
        blob = f.read(n)
        if len(blob) != n:
            raise SafetensorsError(f"{path}: truncated header")
    return parse_header(blob, size - 8 - n), 8 + n


def load_file(path: str) -> Dict[str, torch.Tensor]:
    """Read every tensor of `path` into host memory, dtype as stored (ints -> int32)."""
    entries, base = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        size = os.path.getsize(path)
        mm = mmap.mmap(f.fileno(), size, access=mmap.ACCESS_READ) if size else None
        try:
            for name, e in entries.items():
                tdt, _ = _DTYPES[e.dtype]
                nbytes = e.end - e.begin
                if nbytes == 0:
                    t = torch.empty(e.shape, dtype=tdt)
                else:
                    raw = bytearray(mm[base + e.begin: base + e.end])  # own the bytes; the map is closed below
                    t = torch.frombuffer(raw, dtype=tdt).reshape(e.shape)
                if tdt in (torch.int64, torch.int16, torch.int8, torch.uint8):
                    t = t.to(torch.int32)
                out[name] = t
        finally:
            if mm is not None:
                mm.close()
    return out


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] | None = None) -> None:
    """Write `tensors` (host or device, any supported dtype) to `path`, names sorted, 8-byte aligned header."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    off = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
