"""A minimal safetensors writer for the tests (numpy only): names sorted, header padded to 8 bytes."""
import json
import struct

import numpy as np

_NAMES = {np.dtype("float32"): "F32", np.dtype("float16"): "F16", np.dtype("int64"): "I64", np.dtype("int32"): "I32", np.dtype("uint8"): "U8"}


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def write(path, tensors, bf16=()):
    """`tensors`: name -> numpy array; names in `bf16` are float32 arrays stored as BF16."""
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        a = np.asarray(tensors[name])
        shape = list(a.shape)                       # (ascontiguousarray would make a scalar one-dimensional)
        a = np.ascontiguousarray(a)
        if name in bf16:
            raw, dt = to_bf16_bits(a).tobytes(), "BF16"
        else:
            raw, dt = a.tobytes(), _NAMES[a.dtype]
        header[name] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    blob = json.dumps(header).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + b"".join(blobs))
