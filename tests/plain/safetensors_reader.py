"""A minimal safetensors reader for the test oracle (numpy only).

Format: 8-byte little-endian header length N, N bytes of JSON mapping tensor
name -> {dtype, shape, data_offsets:[begin,end)} relative to the byte after the
header, then the raw little-endian tensor bytes.
"""
import json
import struct

import numpy as np


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path):
    """Returns {name: float32/float64/int ndarray}; bf16/f16 are widened to f32."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    base = 8 + n
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        buf = blob[base + b:base + e]
        shape = tuple(info["shape"])
        dt = info["dtype"]
        if dt == "BF16":
            arr = _bf16_to_f32(np.frombuffer(buf, dtype="<u2"))
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(np.float32)
        elif dt == "F32":
            arr = np.frombuffer(buf, dtype="<f4")
        elif dt == "F64":
            arr = np.frombuffer(buf, dtype="<f8")
        elif dt == "I32":
            arr = np.frombuffer(buf, dtype="<i4")
        elif dt == "I64":
            arr = np.frombuffer(buf, dtype="<i8")
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name} not handled")
        out[name] = arr.reshape(shape).copy()
    return out
