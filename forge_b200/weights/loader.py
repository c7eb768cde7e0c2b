"""Loads a model's tensors from safetensors by name.

The model says which tensors it expects (name, shape, whether it may be absent); the loader checks the
whole file against that list first and raises ONE error that lists every missing tensor, every
unexpected tensor and every wrong shape or dtype, instead of the reference's silent skipping of absent
names and first-forward shape failures (src/model/model.cpp:220-232, src/operators/cpu/matmul.cpp:1142-1146).
The table of names is the Hugging Face column of the reference's mapping (tools/name_mapping.py:9-26,
src/model/weight_mapper.cpp:11-29); each part owns the names of its own tensors.
"""
from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from .safetensors_io import SafetensorsError, open_model_files

FLOAT_DTYPES = (torch.bfloat16, torch.float16, torch.float32)


class WeightError(ValueError):
    """The model folder's tensors do not match what the model needs."""

    def __init__(self, where, missing=(), unexpected=(), wrong=()):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = [f"{where}: tensors do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}): " + "; ".join(self.wrong))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    required: bool = True
    integer: bool = False        # an integer table (kept int32) rather than floating-point weights
    role: str = "matrix"         # "matrix" | "embedding" | "norm" | "bias": how random weights are drawn for it


def check_tensors(where, expected: Dict[str, TensorSpec], present: Dict[str, Tuple[Tuple[int, ...], torch.dtype]]):
    missing = [n for n, s in expected.items() if s.required and n not in present]
    unexpected = [n for n in present if n not in expected]
    wrong = []
    for n, s in expected.items():
        if n not in present:
            continue
        shape, dt = present[n]
        if tuple(shape) != tuple(s.shape):
            wrong.append(f"{n}: file has {list(shape)}, model needs {list(s.shape)}")
        elif s.integer and dt not in (torch.int32, torch.int64):
            wrong.append(f"{n}: file has {dt}, model needs an integer table")
        elif not s.integer and dt not in FLOAT_DTYPES:
            wrong.append(f"{n}: file has {dt}, model needs bfloat16, float16 or float32")
    if missing or unexpected or wrong:
        raise WeightError(where, missing, unexpected, wrong)


def load_tensors(model_dir, expected: Dict[str, TensorSpec]):
    """{name: CPU tensor as stored} for every expected tensor present in the folder; raises WeightError /
    SafetensorsError.  float16 is widened to float32 (the kernels take bfloat16 and float32); int64 tables
    become int32."""
    files, opened = open_model_files(model_dir)
    try:
        present = {n: (f.shape(n), f.dtype(n)) for n, f in files.items()}
        check_tensors(model_dir, expected, present)
        out = {}
        for n in expected:
            if n not in files:
                continue
            t = files[n].tensor(n)
            if t.dtype == torch.float16:
                t = t.to(torch.float32)
            elif t.dtype == torch.int64:
                t = t.to(torch.int32)
            out[n] = t
        return out
    finally:
        for f in opened:
            f.close()


__all__ = ["WeightError", "TensorSpec", "SafetensorsError", "check_tensors", "load_tensors"]
