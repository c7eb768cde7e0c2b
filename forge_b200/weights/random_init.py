"""Random-weights mode: from a configuration and a seed to a model folder (config.json + model.safetensors)
that loads like any other.  Matrices and biases are N(0, std) (0.02 as in the reference's
tools/create_test_model.py:14-63, which however also draws the norm weights from it; here norm weights are
1, or 1 + N(0, norm_std) when asked).  Matrices are stored in bfloat16, norm weights in float32.
"""
import json
import os

import torch

from .safetensors_io import write_safetensors


def random_tensors(config, seed=0, std=0.02, embed_std=None, norm_std=0.0, bias_std=None, dtype=torch.bfloat16,
                   device="cpu"):
    """{file tensor name: tensor} for every tensor the configuration's model expects, in file order."""
    from ..engine.model import Model
    from ..parts import Runtime
    model = Model(config.plan(), Runtime(torch.device("cpu"), dtype))
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for name, spec in model.tensor_specs().items():
        if not spec.required:
            continue
        if spec.integer:
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.role == "norm":
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
            if norm_std:
                t += torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * norm_std
            out[name] = t
        else:
            s = std
            if spec.role == "bias" and bias_std is not None:
                s = bias_std
            if spec.role == "embedding" and embed_std is not None:
                s = embed_std
            out[name] = (torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * s).to(dtype)
    return out


def write_random_model(config, out_dir, seed=0, **kwargs):
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns out_dir."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(config, seed=seed, **kwargs),
                      metadata={"format": "pt", "seed": seed})
    return out_dir
