"""Sampling in the reference's manner: greedy, or temperature softmax with optional top-k, top-p and
repeat penalty, driven by a xorshift64 generator (include/forge/sampler.h:12-19,
src/inference/sampler.cpp:22-55, 197-351).  The arithmetic over the vocabulary runs in CUDA kernels
(`forge_b200.kernels.argmax / sample / repeat_penalty`); the per-request state (generator, history of
generated tokens) lives here on the host, one per request, so a request's tokens do not depend on what
else is in the batch (the reference's scheduler shares one Sampler among all requests,
src/inference/request_scheduler.cpp:319-322).
"""
from collections import Counter
from dataclasses import dataclass

import torch

from .. import kernels

_MASK64 = (1 << 64) - 1


@dataclass
class SamplerConfig:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repeat_penalty: float = 1.0
    do_sample: bool = True
    seed: int = 0

    @property
    def greedy(self):
        return (not self.do_sample) or self.temperature <= 0.0


class XorShift64:
    """x ^= x<<13; x ^= x>>7; x ^= x<<17; u = (x & 0x7FFFFFFF) / 0x7FFFFFFF  (sampler.cpp:35-44).
    Seed 0 means state 12345 (sampler.cpp:22-24)."""

    def __init__(self, seed=0):
        self.state = (int(seed) & _MASK64) or 12345

    def next_u64(self):
        x = self.state
        x ^= (x << 13) & _MASK64
        x ^= x >> 7
        x ^= (x << 17) & _MASK64
        self.state = x
        return x

    def uniform(self):
        return float(self.next_u64() & 0x7FFFFFFF) / float(0x7FFFFFFF)


class RequestSampler:
    """Sampling state of one request."""

    def __init__(self, config: SamplerConfig):
        self.config = config
        self.rng = XorShift64(config.seed)
        self.history = Counter()

    def record(self, token):
        self.history[int(token)] += 1


def sample_batch(logits, samplers):
    """logits: fp32 [R,V] on the device, one row per sampler (modified in place by repeat penalties).
    Returns a list of R token ids and records each in its sampler's history."""
    R = logits.shape[0]
    if R != len(samplers):
        raise ValueError(f"{R} rows of logits for {len(samplers)} requests")
    dev = logits.device
    if any(s.config.repeat_penalty != 1.0 and s.history for s in samplers):
        toks, counts, offsets, pen = [], [], [0], []
        for s in samplers:
            if s.config.repeat_penalty != 1.0:
                for t, c in s.history.items():
                    toks.append(t)
                    counts.append(c)
            offsets.append(len(toks))
            pen.append(float(s.config.repeat_penalty))
        kernels.repeat_penalty(logits, torch.tensor(toks or [0], dtype=torch.int32, device=dev),
                               torch.tensor(counts or [0], dtype=torch.int32, device=dev),
                               torch.tensor(offsets, dtype=torch.int32, device=dev),
                               torch.tensor(pen, dtype=torch.float32, device=dev))
    greedy = [s.config.greedy for s in samplers]
    if all(greedy):
        out = kernels.argmax(logits).tolist()
    else:
        # rows that sample get their own temperature / k / p / u; greedy rows ride along as top_k = 1
        temp = [1.0 if g else float(s.config.temperature) for g, s in zip(greedy, samplers)]
        top_k = [1 if g else int(s.config.top_k) for g, s in zip(greedy, samplers)]
        top_p = [1.0 if g else float(s.config.top_p) for g, s in zip(greedy, samplers)]
        u = [0.5 if g else s.rng.uniform() for g, s in zip(greedy, samplers)]
        params = torch.tensor([temp, top_p, u], dtype=torch.float32).to(dev)
        drawn = kernels.sample(logits, params[0].contiguous(), torch.tensor(top_k, dtype=torch.int32, device=dev),
                               params[1].contiguous(), params[2].contiguous())
        out = drawn.tolist()
        if any(greedy):
            am = kernels.argmax(logits).tolist()     # exact tie rule (lowest index) for greedy rows
            out = [a if g else o for g, a, o in zip(greedy, am, out)]
    for s, t in zip(samplers, out):
        s.record(t)
    return out
