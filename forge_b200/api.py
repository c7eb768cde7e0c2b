"""The Python entry point, in the reference's manner (src/bindings/model.cpp:82-120, README.md:64-72):

    import forge_b200 as forge
    model = forge.Model("path/to/model_dir", device="cuda", dtype="bfloat16")
    out = model.generate(prompt_ids, max_new_tokens=64, temperature=0.8, seed=1)
    out["token_ids"], out["finish_reason"]          # "eos" | "stop" | "length"

    ctx = model.create_context(); logits = ctx.forward(ids, start_pos=0)   # np.float32 [T, V]
    sched = forge.RequestScheduler(model, block_size=16, max_num_seqs=4)   # submit / step / get_finished

Option names and defaults are the reference's (generate: src/bindings/model.cpp:103-108; SamplerConfig:
include/forge/sampler.h:12-19).  Options of the reference that select what this engine does not have
(kv_cache_dtype, gpu_layers) are accepted only at their defaults.
"""
import numpy as np
import torch

from .config import registered_architectures
from .engine.runner import ModelRunner, StepEntry
from .engine.scheduler import GenerateRequest, RequestScheduler as _Scheduler, RequestStatus
from .sampling import SamplerConfig


def _ids(prompt_ids):
    if isinstance(prompt_ids, torch.Tensor):
        prompt_ids = prompt_ids.detach().cpu().numpy()
    arr = np.asarray(prompt_ids)
    if arr.ndim != 1:
        raise ValueError("prompt_ids must be 1D")
    return [int(t) for t in arr.tolist()]


class Model:
    def __init__(self, path=None, device="cuda", dtype="bfloat16", *, config=None, tensors=None, block_size=64,
                 max_num_seqs=4, cache_tokens=None, max_tokens_per_step=2048, memory_fraction=0.6):
        """path: model folder (config.json + model.safetensors[.index.json]); or ``config`` + ``tensors``.
        ``block_size``: tokens per cache page.  64 (the default) is what the prompt attention is fastest with (a key
        tile of 64 is then one TMA box; 43 us a layer at 2,048 tokens against 54 us with pages of 16) and what the
        benchmark uses; 8, 16 and 32 give the same results with finer-grained memory."""
        dev = "cuda:0" if device in ("cuda", "gpu") else device
        if not str(dev).startswith("cuda"):
            raise ValueError(f"forge_b200 runs on CUDA devices only, not {device!r}")
        self.runner = ModelRunner(path, config=config, tensors=tensors, dtype=dtype, device=dev, page_size=block_size,
                                  cache_tokens=cache_tokens, max_requests=max_num_seqs, memory_fraction=memory_fraction)
        self.max_tokens_per_step = max_tokens_per_step
        self._busy = False

    @property
    def config(self):
        return self.runner.config

    @property
    def device(self):
        return str(self.runner.device)

    @staticmethod
    def registered_archs():
        return registered_architectures()

    def _scheduler(self, max_num_seqs=None):
        if self.runner.manager.live_requests():
            raise RuntimeError("the model's cache is in use by another scheduler or context; reset it first")
        return _Scheduler(self.runner, max_num_seqs or self.runner.max_requests, self.max_tokens_per_step)

    def generate(self, prompt_ids, max_new_tokens=256, temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                 do_sample=True, seed=0, eos_token_id=-1, kv_cache_dtype=None, gpu_layers=-1, stop_token_ids=(),
                 callback=None):
        """Generates up to max_new_tokens tokens (the one sampled from the prompt counts, as in
        src/inference/generator.cpp:135).  Returns the reference's dict: token_ids (generated only),
        num_prompt_tokens, num_generated_tokens, finished, finish_reason."""
        if kv_cache_dtype not in (None, "fp32", "bf16", "bfloat16", "float32") or gpu_layers not in (-1, None):
            raise ValueError("quantized caches and CPU offload are not part of this engine")
        prompt = _ids(prompt_ids)
        sched = self._scheduler(1)
        cb = (lambda rid, tok, step, status: callback(tok, step)) if callback else None
        sched.submit(prompt, max_new_tokens, eos_token_id,
                     SamplerConfig(temperature, top_k, top_p, repeat_penalty, do_sample, seed), cb, stop_token_ids)
        (req,) = sched.run()
        if req.status == RequestStatus.Failed:
            raise RuntimeError(f"generation failed: {req.finish_reason}")
        return {"token_ids": list(req.output_tokens), "num_prompt_tokens": len(prompt),
                "num_generated_tokens": req.num_generated, "finished": True, "finish_reason": req.finish_reason}

    def generate_stream(self, prompt_ids, callback, **kwargs):
        """callback(token_id, step) per generated token (src/bindings/model.cpp:42-80)."""
        self.generate(prompt_ids, callback=callback, **kwargs)

    def create_context(self, kv_cache_dtype=None, gpu_layers=-1):
        return InferenceContext(self)


class InferenceContext:
    """Single-sequence forward from Python: ``forward(ids, start_pos)`` appends ids at start_pos (which must
    be where the sequence ends) and returns all their logits (src/bindings/common.h:147-170)."""
    _ID = "__context__"

    def __init__(self, model):
        self.model, self.runner = model, model.runner
        if self.runner.is_live(self._ID):
            self.runner.release(self._ID)

    def forward(self, input_ids, start_pos=0):
        ids = _ids(input_ids)
        if not self.runner.is_live(self._ID):
            self.runner.admit(self._ID)
        have = self.runner.manager.num_tokens(self._ID)
        if start_pos == 0 and have:
            self.reset_kv()
            self.runner.admit(self._ID)
            have = 0
        if start_pos != have:
            raise ValueError(f"start_pos {start_pos} does not continue the sequence ({have} tokens cached)")
        logits = self.runner.step([StepEntry(self._ID, ids, list(range(len(ids))))])
        out = logits.cpu().numpy()
        self.runner.check_status()
        return out

    def reset_kv(self):
        if self.runner.is_live(self._ID):
            self.runner.release(self._ID)

    reset = reset_kv

    @property
    def device(self):
        return self.model.device


class RequestScheduler(_Scheduler):
    """forge.RequestScheduler(model, block_size=16, max_num_seqs=4): block_size is the model's page size and
    is fixed when the model is made (the reference ignores the argument too,
    src/inference/request_scheduler.cpp:126-128)."""

    def __init__(self, model, block_size=16, max_num_seqs=4, max_tokens_per_step=None):
        if model.runner.manager.live_requests():
            raise RuntimeError("the model's cache is in use; reset the other scheduler or context first")
        super().__init__(model.runner, max_num_seqs, max_tokens_per_step or model.max_tokens_per_step)


__all__ = ["Model", "InferenceContext", "RequestScheduler", "SamplerConfig", "GenerateRequest", "RequestStatus"]
