#!/usr/bin/env python3
"""Serving benchmark of forge_b200 on one B200: decode tokens/s of the TinyLlama-1.1B-shaped LLaMA decoder
(random bf16 weights, uniform-random prompts) at batch 8, plus batch 1 and 64, a 2,048-token prefill and
the decode step's HBM roofline.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step (one new token for every request of the batch).  `value` is timed on the
device with CUDA events around exactly K steps whose input tokens are the previous step's argmax, fed back
on the device; `e2e` runs the same decoding through the Python entry point (RequestScheduler.submit/step):
every step copies that step's integers from pinned host memory to the device and reads sampled tokens back
to the host (the scheduler launches step k before it reads step k-1's tokens, so the read of every step's
result happens one step late and off the device's critical path).  Weights (2.07 GB) exceed the 126 MB L2, so every step streams them from HBM.
The cache has pages of 64 tokens (--block-size; `config` names it): the prompt attention moves one TMA box per page,
and a key tile of 64 is then one box.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# sizes of BASELINE.json configs[2] (TinyLlama-1.1B shape)
SHAPE = dict(architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=2048, intermediate_size=5632,
             num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64, rope_theta=10000.0,
             rms_norm_eps=1e-5, attention_bias=False, tie_word_embeddings=False, max_position_embeddings=2048)
PROMPT_LEN, CONTEXT, PREFILL_TOKENS = 512, 2048, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def stop(self):
        if self.proc:
            self.proc.terminate()
        s = self.samples
        if not s:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[2 + i].lower() == "active" for r in s)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in s), "sm_max_mhz": int(s[0][1]), "reasons": reasons,
                "samples": len(s)}


REF_DIR = os.environ.get("FORGE_REFERENCE_BUILD", os.path.join(ROOT, "baseline", "_ref", "cuda"))
REF_SOURCE = os.environ.get("FORGE_REFERENCE_SOURCE", "/root/reference")


def reference_arm(a):
    """The UNMODIFIED reference on its CUDA backend, through its own engine API (baseline/ref_bench.cpp says how it
    is driven, baseline/build_reference.py how it is built: by hand, because its pip/CMake build needs the
    network).  The reference computes in FP32 and serves one sequence at a time on the GPU, so its line is batch 1 in
    fp32 at the same layer sizes, prompt length and prefill length; `config.same_config` says so."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
        return 0
    if a.gpus != 1:
        return unavailable("the reference's engine runs on one GPU; asked for %d" % a.gpus)
    exe = os.path.join(REF_DIR, "ref_bench")
    if not os.path.exists(exe):
        if not os.path.isdir(REF_SOURCE):
            return unavailable(f"baseline/_ref/cuda/ref_bench is not built and the reference's sources are not at {REF_SOURCE}")
        b = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), "--reference", REF_SOURCE],
                           capture_output=True, text=True)
        if b.returncode != 0 or not os.path.exists(exe):
            return unavailable("building the reference's CUDA backend by hand failed: " + (b.stdout + b.stderr)[-300:])
    s = SHAPE
    steps, warmup = a.steps, max(a.warmup, 3)
    args = [s["num_hidden_layers"], s["hidden_size"], s["num_attention_heads"], s["num_key_value_heads"], s["head_dim"],
            s["intermediate_size"], s["vocab_size"], s["rope_theta"], s["rms_norm_eps"], CONTEXT, PROMPT_LEN,
            PREFILL_TOKENS, steps, warmup]
    clocks = ClockSampler()
    clocks.start()
    try:
        r = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=1500)
    except subprocess.TimeoutExpired:
        clocks.stop()
        return unavailable("the reference's ref_bench did not finish within 1500 s")
    clk = clocks.stop()
    line = next((l for l in reversed(r.stdout.splitlines()) if l.startswith("{")), None)
    if r.returncode != 0 or line is None:
        return unavailable(f"the reference's ref_bench exited with {r.returncode}: " + (r.stderr or r.stdout)[-300:])
    m = json.loads(line)
    ms, e2e_ms = m["decode_ms_per_step"], m["e2e_ms_per_step"]
    L, H, I, V = s["num_hidden_layers"], s["hidden_size"], s["intermediate_size"], s["vocab_size"]
    qkv = (s["num_attention_heads"] + 2 * s["num_key_value_heads"]) * s["head_dim"]
    T = PREFILL_TOKENS
    flops = 2 * T * L * (qkv * H + H * s["num_attention_heads"] * s["head_dim"] + 3 * I * H) \
        + L * 2 * T * T * s["head_dim"] * s["num_attention_heads"] + 2 * T * V * H      # its head runs on all T rows
    print(json.dumps({
        "metric": "decode tok/s at batch 8; also batch 1/64 and prefill tok/s at 2,048 tokens (TinyLlama-1.1B shape)",
        "value": round(1e3 / ms, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic: random-init fp32 weights ~N(0,0.02), random token ids",
        "impl": "reference",
        "config": {"model": "TinyLlama-1.1B shape (arch llama, GenericEngine)", "layers": L, "layers_full": L, "hidden": H,
                   "heads": s["num_attention_heads"], "kv_heads": s["num_key_value_heads"], "head_dim": s["head_dim"],
                   "intermediate": I, "vocab": V, "global_batch": 1, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT,
                   "parallelism": "1 GPU", "same_config": False,
                   "why": "the reference has no bf16 path (fp32 weights and cache) and decodes one sequence at a time on "
                          "the GPU: its batched path copies device memory with host memcpy "
                          "(transformer_engine.cpp:236-240) and is not run; compare with points.decode_b1",
                   "build": "by hand from unmodified sources, nvcc sm_100, cuBLAS on (baseline/build_reference.py)"},
        "clocks": clk,
        "e2e": {"value": round(1e3 / e2e_ms, 1), "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "points": {"decode_b1": round(1e3 / ms, 1)},
        "prefill": {"value": round(T / m["prefill_ms"] * 1e3, 1), "tokens": T, "ms": round(m["prefill_ms"], 3), "flops": flops},
    }))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="forge_b200", choices=["forge_b200", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SHAPE["num_hidden_layers"], help="fewer layers (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and the prefill")
    ap.add_argument("--block-size", type=int, default=64, help="tokens per cache page (named in config)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(json.dumps({"error": "forge_b200 is a single-GPU engine: bench.py runs at --gpus 1 only", "n_gpus": a.gpus}))
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    import forge_b200 as forge
    from forge_b200 import kernels
    from forge_b200.config import config_from_dict
    from forge_b200.engine import StepEntry
    from forge_b200.weights import random_tensors

    shape = dict(SHAPE, num_hidden_layers=a.layers)
    cfg = config_from_dict(shape)
    torch.cuda.set_device(0)
    tensors = random_tensors(cfg, seed=0, std=0.02, device="cuda")
    max_b = 64 if not a.no_points else a.batch
    total_steps = a.steps + a.warmup + 2
    per_request = -(-(PROMPT_LEN + total_steps + 16) // a.block_size) * a.block_size      # a request holds whole pages
    cache_tokens = max(max_b * per_request, PREFILL_TOKENS + a.block_size)
    model = forge.Model(config=cfg, tensors=tensors, dtype="bfloat16", max_num_seqs=max_b, cache_tokens=cache_tokens,
                        max_tokens_per_step=2048, block_size=a.block_size)
    del tensors
    runner = model.runner
    V = cfg.vocab_size
    gen = torch.Generator().manual_seed(0)
    pk = peaks()

    def prompts(B):
        return [torch.randint(0, V, (PROMPT_LEN,), generator=gen).tolist() for _ in range(B)]

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    def decode_device(B, steps, warmup):
        """Device-timed decode: argmax of step i is the input of step i+1 without leaving the device."""
        ids = [f"d{B}_{i}" for i in range(B)]
        ps = prompts(B)
        for rid in ids:
            runner.admit(rid)
        per_step = max(1, 2048 // PROMPT_LEN)
        for i in range(0, B, per_step):
            runner.step([StepEntry(ids[j], ps[j], []) for j in range(i, min(B, i + per_step))])
        dummy = [StepEntry(rid, [0], [0]) for rid in ids]
        graph_first = [StepEntry(rid, [p[-1]], [0]) for rid, p in zip(ids, ps)]   # any token starts the chain
        runner.decode_step(graph_first)

        def one():
            runner.decode_step(dummy, tokens_on_device=True)
        for _ in range(warmup):
            one()
        n0 = kernels.launch_count()
        ms = timed(one, steps)
        launches = kernels.launch_count() - n0
        ctx = PROMPT_LEN + 1 + warmup + steps // 2
        for rid in ids:
            runner.release(rid)
        return B * steps / ms * 1e3, ms / steps, launches, ctx

    def decode_e2e(B, steps, warmup):
        sched = forge.RequestScheduler(model, max_num_seqs=B)
        greedy = forge.SamplerConfig(do_sample=False)
        for p in prompts(B):
            sched.submit(p, max_new_tokens=steps + warmup + 8, sampler_config=greedy)
        while any(r.status.name != "Decoding" for r in sched.get_all_requests()):
            sched.step()
        for _ in range(warmup):
            sched.step()
        ms = timed(sched.step, steps)
        g = next(v for (s_, _), v in runner._decode_graphs.items() if s_ == B)
        sched.reset()
        return B * steps / ms * 1e3, g.host.numel() * 4, B * 4

    clocks = ClockSampler()
    clocks.start()
    value, ms_per_step, launches, ctx = decode_device(a.batch, a.steps, a.warmup)
    clk = clocks.stop()
    e2e_value, h2d, d2h = decode_e2e(a.batch, a.steps, a.warmup)

    # bytes one decode step must read: every matrix once, norms, the embedding rows, and the live cache
    L, H, I = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    w_bytes = 2 * (L * (qkv * H + H * cfg.num_attention_heads * cfg.head_dim + 3 * I * H) + V * H) + 4 * H * (2 * L + 1)
    kv_per_token = 2 * cfg.num_key_value_heads * cfg.head_dim * 2 * L
    step_bytes = w_bytes + a.batch * (ctx * kv_per_token + H * 2)
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8; also batch 1/64 and prefill tok/s at 2,048 tokens (TinyLlama-1.1B shape)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init bf16 weights N(0,0.02), uniform-random token ids",
        "impl": "forge_b200",
        "config": {"model": "TinyLlama-1.1B shape (LlamaForCausalLM)", "layers": L, "layers_full": SHAPE["num_hidden_layers"],
                   "hidden": H, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": I, "vocab": V, "global_batch": a.batch,
                   "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "page_size": runner.page_size,
                   "parallelism": "1 GPU", "cuda_graph": True,
                   "l2": "inputs larger than L2: 2.07 GB of weights streamed per step vs 126 MB L2"},
        "clocks": clk,
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"], "bytes_per_step": step_bytes},
    }
    if not a.no_points:
        points = {}
        for B in (1, 64):
            v, _, _, _ = decode_device(B, a.steps, a.warmup)
            points[f"decode_b{B}"] = round(v, 1)
        points[f"decode_b{a.batch}"] = round(value, 1)
        out["points"] = points
        # prefill of 2,048 tokens, one request, one step; logits at the last position only
        toks = torch.randint(0, V, (PREFILL_TOKENS,), generator=gen).tolist()

        def prefill():
            runner.admit("p")
            runner.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
            runner.release("p")
        for _ in range(3):
            prefill()
        reps = 5
        ms = timed(prefill, reps) / reps
        T = PREFILL_TOKENS
        flops = 2 * T * L * (qkv * H + H * cfg.num_attention_heads * cfg.head_dim + 3 * I * H) \
            + L * 2 * T * T * cfg.head_dim * cfg.num_attention_heads + 2 * V * H
        out["prefill"] = {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                          "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "peaks": pk["source"],
                          "flops": flops}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
