#!/usr/bin/env python3
"""Serving benchmark of forge_b200 on one B200: decode tokens/s of the TinyLlama-1.1B-shaped LLaMA decoder
(random bf16 weights, uniform-random prompts) at batch 8, plus batch 1 and 64, a 2,048-token prefill and
the decode step's HBM roofline.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Further speed points (`points`): the decode step without the CUDA graph, and two more sizes of the same architecture
with random weights, the Llama-3-8B shape (decode at batch 1/8/64 after 1,024-token prompts, a 1,024-token prefill) and
the Qwen2.5-7B shape (64 requests with prompts of 128 to 8,192 tokens served with at most 2,048 tokens a step).

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
    ap.add_argument("--no-shapes", action="store_true", help="skip the Llama-3-8B and Qwen2.5-7B shaped points")
    ap.add_argument("--block-size", type=int, default=64, help="tokens per cache page (named in config)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(json.dumps({"error": "forge_b200 is a single-GPU engine: bench.py runs at --gpus 1 only", "n_gpus": a.gpus}))
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    torch.cuda.set_device(0)
    pk = peaks()
    shape = dict(SHAPE, num_hidden_layers=a.layers)
    max_b = 64 if not a.no_points else a.batch
    bench = ShapeBench(shape, PROMPT_LEN, max_b, a.steps, a.warmup, a.block_size, prefill_tokens=PREFILL_TOKENS)
    cfg = bench.cfg

    clocks = ClockSampler()
    clocks.start()
    value, ms_per_step, launches, ctx = bench.decode_device(a.batch)
    clk = clocks.stop()
    e2e_value, h2d, d2h = bench.decode_e2e(a.batch)
    step_bytes = bench.decode_bytes(a.batch, ctx)
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    L, H, I, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    out = {
        "metric": "decode tok/s at batch 8; also batch 1/64 and prefill tok/s at 2,048 tokens (TinyLlama-1.1B shape)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init bf16 weights N(0,0.02), uniform-random token ids",
        "impl": "forge_b200",
        "config": {"model": "TinyLlama-1.1B shape (LlamaForCausalLM)", "layers": L, "layers_full": SHAPE["num_hidden_layers"],
                   "hidden": H, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": I, "vocab": V, "global_batch": a.batch,
                   "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "page_size": bench.runner.page_size,
                   "parallelism": "1 GPU", "cuda_graph": True,
                   "l2": "inputs larger than L2: 2.07 GB of weights streamed per step vs 126 MB L2"},
        "clocks": clk,
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"], "bytes_per_step": step_bytes},
    }
    if not a.no_points:
        points = {f"decode_b{a.batch}": round(value, 1)}
        for B in (1, 64):
            v, ms, _, c = bench.decode_device(B)
            points[f"decode_b{B}"] = round(v, 1)
            points[f"decode_b{B}_hbm_frac"] = round(bench.decode_bytes(B, c) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        # the same decode step launched kernel by kernel from the host, no CUDA graph (device-timed like `value`)
        points[f"decode_b{a.batch}_no_graph"] = round(bench.decode_no_graph(a.batch), 1)
        out["points"] = points
        ms, flops = bench.prefill()
        out["prefill"] = {"value": round(PREFILL_TOKENS / ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                          "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "peaks": pk["source"],
                          "flops": flops}
        bench.close()
        del bench
        if not a.no_shapes:
            # further sizes of the same architecture (the other shapes the project's baseline names): speed points only
            for name, shp, prompt_len in (("llama3_8b", LLAMA3_8B, 1024),):
                b2 = ShapeBench(shp, prompt_len, 64, min(a.steps, 16), a.warmup, a.block_size, prefill_tokens=prompt_len)
                for B in (1, 8, 64):
                    v, ms, _, c = b2.decode_device(B)
                    points[f"{name}_decode_b{B}"] = round(v, 1)
                    points[f"{name}_decode_b{B}_hbm_frac"] = round(b2.decode_bytes(B, c) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                ms, flops = b2.prefill(reps=3)
                points[f"{name}_prefill_{prompt_len}"] = round(prompt_len / ms * 1e3, 1)
                points[f"{name}_prefill_{prompt_len}_frac"] = round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
                b2.close()
                del b2
            points.update(qwen_mixed_serving(a, pk))
    print(json.dumps(out))
    return 0


# the other two shapes of the project's baseline: speed points at further sizes of the same architecture
LLAMA3_8B = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                 num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=500000.0,
                 rms_norm_eps=1e-5, attention_bias=False, tie_word_embeddings=False, max_position_embeddings=8192)
QWEN25_7B = dict(architectures=["Qwen2ForCausalLM"], vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                 num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, head_dim=128, rope_theta=1000000.0,
                 rms_norm_eps=1e-6, attention_bias=True, tie_word_embeddings=False, max_position_embeddings=32768)


def matmul_params(cfg):
    """(per-layer matrix elements, head elements)"""
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    per_layer = qkv * cfg.hidden_size + cfg.hidden_size * cfg.num_attention_heads * cfg.head_dim + 3 * cfg.intermediate_size * cfg.hidden_size
    return per_layer, cfg.vocab_size * cfg.hidden_size


class ShapeBench:
    """A model of one shape with random weights, and the measurements made on it."""

    def __init__(self, shape, prompt_len, max_batch, steps, warmup, block_size, prefill_tokens):
        import torch
        import forge_b200 as forge
        from forge_b200.config import config_from_dict
        from forge_b200.weights import random_tensors
        self.torch, self.forge = torch, forge
        self.cfg = cfg = config_from_dict(shape)
        self.prompt_len, self.steps, self.warmup, self.prefill_tokens = prompt_len, steps, warmup, prefill_tokens
        tensors = random_tensors(cfg, seed=0, std=0.02, device="cuda")
        total_steps = steps + warmup + 2
        per_request = -(-(prompt_len + total_steps + 16) // block_size) * block_size        # a request holds whole pages
        cache_tokens = max(max_batch * per_request, prefill_tokens + block_size)
        self.model = forge.Model(config=cfg, tensors=tensors, dtype="bfloat16", max_num_seqs=max_batch, cache_tokens=cache_tokens,
                                 max_tokens_per_step=2048, block_size=block_size)
        del tensors
        self.runner = self.model.runner
        self.gen = torch.Generator().manual_seed(0)

    def close(self):
        self.model = self.runner = None
        import gc
        gc.collect()
        self.torch.cuda.empty_cache()

    def prompts(self, B, n=None):
        return [self.torch.randint(0, self.cfg.vocab_size, (n or self.prompt_len,), generator=self.gen).tolist() for _ in range(B)]

    def timed(self, fn, steps):
        torch = self.torch
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    def _fill(self, B, tag):
        from forge_b200.engine import StepEntry
        ids = [f"{tag}{B}_{i}" for i in range(B)]
        ps = self.prompts(B)
        for rid in ids:
            self.runner.admit(rid)
        per_step = max(1, 2048 // self.prompt_len)
        for i in range(0, B, per_step):
            self.runner.step([StepEntry(ids[j], ps[j], []) for j in range(i, min(B, i + per_step))])
        return ids, ps

    def decode_device(self, B):
        """Device-timed decode: argmax of step i is the input of step i+1 without leaving the device.
        Returns (tokens/s, ms per step, kernel launches in the timed region, mean context length)."""
        from forge_b200 import kernels
        from forge_b200.engine import StepEntry
        runner = self.runner
        ids, ps = self._fill(B, "d")
        dummy = [StepEntry(rid, [0], [0]) for rid in ids]
        runner.decode_step([StepEntry(rid, [p[-1]], [0]) for rid, p in zip(ids, ps)])     # any token starts the chain

        def one():
            runner.decode_step(dummy, tokens_on_device=True)
        for _ in range(self.warmup):
            one()
        n0 = kernels.launch_count()
        ms = self.timed(one, self.steps)
        launches = kernels.launch_count() - n0
        ctx = self.prompt_len + 1 + self.warmup + self.steps // 2
        for rid in ids:
            runner.release(rid)
        return B * self.steps / ms * 1e3, ms / self.steps, launches, ctx

    def decode_no_graph(self, B):
        """The decode step as separate launches from the host (the ordinary step function), greedy tokens read back
        every step: what the CUDA graph saves."""
        from forge_b200 import kernels
        from forge_b200.engine import StepEntry
        runner = self.runner
        ids, ps = self._fill(B, "n")
        was, runner.cuda_graphs = runner.cuda_graphs, False
        toks = [p[-1] for p in ps]

        def one():
            nonlocal toks
            logits = runner.step([StepEntry(rid, [t], [0]) for rid, t in zip(ids, toks)])
            toks = kernels.argmax(logits).tolist()
        try:
            for _ in range(self.warmup):
                one()
            ms = self.timed(one, self.steps)
        finally:
            runner.cuda_graphs = was
            for rid in ids:
                runner.release(rid)
        return B * self.steps / ms * 1e3

    def decode_e2e(self, B):
        forge, runner = self.forge, self.runner
        sched = forge.RequestScheduler(self.model, max_num_seqs=B)
        greedy = forge.SamplerConfig(do_sample=False)
        for p in self.prompts(B):
            sched.submit(p, max_new_tokens=self.steps + self.warmup + 8, sampler_config=greedy)
        while any(r.status.name != "Decoding" for r in sched.get_all_requests()):
            sched.step()
        for _ in range(self.warmup):
            sched.step()
        ms = self.timed(sched.step, self.steps)
        g = next(v for (s_, _), v in runner._decode_graphs.items() if s_ == B)
        sched.reset()
        return B * self.steps / ms * 1e3, g.host.numel() * 4, B * 4

    def decode_bytes(self, B, ctx):
        """Bytes one decode step must read: every matrix once, norms, the embedding rows, and the live cache."""
        cfg = self.cfg
        per_layer, head = matmul_params(cfg)
        L, H = cfg.num_hidden_layers, cfg.hidden_size
        w_bytes = 2 * (L * per_layer + head) + 4 * H * (2 * L + 1)
        kv_per_token = 2 * cfg.num_key_value_heads * cfg.head_dim * 2 * L
        return w_bytes + B * (ctx * kv_per_token + H * 2)

    def prefill(self, reps=5):
        """One request of prefill_tokens tokens in one step, logits at the last position only: (ms, FLOPs)."""
        from forge_b200.engine import StepEntry
        cfg, T, runner = self.cfg, self.prefill_tokens, self.runner
        toks = self.prompts(1, T)[0]

        def run():
            runner.admit("p")
            runner.step([StepEntry("p", toks, [T - 1])])
            runner.release("p")
        for _ in range(3):
            run()
        ms = self.timed(run, reps) / reps
        per_layer, head = matmul_params(cfg)
        L = cfg.num_hidden_layers
        flops = 2 * T * L * per_layer + L * 2 * T * T * cfg.head_dim * cfg.num_attention_heads + 2 * head
        return ms, flops


def qwen_mixed_serving(a, pk):
    """The Qwen2.5-7B-shaped scenario: 64 requests with prompt lengths uniform in 128..8192 (seeded), served through the
    scheduler with at most 2,048 tokens a step, prompts cut into portions beside decoded tokens, 16 new tokens each.
    Returns points: all tokens computed per second, the share of the sustained tensor peak, steps and preemptions."""
    import torch
    import forge_b200 as forge
    from forge_b200.config import config_from_dict
    from forge_b200.weights import random_tensors
    cfg = config_from_dict(QWEN25_7B)
    gen = torch.Generator().manual_seed(1)
    lens = torch.randint(128, 8193, (64,), generator=gen).tolist()
    new_tokens = 16
    total = sum(lens) + 64 * new_tokens
    cache_tokens = sum(-(-(n + new_tokens + 1) // a.block_size) * a.block_size for n in lens)
    tensors = random_tensors(cfg, seed=0, std=0.02, device="cuda")
    model = forge.Model(config=cfg, tensors=tensors, dtype="bfloat16", max_num_seqs=64, cache_tokens=cache_tokens,
                        max_tokens_per_step=2048, block_size=a.block_size)
    del tensors
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
    greedy = forge.SamplerConfig(do_sample=False)

    def serve(ps):
        sched = forge.RequestScheduler(model, max_num_seqs=64)
        for p in ps:
            sched.submit(p, max_new_tokens=new_tokens, sampler_config=greedy)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        done = sched.run()
        torch.cuda.synchronize()
        return time.perf_counter() - t0, sched, done
    # once untimed: kernels compiled, and a CUDA graph captured for every number of requests that decode together as
    # the batch drains (a server would see each of them again and again)
    model.runner.max_decode_graphs = 256
    serve(prompts)
    secs, sched, done = serve(prompts)
    per_layer, head = matmul_params(cfg)
    L = cfg.num_hidden_layers
    # attention: every token attends to what precedes it in its request
    att = sum(2 * 2 * cfg.head_dim * cfg.num_attention_heads * L * (n + new_tokens) * (n + new_tokens) / 2 for n in lens)
    flops = 2 * total * L * per_layer + att + 2 * head * 64 * new_tokens
    out = {"qwen25_7b_mixed_tok_s": round(total / secs, 1), "qwen25_7b_mixed_tokens": total, "qwen25_7b_mixed_steps": sched.num_steps,
           "qwen25_7b_mixed_preemptions": sched.num_preemptions,
           "qwen25_7b_mixed_frac_sustained": round(flops / secs / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12), 4),
           "qwen25_7b_mixed_finished": sum(r.finish_reason == "length" for r in done)}
    model = sched = None
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


if __name__ == "__main__":
    sys.exit(main())
