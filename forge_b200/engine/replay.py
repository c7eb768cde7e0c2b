"""Trace replay: feeds given token ids through the model step by step and writes logits.  It samples
nothing and decides nothing: the trace is the schedule.  It drives the same ``ModelRunner.step`` (model,
cache manager, kernels) that generation uses.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["b"]}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the wanted places in the
order of the entries and of ``want``, little-endian float32 [wanted, vocab].  After every step a line
``done <step>`` is printed and flushed.
"""
import json
import os
import sys

from .runner import ModelRunner, StepEntry

DEFAULT_MAX_LIVE = 4


def replay(model_dir, dtype, out_dir, max_tokens, lines, page_size=64, stdout=None, max_live=DEFAULT_MAX_LIVE):
    stdout = stdout or sys.stdout
    os.makedirs(out_dir, exist_ok=True)
    # the pool holds max_tokens tokens, each live request rounded up to a multiple of 64
    page = page_size if 64 % page_size == 0 else 64
    runner = ModelRunner(model_dir, dtype=dtype, page_size=page, cache_tokens=max_tokens, max_requests=max_live)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            if not runner.is_live(e["id"]):
                runner.admit(e["id"])
            entries.append(StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                arr = logits.to("cpu").contiguous().numpy().astype("<f4", copy=False)
                with open(os.path.join(out_dir, f"{rec['step']}.f32"), "wb") as f:
                    f.write(arr.tobytes())
            runner.check_status()
        for rid in rec.get("end", []):
            if runner.is_live(rid):
                runner.release(rid)
        print(f"done {rec['step']}", file=stdout, flush=True)
    return 0


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="replay a token trace and dump logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--max-requests", type=int, default=DEFAULT_MAX_LIVE, help="most requests live at a time")
    a = ap.parse_args(argv)
    return replay(a.model, a.dtype, a.out, a.max_tokens, sys.stdin, page_size=a.page_size, max_live=a.max_requests)
