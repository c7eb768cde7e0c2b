"""bench.py's answers that need no GPU: more than one GPU is refused with one line and exit code 2, and the
reference arm says in one JSON line why it is unavailable."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    return p.returncode, lines


def test_more_than_one_gpu_is_refused_with_one_line():
    rc, lines = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert rc == 2 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["n_gpus"] == 2 and "single-GPU" in d["error"]


def test_reference_arm_is_unavailable_and_says_why():
    rc, lines = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert rc == 0 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and len(d["unavailable"]) > 10 and "\n" not in d["unavailable"]
