"""bench.py's answers that need no GPU: more than one GPU is refused with one line and exit code 2, and the
reference arm, where the reference is neither built nor to be found, says so in one JSON line and exits with 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120,
                       env=dict(os.environ, **(env or {})))
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    return p.returncode, lines


def test_more_than_one_gpu_is_refused_with_one_line():
    rc, lines = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert rc == 2 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["n_gpus"] == 2 and "single-GPU" in d["error"]


def test_reference_arm_without_a_build_says_why(tmp_path):
    """With no built reference and no sources to build it from, the arm prints its one `unavailable` line (the
    real arm runs baseline/_ref/cuda/ref_bench, the unmodified reference built by baseline/build_reference.py)."""
    rc, lines = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1",
                     env={"FORGE_REFERENCE_BUILD": str(tmp_path / "nothing"), "FORGE_REFERENCE_SOURCE": str(tmp_path / "absent")})
    assert rc == 0 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "not built" in d["unavailable"] and "\n" not in d["unavailable"]
