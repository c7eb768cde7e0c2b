#!/usr/bin/env python3
"""Makes tests/golden/ref_logits_*.npy by running the UNMODIFIED reference CPU engine.

    python tests/golden/make_golden.py --reference /path/to/Forge [--workdir DIR]

It compiles the reference's CPU sources as plain scalar C++ (no AVX2, no BLAS, no CUDA),
links ref_driver.cpp against them, feeds the deterministic tiny models of golden_model.py
through `InferenceEngine::forward` and stores the logits.  The test
tests/test_plain_vs_golden.py then checks the plain implementation against these files, so
the suite itself never needs the reference.  Both models were also checked here against the
plain implementation when the files were made (max |diff| printed at the end).
"""
import argparse
import glob
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from golden_model import GOLDEN_CONFIGS, GOLDEN_STEPS, golden_tensors  # noqa: E402

FLAGS = ["-std=c++20", "-O1", "-fopenmp", "-DFORGE_USE_CUBLAS=0", "-DFORGE_USE_OPENBLAS=0"]


def build(ref, work):
    os.makedirs(os.path.join(work, "obj"), exist_ok=True)
    lib = os.path.join(work, "libforge_scalar.a")
    if not os.path.exists(lib):
        srcs = []
        for pat in ["src/core/*.cpp", "src/debug/logger.cpp", "src/inference/*.cpp",
                    "src/inference/engines/*.cpp", "src/operators/cpu/*.cpp", "src/model/*.cpp"]:
            srcs += sorted(glob.glob(os.path.join(ref, pat)))
        procs = []
        for i, s in enumerate(srcs):
            o = os.path.join(work, "obj", f"{i:03d}_{os.path.basename(s)[:-4]}.o")
            procs.append(subprocess.Popen(["g++", *FLAGS, f"-I{ref}/include", f"-I{ref}/src", "-c", s, "-o", o]))
            if len(procs) >= 8:
                assert procs.pop(0).wait() == 0
        for p in procs:
            assert p.wait() == 0
        subprocess.check_call(["ar", "rcs", lib, *sorted(glob.glob(os.path.join(work, "obj", "*.o")))])
    exe = os.path.join(work, "ref_driver")
    subprocess.check_call(["g++", *FLAGS[:3], f"-I{ref}/include", f"-I{ref}/src",
                           os.path.join(HERE, "ref_driver.cpp"), "-Wl,--whole-archive", lib,
                           "-Wl,--no-whole-archive", "-o", exe])
    return exe


def run(exe, work, name):
    cfg, steps = GOLDEN_CONFIGS[name], GOLDEN_STEPS[name]
    tensors = golden_tensors(cfg, seed=7)
    wpath, opath = os.path.join(work, name + ".w.bin"), os.path.join(work, name + ".out.bin")
    with open(wpath, "wb") as f:
        for arr in tensors.values():          # insertion order == the driver's read order
            f.write(np.ascontiguousarray(arr, dtype="<f4").tobytes())
    spec = [cfg["vocab_size"], cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"],
            cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rope_theta"],
            cfg["rms_norm_eps"], int(cfg["tie_word_embeddings"]), int(cfg["attention_bias"]), len(steps)]
    text = " ".join(str(x) for x in spec) + "\n"
    for start, toks in steps:
        text += f"{start} {len(toks)} " + " ".join(map(str, toks)) + "\n"
    subprocess.run([exe, wpath, opath], input=text.encode(), check=True, stdout=subprocess.DEVNULL)
    total = sum(len(t) for _, t in steps)
    return np.fromfile(opath, dtype="<f4").reshape(total, cfg["vocab_size"])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--workdir", default=os.path.join(HERE, "..", "..", "baseline", "_ref"))
    a = ap.parse_args()
    exe = build(os.path.abspath(a.reference), os.path.abspath(a.workdir))
    sys.path.insert(0, os.path.join(HERE, ".."))
    import torch
    from plain.llama import PlainLlama
    for name in GOLDEN_CONFIGS:
        ref = run(exe, os.path.abspath(a.workdir), name)
        np.save(os.path.join(HERE, f"ref_logits_{name}.npy"), ref)
        plain = PlainLlama.from_tensors(GOLDEN_CONFIGS[name], golden_tensors(GOLDEN_CONFIGS[name], seed=7))
        ids = [t for _, toks in GOLDEN_STEPS[name] for t in toks]
        mine = plain.logits(ids).to(torch.float32).numpy()
        print(name, "rows", ref.shape, "max|plain - reference| =", float(np.abs(mine - ref).max()),
              "logit scale", float(np.abs(ref).max()))


if __name__ == "__main__":
    main()
