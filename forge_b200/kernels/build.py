"""Compiles the CUDA libraries of forge_b200 for sm_100a with plain nvcc, in-tree, on first use.

Each library is a handful of ``.cu`` files under ``forge_b200/csrc`` with ``extern "C"`` entry points
and no dependency but the CUDA runtime, so a library compiles in seconds and only the libraries a run
needs are built (the 32-bit path never compiles the tensor-core kernels).  Objects and ``.so`` files go
to ``forge_b200/csrc/_build`` (or, if the checkout is read-only, to a per-user temporary folder) and
are rebuilt when a source, a header or a flag changes.
"""
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

LIBRARIES = {
    # embedding, norm, rotary + cache write, activation, fp32 GEMM, fp32/any-shape attention, sampling
    "core": ["embedding.cu", "norm.cu", "rope_cache.cu", "activation.cu", "gemm_simt.cu",
             "attention_simt.cu", "sampling.cu"],
    # bf16 tcgen05 + TMA GEMM with fused epilogues
    "gemm_sm100": ["gemm_sm100.cu"],
    # bf16 tensor-core paged attention (mma.sync) for any head size, prompt portions and decode
    # ... and the decode step's attention that streams a long context through a TMA ring (head sizes 64 and 128)
    "attention_mma": ["attention_mma.cu", "attention_decode_stream.cu"],
    # bf16 tcgen05/TMEM paged attention for prompt portions, head sizes 64 and 128 (built per head size)
    "attention_sm100": ["attention_sm100.cu"],
    # all layers of a decode step in one persistent kernel (tcgen05 + TMA weight stream, attention inside)
    "decode_layers": ["decode_layers.cu"],
}

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise BuildError("forge_b200 needs nvcc (CUDA 12.8+) to compile its sm_100a kernels; none found on PATH "
                         "or at /usr/local/cuda/bin/nvcc")
    return exe


def _build_dir():
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        open(probe, "w").close()
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"forge_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _digest(files):
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for f in files:
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _say(msg):
    # compilation takes seconds to a minute: said whatever the log level, so that a first call does not look hung
    print(f"[forge_b200] {msg}", file=sys.stderr, flush=True)


def _run_with_heartbeat(cmds, what):
    """Runs the commands in parallel; prints a line every few seconds while they run."""
    t0 = time.time()
    procs = [subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for c in cmds]
    done = threading.Event()

    def beat():
        while not done.wait(8.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=beat, daemon=True)
    th.start()
    outs = [p.communicate()[0] for p in procs]
    done.set()
    for p, c, o in zip(procs, cmds, outs):
        if p.returncode != 0:
            raise BuildError(f"nvcc failed ({' '.join(c)}):\n{o}")


def build_library(name, force=False, defines=None):
    """Returns the path of lib ``name``, compiling it first if it is missing or stale.  ``defines``
    ({macro: value}) selects a variant of the library, built and cached under its own file name (the
    attention library is compiled per head size)."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    srcs = [os.path.join(CSRC, s) for s in LIBRARIES[name]]
    dflags = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    lib_sources = LIBRARIES[name]
    name = name + "".join(f"_{k.lower().replace('forge_', '')}{v}" for k, v in sorted((defines or {}).items()))
    headers = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for s in srcs:
        if not os.path.exists(s):
            raise BuildError(f"kernel source {s} is missing")
    out_dir = _build_dir()
    so = os.path.join(out_dir, f"libforge_{name}.so")
    stamp = so + ".sha256"
    want = _digest(srcs + headers) + "".join(dflags)
    with open(os.path.join(out_dir, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and os.path.exists(so) and os.path.exists(stamp) and open(stamp).read() == want:
            return so
        nvcc = _nvcc()
        _say(f"compiling kernel library '{name}' for sm_100a ({len(lib_sources)} files) ...")
        t0 = time.time()
        objs = [os.path.join(out_dir, f"{name}_{os.path.basename(s)[:-3]}.o") for s in srcs]
        _run_with_heartbeat([[nvcc, *NVCC_FLAGS, *dflags, "-I", CSRC, "-c", s, "-o", o] for s, o in zip(srcs, objs)],
                            f"'{name}'")
        tmp = so + f".tmp{os.getpid()}"
        _run_with_heartbeat([[nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]],
                            f"'{name}' (link)")
        os.replace(tmp, so)
        with open(stamp, "w") as f:
            f.write(want)
        _say(f"built {os.path.basename(so)} in {time.time() - t0:.1f} s")
    return so


# head sizes whose attention library build_all compiles ahead of time; others compile on first use
COMMON_HEAD_DIMS = (64, 128)


def build_all(force=False):
    out = {}
    for name in LIBRARIES:
        if name in ("attention_mma", "attention_sm100", "decode_layers"):
            for hd in COMMON_HEAD_DIMS:
                out[f"{name}_hd{hd}"] = build_library(name, force=force, defines={"FORGE_ATT_HD": hd})
        else:
            out[name] = build_library(name, force=force)
    return out
