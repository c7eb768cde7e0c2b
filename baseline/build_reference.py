#!/usr/bin/env python3
"""Builds the UNMODIFIED reference (Cyxuan0311/Forge) with its CUDA backend, by hand, into baseline/_ref/cuda.

    python baseline/build_reference.py --reference /path/to/Forge

The reference's own build (pip / CMake) cannot run offline: its CMakeLists fetches pybind11 over the network
(CMakeLists.txt:96-101) and its architecture list has no sm_100 (CMakeLists.txt:79-84).  Its sources need
neither: this script compiles the same source lists as its CMake targets forge_core, forge_ops, forge_model
and forge_infer (CMakeLists.txt:104-239) with the same definitions (USE_CUDA, FORGE_USE_CUBLAS=1,
FORGE_USE_OPENBLAS=0, USE_AVX2), the .cu files with `nvcc -gencode arch=compute_100,code=sm_100`, and links
them with baseline/ref_bench.cpp, a small driver that times the stock engine (EngineRegistry::create ->
InferenceEngine::forward).  Nothing of the reference is changed or copied; the objects and the executable
stay in baseline/_ref (not tracked).
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")

CPP = ["src/core/*.cpp", "src/debug/logger.cpp", "src/inference/*.cpp", "src/inference/engines/*.cpp",
       "src/operators/cpu/*.cpp", "src/model/*.cpp"]
CU = ["src/operators/cuda/*.cu"]
DEFS = ["-DUSE_CUDA", "-DFORGE_USE_CUBLAS=1", "-DFORGE_USE_OPENBLAS=0", "-DUSE_AVX2"]
CXXFLAGS = ["-std=c++20", "-O3", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-fPIC"]
NVCCFLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100,code=sm_100", "-Wno-deprecated-gpu-targets",
             "-Xcompiler", "-fPIC", "-rdc=true"]


def run_all(cmds, jobs=8):
    procs = []
    for c in cmds:
        procs.append((c, subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        if len(procs) >= jobs:
            c0, p0 = procs.pop(0)
            out = p0.communicate()[0]
            if p0.returncode != 0:
                raise SystemExit(f"FAILED: {' '.join(c0)}\n{out[-4000:]}")
    for c0, p0 in procs:
        out = p0.communicate()[0]
        if p0.returncode != 0:
            raise SystemExit(f"FAILED: {' '.join(c0)}\n{out[-4000:]}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(HERE, "_ref", "cuda"))
    a = ap.parse_args()
    ref, out = os.path.abspath(a.reference), os.path.abspath(a.out)
    os.makedirs(os.path.join(out, "obj"), exist_ok=True)
    inc = [f"-I{ref}/include", f"-I{ref}/src", f"-I{CUDA}/include"]
    nvcc = shutil.which("nvcc") or os.path.join(CUDA, "bin", "nvcc")
    cmds, objs = [], []
    for i, pat in enumerate(CPP):
        for s in sorted(glob.glob(os.path.join(ref, pat))):
            o = os.path.join(out, "obj", f"c{i}_{os.path.basename(s)[:-4]}.o")
            objs.append(o)
            if not os.path.exists(o):
                cmds.append(["g++", *CXXFLAGS, *DEFS, *inc, "-c", s, "-o", o])
    for s in sorted(glob.glob(os.path.join(ref, CU[0]))):
        o = os.path.join(out, "obj", f"cu_{os.path.basename(s)[:-3]}.o")
        objs.append(o)
        if not os.path.exists(o):
            cmds.append([nvcc, *NVCCFLAGS, *DEFS, *inc, "-c", s, "-o", o])
    print(f"compiling {len(cmds)} of {len(objs)} files ...", flush=True)
    run_all(cmds)
    drv = os.path.join(out, "obj", "ref_bench.o")
    run_all([["g++", *CXXFLAGS, *DEFS, *inc, "-c", os.path.join(HERE, "ref_bench.cpp"), "-o", drv]])
    exe = os.path.join(out, "ref_bench")
    # nvcc links: it resolves the relocatable device code of the .cu objects
    run_all([[nvcc, "-gencode", "arch=compute_100,code=sm_100", "-o", exe, drv, *objs, "-Xcompiler", "-fopenmp",
              "-lcublas", "-lcudart", "-lgomp"]])
    print("built", exe)


if __name__ == "__main__":
    sys.exit(main())
