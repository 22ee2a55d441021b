"""Builds libfnx_b200.so in-tree with nvcc for sm_100a (no GPU needed: nvcc cross-compiles).

    python <package>/build.py [--force] [--verbose]

The shared library has a plain C ABI (include/fnx_b200.h) and links only the CUDA runtime.  Beside it, fnx_serve: the
engine process of the line protocol (csrc/serve.cpp), a plain C++ program over that ABI.
"""
from __future__ import annotations

import argparse
import os
import pathlib
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libfnx_b200.so"
SERVE = HERE / "fnx_serve"
SOURCES = ["common.cu", "iq3s_prep.cu", "iq3s_mmv.cu", "moe_route.cu", "attn.cu", "attn_prompt_tc.cu", "gdn.cu", "moe_prefill.cu", "gemm_tma.cu", "head.cu", "spec.cu", "lane_plan.cu", "gguf.cu", "model_load.cu", "engine.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-Xcompiler", "-Wall"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (c == "nvcc" or pathlib.Path(c).exists()):
            return c
    raise RuntimeError("nvcc not found")


def _stale() -> bool:
    if not OUT.exists() or not SERVE.exists():
        return True
    t = min(OUT.stat().st_mtime, SERVE.stat().st_mtime)
    deps = (list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cpp")) + list(CSRC.glob("*.hpp"))
            + [HERE.parent / "include" / "fnx_b200.h"])
    return any(d.stat().st_mtime > t for d in deps)


def _build_serve() -> None:
    cmd = ["g++", "-O2", "-std=c++17", "-Wall", str(CSRC / "serve.cpp"), "-o", str(SERVE), "-L", str(HERE), "-lfnx_b200", "-Wl,-rpath,$ORIGIN", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("fnx_serve failed to build")


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not _stale():
        return OUT
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    procs = []
    for src in SOURCES:
        obj = objdir / (src + ".o")
        cmd = [nvcc, *FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(f"--- {src}\n{out}\n")
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(str(obj))
    cmd = [nvcc, "-shared", "-o", str(OUT), *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    _build_serve()
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
