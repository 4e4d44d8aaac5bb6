"""Builds lumi_b200/lib/liblumi_b200.so (and the `lumi-infer-b200` CLI) with nvcc for sm_100a only.

    python -m lumi_b200.build [--force] [--verbose]

The shared library is kept in-tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "liblumi_b200.so")
CLI = os.path.join(LIBDIR, "lumi-infer-b200")

SOURCES = ["api.cu", "kernels.cu", "gemm_tcgen05.cu", "attention.cu", "decode_b1.cu", "block_static.cu", "prefill_ssd.cu", "safetensors.cpp"]
HEADERS = ["internal.h", "json_min.h", os.path.join("..", "..", "include", "lumi_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-ccbin", "/usr/bin/g++"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    flags = list(NVCC_FLAGS)
    if not os.path.exists("/usr/bin/g++"):
        flags = flags[:-2]
    if verbose:
        flags += ["-Xptxas", "-v"]
    procs = []
    for src in SOURCES:
        sp = os.path.join(CSRC, src)
        obj = os.path.join(LIBDIR, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [sp] + hdrs):
            cmd = [_nvcc()] + flags + ["-x", "cu", "-c", sp, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(f"--- {src}\n{out}\n")
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    if force or procs or _stale(LIB, objs):
        cmd = [_nvcc()] + flags + ["-shared", "--cudart", "static", "-o", LIB] + objs
        subprocess.run(cmd, check=True)
    cli_src = os.path.join(CSRC, "cli_main.cpp")
    if os.path.exists(cli_src) and (force or _stale(CLI, [cli_src, LIB])):
        cmd = [_nvcc()] + flags + [cli_src, "-o", CLI, "-L" + LIBDIR, "-llumi_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
