"""Builds libb200dnn.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m juliavision_b200.build [--force] [--verbose]

The shared object lands next to the sources (juliavision_b200/csrc/libb200dnn.so) so that it
travels with the tree.  There is no CPU or other-architecture build of this library.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO = os.path.join(CSRC, "libb200dnn.so")
SOURCES = ["ctx.cu", "layernorm.cu", "gemm.cu", "attention.cu", "glue.cu", "conv.cu", "gemv.cu", "attention_window.cu", "selftest.cu"]
HEADERS = ["internal.h", "ptx.cuh", "act.cuh", os.path.join("..", "..", "include", "b200dnn.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
    "-ccbin", "/usr/bin/g++",
]


def _stale(obj: str, deps) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    procs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [NVCC, *FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    if force or procs or _stale(SO, objs):
        cmd = [NVCC, "-shared", "-o", SO, *objs, "-ccbin", "/usr/bin/g++", "-cudart", "static",
               "-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.run(cmd, check=True)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
