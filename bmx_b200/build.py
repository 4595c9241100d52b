"""Builds libbmxk.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: python -m bmx_b200.build [--force]
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbmxk.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
# (source, extra flags).  The codec file keeps multiplies and adds separate, as the reference's
# float32 arithmetic does; fused sums in it are written with fmaf.
SOURCES = [
    ("api.cu", []),
    ("k2b_codec.cu", ["-fmad=false"]),
    ("k2b_decode.cu", []),
    ("k2b_decode_t5.cu", []),
    ("k2b_prefill.cu", []),
    ("k2b_prefill_t5.cu", []),
    ("rtn.cu", ["-fmad=false"]),
    ("spectral.cu", ["-fmad=false"]),
    ("spectral_decode_t5.cu", []),
    ("value_blocks.cu", ["-fmad=false"]),
    ("xchg.cu", []),
]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "bmxk.h"))
    objs = []
    for src, extra in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = ["nvcc", *ARCH, *COMMON, *extra, "-c", s, "-o", o]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
    if force or _stale(LIB, objs):
        cmd = ["nvcc", *ARCH, "-shared", "-o", LIB, *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
