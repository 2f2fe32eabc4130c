"""Builds ``libbitdecode.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python -m bitladder_b200.build`` or call :func:`build`.  nvcc
cross-compiles without a GPU, so this works on a CPU-only host; the resulting
shared object sits beside this file and is what :mod:`bitladder_b200._lib` loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
BUILD_DIR = os.path.join(_HERE, "build")
LIB_PATH = os.path.join(_HERE, "libbitdecode.so")
SOURCES = ["bd_pack.cu", "bd_decode.cu", "bd_combine.cu", "bd_exchange.cu", "bd_rope.cu", "bd_api.cu"]
HEADERS = ["bd_common.cuh", "bd_kernels.h", os.path.join("..", "..", "include", "bitdecode.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


# Per-file additions.  The decode kernel may use the approximate exp/log/division and
# flush-to-zero fp32 (its parity bound is 2e-3 and these act on softmax weights and the final
# normalisation; measured 0.8 us on a 63 us step).  The pack kernel must NOT: its quantizer is
# bit-exact IEEE arithmetic with explicit rounding intrinsics.
PER_FILE_FLAGS = {"bd_decode.cu": ["--use_fast_math"]}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: cannot build libbitdecode.so")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=()) -> str:
    """Compile every CUDA source and link the shared library; returns its path."""
    nvcc = _nvcc()
    os.makedirs(BUILD_DIR, exist_ok=True)
    hdrs = [os.path.normpath(os.path.join(CSRC, h)) for h in HEADERS]
    jobs = []
    objs = []
    for src in SOURCES:
        spath = os.path.join(CSRC, src)
        obj = os.path.join(BUILD_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [spath, os.path.abspath(__file__)] + hdrs):
            cmd = [nvcc, *NVCC_FLAGS, *PER_FILE_FLAGS.get(src, []), *extra_flags, "-c", spath, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stdout + r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(4, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out)
    if force or jobs or _stale(LIB_PATH, objs):
        run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-lcudart"])
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
