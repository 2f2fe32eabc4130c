"""Compiles the reference project's own CUDA kernels for sm_100a into ``oracle/_ref/``.

Test infrastructure, not product code: the modules built here are used only to produce
golden fixtures (``tests/golden/make_ref_golden.py``) and, optionally, to cross-check the
CPU restatement on a GPU host.  Nothing under ``bitladder_b200/`` loads them.

What is compiled, from where it lies (nothing is copied into this repository's history):

* ``csrc/bit_decode/src/genfile/*.cu`` — the five translation units the reference's
  ``setup.py:126-138`` lists (quantize-pack 2/4-bit, split-KV decode 2/4-bit, the empty
  non-split instance), with the flags of ``setup.py:140-157`` except for the target
  architecture (``sm_100a`` instead of sm_80/sm_90);
* ``csrc/bit_decode/decode_api.cpp`` — the pybind11 host API, twice:
  ``bit_decode_cuda`` from the file as it is (its pack entry ``kvcache_pack_i4`` has no
  architecture check and runs unmodified; its decode entry refuses every device that is not
  sm_8x / sm_90, ``decode_api.cpp:320-324``), and ``bit_decode_cuda_sm100`` from a copy under
  ``oracle/_ref/build/`` in which that one ``TORCH_CHECK`` is removed — a MODIFIED reference,
  labelled so wherever its outputs are used.

CUTLASS: the reference's ``libs/cutlass`` submodule is empty and un-pinned
(``.gitmodules:1-3``); the CuTe/CUTLASS header tree that ships inside the ``flashinfer``
wheel of this image is used instead.

Two variants are built: ``fast`` with ``--use_fast_math`` as the reference builds, and ``ieee``
without it, so that differences caused by approximate division show up as such.

    python oracle/build_ref.py [--variant fast|ieee|both] [--reference /path/to/reference]
"""
from __future__ import annotations

import argparse
import os
import re
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(_HERE, "_ref")
# the reference project's checkout: $BITDECODE_REFERENCE, else a directory `reference` beside this repository
DEFAULT_REFERENCE = os.environ.get("BITDECODE_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")

GENFILES = [
    "flash_fwd_hdim128_fp16_sm80.cu",
    "flash_qpack_hdim128_fp16_sm80_2bit.cu",
    "flash_qpack_hdim128_fp16_sm80_4bit.cu",
    "flash_fwd_split_hdim128_fp16_sm80_2bit.cu",
    "flash_fwd_split_hdim128_fp16_sm80_4bit.cu",
]

GUARD_RE = re.compile(r'TORCH_CHECK\(is_sm90 \|\| is_sm8x,[^;]*;')


def _cutlass_include() -> str:
    import importlib.util
    spec = importlib.util.find_spec("flashinfer")
    if spec is None or not spec.submodule_search_locations:
        raise RuntimeError("no CUTLASS headers: the flashinfer package (which vendors them) is not installed")
    inc = os.path.join(list(spec.submodule_search_locations)[0], "data", "cutlass", "include")
    if not os.path.isdir(os.path.join(inc, "cute")):
        raise RuntimeError(f"no CuTe headers under {inc}")
    return inc


def _torch_paths():
    import torch
    tdir = os.path.dirname(torch.__file__)
    inc = [os.path.join(tdir, "include"), os.path.join(tdir, "include", "torch", "csrc", "api", "include")]
    return inc, os.path.join(tdir, "lib"), int(torch._C._GLIBCXX_USE_CXX11_ABI)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed:\n" + " ".join(cmd) + "\n" + r.stdout[-4000:] + r.stderr[-4000:])
    return r.stdout + r.stderr


def build(reference: str = DEFAULT_REFERENCE, variants=("fast", "ieee"), jobs: int = 0, force: bool = False):
    """Build the modules; returns {variant: directory holding bit_decode_cuda*.so}."""
    src_root = os.path.join(reference, "csrc", "bit_decode")
    api = os.path.join(src_root, "decode_api.cpp")
    if not os.path.exists(api):
        raise RuntimeError(f"reference sources not found under {reference}")
    nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    cutlass = _cutlass_include()
    tinc, tlib, cxx11 = _torch_paths()
    pyinc = sysconfig.get_paths()["include"]
    bdir = os.path.join(OUT, "build")
    os.makedirs(bdir, exist_ok=True)

    # the one host-side modification: a copy of the API file without the architecture check
    text = open(api).read()
    relaxed, n = GUARD_RE.subn("/* architecture check removed for the sm_100a test build */", text)
    if n != 1:
        raise RuntimeError("the architecture check of decode_api.cpp was not found exactly once")
    relaxed_path = os.path.join(bdir, "decode_api_sm100.cpp")
    with open(relaxed_path, "w") as f:
        f.write(relaxed)

    includes = [src_root, os.path.join(src_root, "src"), cutlass, *tinc, pyinc, "/usr/local/cuda/include"]
    inc_flags = [f"-I{p}" for p in includes]
    common = ["-O3", "-std=c++17", f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    nv_common = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", *common,
                 "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
                 "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                 "-Xcompiler", "-fPIC", "-w", *inc_flags]

    cmds, links, result = [], [], {}
    for variant in variants:
        vdir = os.path.join(OUT, variant)
        os.makedirs(vdir, exist_ok=True)
        result[variant] = vdir
        math = ["--use_fast_math"] if variant == "fast" else []
        objs = []
        for g in GENFILES:
            obj = os.path.join(bdir, f"{variant}_{g[:-3]}.o")
            objs.append(obj)
            if force or not os.path.exists(obj):
                cmds.append([*nv_common, *math, "-c", os.path.join(src_root, "src", "genfile", g), "-o", obj])
        for mod, src in (("bit_decode_cuda", api), ("bit_decode_cuda_sm100", relaxed_path)):
            obj = os.path.join(bdir, f"{variant}_{mod}.o")
            if force or not os.path.exists(obj):
                cmds.append(["g++", *common, "-fPIC", "-w", f"-DTORCH_EXTENSION_NAME={mod}", *inc_flags,
                             "-c", src, "-o", obj])
            so = os.path.join(vdir, mod + sysconfig.get_config_var("EXT_SUFFIX"))
            links.append(["g++", "-shared", "-o", so, obj, *objs, f"-L{tlib}", "-L/usr/local/cuda/lib64",
                          "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
                          "-lcudart", f"-Wl,-rpath,{tlib}"])
    workers = jobs or max(1, min(len(cmds), (os.cpu_count() or 2)))
    if cmds:
        with ThreadPoolExecutor(max_workers=workers) as ex:
            list(ex.map(_run, cmds))
    for cmd in links:
        _run(cmd)
    return result


def load(variant: str = "fast", relaxed: bool = True):
    """Import a built module (needs torch imported first so that its libraries are resolved).  Load the
    modules of ONE variant per process: both variants export the same module and kernel names, and with
    both loaded the second one ran the first one's code."""
    import importlib.util
    import torch  # noqa: F401
    name = "bit_decode_cuda_sm100" if relaxed else "bit_decode_cuda"
    path = os.path.join(OUT, variant, name + sysconfig.get_config_var("EXT_SUFFIX"))
    if not os.path.exists(path):
        raise RuntimeError(f"{path} not built; run python oracle/build_ref.py where the reference sources are")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def time_decode_c2(variant: str = "fast", steps: int = 200) -> float:
    """Microseconds per step of the reference's split-KV decode (+ combine) kernels on the headline shape
    (batch 8, 32 query / 8 KV heads, 32768 tokens, 4-bit, group 128; no tail: the reference has none),
    CUDA-event timed over three rotating caches packed by the reference's own pack kernel.  Launched
    eagerly through the reference's host API, which allocates its split buffers on every call."""
    import math
    import torch
    mod_pack, mod_decode = load(variant, relaxed=False), load(variant, relaxed=True)
    b, s, h, h_k, dev = 8, 32768, 32, 8, "cuda"
    g = torch.Generator(device=dev).manual_seed(7)
    caches = []
    for _ in range(3):
        k_pack = torch.zeros((b, s // 4, h_k, 128), dtype=torch.uint16, device=dev)
        k_params = torch.zeros((b, s // 128, h_k, 128), dtype=torch.float32, device=dev)
        v_pack = torch.zeros((b, s, h_k, 32), dtype=torch.uint16, device=dev)
        v_params = torch.zeros((b, 1, h_k, s), dtype=torch.float32, device=dev)
        for ib in range(b):
            k = torch.randn(s, h_k, 128, generator=g, device=dev).half()
            v = torch.randn(s, h_k, 128, generator=g, device=dev).half()
            cu = torch.tensor([0, s], dtype=torch.int32, device=dev)
            mod_pack.kvcache_pack_i4(k, k_pack[ib:ib + 1], k_params[ib:ib + 1], v, v_pack[ib:ib + 1],
                                     v_params[ib:ib + 1], None, cu, s, "k-channel", 128)
        caches.append((k_pack, k_params, v_pack, v_params))
    q = torch.randn(b, 1, h, 128, generator=g, device=dev).half()
    sc = 1.0 / math.sqrt(128)

    def step(i):
        c = caches[i % 3]
        return mod_decode.fwd_kvcache_i4(q, c[0], c[1], c[2], c[3], None, sc, "k-channel", 128, False, -1, -1, 0.0,
                                         True, 0)
    for i in range(20):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1e3


def available(variant: str = "fast") -> bool:
    return os.path.exists(os.path.join(OUT, variant, "bit_decode_cuda_sm100" + sysconfig.get_config_var("EXT_SUFFIX")))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--variant", default="both", choices=["fast", "ieee", "both"])
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--jobs", type=int, default=0)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--clean", action="store_true")
    a = ap.parse_args()
    if a.clean and os.path.isdir(OUT):
        shutil.rmtree(OUT)
    out = build(a.reference, ("fast", "ieee") if a.variant == "both" else (a.variant,), a.jobs, a.force)
    for k, v in out.items():
        print(k, v, sorted(os.listdir(v)))
    sys.exit(0)
