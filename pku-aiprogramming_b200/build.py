"""In-tree build of the native library (sm_100a only).

    python pku-aiprogramming_b200/build.py [--force] [--verbose]

Compiles every translation unit under `csrc/` with nvcc for `sm_100a` and links
`lib/libtt_attn.so`, the C-ABI shared library declared in `include/tt_attn.h`.
nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libtt_attn.so")

KERNEL_SOURCES = ["tt_api.cu", "tt_mgpu.cu", "attn_simt.cu", "attn_decode.cu", "attn_decode_gq_sm100.cu", "attn_fwd_sm100.cu", "attn_fwd_pair_sm100.cu", "attn_bwd_sm100.cu", "attn_bwd_pair_sm100.cu", "attn_bwd_fused_sm100.cu",
                  "softmax_rows.cu", "fc_gemm_sm100.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Wno-deprecated-gpu-targets",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-I" + os.path.join(ROOT, "include"),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newest_header() -> float:
    t = 0.0
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdr_t = _newest_header()
    objs, jobs = [], []
    for src in KERNEL_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-c", s, "-o", o])
    rebuilt = bool(jobs)
    if jobs:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 2)) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if rebuilt or not os.path.exists(LIB):
        _run([_nvcc(), "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB, *objs, "-cudart", "static", "-ldl"], verbose)
    return LIB


HOST = os.path.join(CSRC, "host")
HOST_DIR = os.path.join(PKG, "host_modules")   # myTensor*.so and myLayer*.so land here


def build_host_modules(force: bool = False, verbose: bool = False):
    """The reference-style pybind11 modules `myTensor` and `myLayer` (they link libtt_attn.so)."""
    import sysconfig
    import pybind11
    build_library(force=False, verbose=verbose)
    os.makedirs(HOST_DIR, exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + HOST]
    import torch  # only for the directory that holds ATen/dlpack.h (the DLPack ABI header)
    inc.append("-I" + os.path.join(os.path.dirname(torch.__file__), "include"))
    flags = [f for f in NVCC_FLAGS if f != "-fvisibility=hidden"]
    # drop the "-Xcompiler" that preceded the removed visibility flag
    cleaned, skip = [], False
    for i, f in enumerate(NVCC_FLAGS):
        if f == "-Xcompiler" and i + 1 < len(NVCC_FLAGS) and NVCC_FLAGS[i + 1] == "-fvisibility=hidden":
            skip = True
            continue
        if skip:
            skip = False
            continue
        cleaned.append(f)
    hdr_t = max(_newest_header(), max(os.path.getmtime(os.path.join(HOST, f)) for f in os.listdir(HOST) if f.endswith(".h")))
    objs, jobs = {}, []
    for src in ("TinyTensor.cu", "Layers.cu", "bind_Tensor.cu", "bind_Layer.cu"):
        s_ = os.path.join(HOST, src)
        o = os.path.join(OBJ, "host_" + src[:-3] + ".o")
        objs[src] = o
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s_), hdr_t):
            jobs.append([_nvcc(), *cleaned, *inc, "-c", s_, "-o", o])
    if jobs:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    link = ["-shared", "-Wno-deprecated-gpu-targets", "-L" + LIB_DIR, "-ltt_attn", "-Xlinker", "-rpath", "-Xlinker",
            "$ORIGIN/../lib", "-cudart", "static"]
    outs = []
    for name, parts in (("myTensor", ["bind_Tensor.cu", "TinyTensor.cu"]),
                        ("myLayer", ["bind_Layer.cu", "Layers.cu", "TinyTensor.cu"])):
        out = os.path.join(HOST_DIR, name + suffix)
        if jobs or not os.path.exists(out):
            _run([_nvcc(), *link, "-o", out, *[objs[p_] for p_ in parts]], verbose)
        outs.append(out)
    return outs


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    for m_ in build_host_modules(force="--force" in sys.argv, verbose="--verbose" in sys.argv):
        print(m_)
