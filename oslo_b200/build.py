"""Ahead-of-time build of the in-tree extensions (``python -m oslo_b200.build``).

* ``oslo_b200/_C.so``      - sm_100a CUDA kernels + ``torch.ops.oslo_b200`` bindings
* ``oslo_b200/_C_bounds.so`` - the same, compiled with ``-DOSLO_DEBUG_BOUNDS`` (``--debug-bounds`` builds only this one)
* ``oslo_b200/_data_C.so`` - host-only dataset index builders

The reference compiles its kernels at first use with ``torch.utils.cpp_extension.load``
(oslo/fused_kernels_utils.py:116-141); here nothing is compiled at run time: the kernels are built
for exactly one target, ``-gencode arch=compute_100a,code=sm_100a``, and loaded from the package
directory. nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "csrc", "build")

CUDA_SOURCES = ["gemm_sm100.cu", "elementwise.cu", "attention.cu", "attention_sm100.cu", "attention_bwd_sm100.cu",
                "decode_sm100.cu", "comm.cu", "fused_comm_gemm.cu", "noalloc_colsum.cu"]
CPP_SOURCES = ["bindings.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout)


def _stamp(paths: List[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _needs(out: str, stamp_file: str, stamp: str) -> bool:
    if not os.path.exists(out) or not os.path.exists(stamp_file):
        return True
    with open(stamp_file) as f:
        return f.read().strip() != stamp


def build_kernels(force: bool = False, verbose: bool = True, debug_bounds: bool = False) -> str:
    """``debug_bounds``: the same sources with ``-DOSLO_DEBUG_BOUNDS`` into ``_C_bounds.so`` (loaded instead of
    ``_C.so`` when ``OSLO_B200_DEBUG_BOUNDS=1``): data-dependent indices that had to be skipped or clamped are
    reported through the device error word."""
    import torch
    from torch.utils import cpp_extension

    os.makedirs(BUILD, exist_ok=True)
    tag = "_C_bounds" if debug_bounds else "_C"
    extra = ["-DOSLO_DEBUG_BOUNDS"] if debug_bounds else []
    out = os.path.join(HERE, tag + ".so")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    cu = [os.path.join(CSRC, f) for f in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, f))]
    cpp = [os.path.join(CSRC, f) for f in CPP_SOURCES]
    stamp = _stamp(cu + cpp + headers, torch.__version__ + " ".join(NVCC_FLAGS + extra))
    stamp_file = os.path.join(BUILD, tag + ".stamp")
    if not force and not _needs(out, stamp_file, stamp):
        return out
    nvcc = _nvcc()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    inc = ["-I" + CSRC, "-I" + os.path.join(cuda_home, "include")]
    tinc = ["-I" + p for p in cpp_extension.include_paths()]
    objs: List[str] = []
    jobs = []
    suffix = ".bounds.o" if debug_bounds else ".o"
    for src in cu:
        obj = os.path.join(BUILD, os.path.basename(src) + suffix)
        objs.append(obj)
        jobs.append([nvcc] + NVCC_FLAGS + extra + inc + ["-c", src, "-o", obj])
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for src in cpp:
        obj = os.path.join(BUILD, os.path.basename(src) + suffix)
        objs.append(obj)
        jobs.append(["g++", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                     "-DTORCH_EXTENSION_NAME=_C"] + inc + tinc + ["-c", src, "-o", obj])
    if verbose:
        print(f"[oslo_b200.build] compiling {len(jobs)} sources for sm_100a", flush=True)
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        list(ex.map(_run, jobs))
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = ["g++", "-shared", "-o", out] + objs + [
        "-L" + tlib, "-L" + os.path.join(cuda_home, "lib64"), "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
        "-ltorch", "-lcudart", "-Wl,-rpath," + tlib, "-Wl,-rpath," + os.path.join(cuda_home, "lib64")]
    _run(link)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    if verbose:
        print(f"[oslo_b200.build] wrote {out}", flush=True)
    return out


def build_data(force: bool = False, verbose: bool = True) -> str:
    os.makedirs(BUILD, exist_ok=True)
    src = os.path.join(CSRC, "data_builders.cpp")
    out = os.path.join(HERE, "_data_C.so")
    if not os.path.exists(src):
        return out
    stamp = _stamp([src], "data")
    stamp_file = os.path.join(BUILD, "_data_C.stamp")
    if not force and not _needs(out, stamp_file, stamp):
        return out
    _run(["g++", "-std=c++17", "-O3", "-fPIC", "-shared", src, "-o", out])
    with open(stamp_file, "w") as f:
        f.write(stamp)
    if verbose:
        print(f"[oslo_b200.build] wrote {out}", flush=True)
    return out


def build_all(force: bool = False, verbose: bool = True, debug_bounds: bool = True) -> None:
    build_kernels(force, verbose)
    if debug_bounds:
        build_kernels(force, verbose, debug_bounds=True)
    build_data(force, verbose)


if __name__ == "__main__":
    if "--debug-bounds" in sys.argv:
        build_kernels(force="--force" in sys.argv, debug_bounds=True)
    else:
        build_all(force="--force" in sys.argv)
