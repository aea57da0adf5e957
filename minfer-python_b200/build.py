"""Build libminfer_attn.so (the C-ABI attention library) for sm_100a, in-tree.

Replaces the reference's setup.py CUDAExtension build
(setup.py:19-86 of dsuarez01/minfer-python, which targets compute_89 and asserts
a GPU at build time): the translation units in SOURCES compiled in parallel and
linked by one `nvcc -shared`, one target architecture, no GPU needed to build.

Usage:  python build.py [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OUT_DIR = os.path.join(HERE, "minfer", "kernels", "torch_ext")
LIB_NAME = "libminfer_attn.so"
SOURCES = ["attn_api.cu", "prefill_persist_sm100.cu", "mask_classify.cu", "decode_sm100.cu", "decode_static_sm100.cu",
           "rope_append_sm100.cu"]
HEADERS = ["attn_internal.h", "ptx.cuh"]
# the LibTorch stable-ABI registration unit (schemas + CUDA impls that call the C ABI), host code only
BINDING_NAME = "_C.abi3.so"
BINDING_SOURCES = ["torch_binding/reg.cpp", "torch_binding/reg_cuda.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def lib_path() -> str:
    return os.path.join(OUT_DIR, LIB_NAME)


def _newest_source_mtime() -> float:
    files = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    files.append(os.path.join(INCLUDE, "minfer_attn.h"))
    return max(os.path.getmtime(f) for f in files)


def _find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libminfer_attn.so cannot be built")
    return nvcc


def binding_path() -> str:
    return os.path.join(OUT_DIR, BINDING_NAME)


def build_binding(force: bool = False, verbose: bool = False) -> str:
    """Compile the torch extension `minfer.kernels.torch_ext._C` (the reference builds the module of that
    name with a CUDAExtension, setup.py:65-80): two host-only translation units against torch's stable-ABI
    headers (-DTORCH_TARGET_VERSION 2.10, Py_LIMITED_API cp312, as the reference's setup.py:41-42), linked
    against libminfer_attn.so next to it."""
    import sysconfig

    import torch
    out = binding_path()
    srcs = [os.path.join(CSRC, f) for f in BINDING_SOURCES]
    newest = max(os.path.getmtime(f) for f in srcs + [os.path.join(INCLUDE, "minfer_attn.h")])
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(newest, os.path.getmtime(lib_path())):
        return out
    tdir = os.path.dirname(torch.__file__)
    cxx = shutil.which("g++") or "g++"
    flags = ["-std=c++17", "-O2", "-fPIC", "-DPy_LIMITED_API=0x030c0000", "-DTORCH_TARGET_VERSION=0x020a000000000000",
             "-DUSE_CUDA", "-I", os.path.join(tdir, "include"), "-I", sysconfig.get_paths()["include"]]
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    objs = []
    for src in srcs:
        obj = os.path.join(build_dir, os.path.basename(src).replace(".cpp", ".o"))
        cmd = [cxx, *flags, "-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        objs.append(obj)
    cmd = [cxx, "-shared", "-o", out, *objs, "-L", OUT_DIR, "-l:" + LIB_NAME, "-Wl,-rpath,$ORIGIN",
           "-L", os.path.join(tdir, "lib"), "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10"]
    subprocess.run(cmd, check=True)
    return out


def build(force: bool = False, verbose: bool = False, binding: bool = True) -> str:
    """Compile if the library is missing or older than its sources (and the torch extension on top of it);
    return the library's path."""
    out = _build_library(force, verbose)
    if binding:
        build_binding(force, verbose)
    return out


def _build_library(force: bool = False, verbose: bool = False) -> str:
    out = lib_path()
    if not force and os.path.exists(out) and os.path.getmtime(out) >= _newest_source_mtime():
        return out
    nvcc = _find_nvcc()
    objs = []
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        log, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stdout.write(log)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    cmd = [nvcc, "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args()
    print(build(force=ns.force, verbose=ns.verbose))
