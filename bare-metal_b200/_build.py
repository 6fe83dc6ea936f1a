"""Builds libbm_igemm.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libbm_igemm.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "--cudart", "static",
]


HOST_DIR = os.path.join(PKG_DIR, "host")
HOST_BIN = os.path.join(HOST_DIR, "bin")
HOST_PROGRAMS = ("bench_igemm", "bench_sparse", "bench_persistent")
DEVICE_TOOLS = ("linkprobe",)        # .cu programs with kernels of their own (sm_100a), no dependency on the library


def build_host(force: bool = False) -> list[str]:
    """Compile the C++ bench drivers (host code only) against libbm_igemm.so; returns their paths."""
    build(force=False)
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(HOST_BIN, exist_ok=True)
    include = os.path.join(os.path.dirname(PKG_DIR), "include")
    out = []
    for name in HOST_PROGRAMS:
        src, exe = os.path.join(HOST_DIR, name + ".cpp"), os.path.join(HOST_BIN, name)
        deps = [src, os.path.join(HOST_DIR, "host_common.h"), os.path.join(HOST_DIR, "sparse_host.h"), LIB_PATH]
        if force or not os.path.exists(exe) or any(os.path.getmtime(d) > os.path.getmtime(exe) for d in deps):
            cmd = [nvcc, "-O2", "-std=c++17", "-I" + include, "-I" + HOST_DIR, "-o", exe, src, "-L" + LIB_DIR,
                   "-lbm_igemm", "-Xlinker", "-rpath," + "$ORIGIN/../../lib", "--cudart", "static"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError("nvcc failed on " + name + ":\n" + res.stdout + res.stderr)
        out.append(exe)
    for name in DEVICE_TOOLS:
        src, exe = os.path.join(HOST_DIR, name + ".cu"), os.path.join(HOST_BIN, name)
        deps = [src, os.path.join(CSRC, "host_common.cuh"), os.path.join(CSRC, "sm100_ptx.cuh")]
        if force or not os.path.exists(exe) or any(os.path.getmtime(d) > os.path.getmtime(exe) for d in deps):
            cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-o", exe, src,
                   "--cudart", "static"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError("nvcc failed on " + name + ":\n" + res.stdout + res.stderr)
        out.append(exe)
    return out


COMPAT_DIR = os.path.join(PKG_DIR, "compat")
SHIM_PATH = os.path.join(LIB_DIR, "libbm_cubin_shim.so")


def build_shim(force: bool = False) -> str:
    """Compile the LD_PRELOAD shim that serves the reference benches' cubin loads from libbm_igemm.so."""
    build(force=False)
    src = os.path.join(COMPAT_DIR, "bm_cubin_shim.cpp")
    if force or not os.path.exists(SHIM_PATH) or os.path.getmtime(src) > os.path.getmtime(SHIM_PATH) \
            or os.path.getmtime(LIB_PATH) > os.path.getmtime(SHIM_PATH):
        include = os.path.join(os.path.dirname(PKG_DIR), "include")
        cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
        cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-I" + include, "-I" + cuda_inc,
               "-o", SHIM_PATH, src, "-L" + LIB_DIR, "-lbm_igemm", "-Wl,-rpath,$ORIGIN", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("building the cubin shim failed:\n" + res.stdout + res.stderr)
    return SHIM_PATH


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh")))


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    header = os.path.join(os.path.dirname(PKG_DIR), "include", "bm_igemm.h")
    return any(os.path.getmtime(s) > built for s in _sources() + [header])


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source of the package into one shared library; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(LIB_DIR, exist_ok=True)
    units = [s for s in _sources() if s.endswith(".cu")]
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH, *units]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH
