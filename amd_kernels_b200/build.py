"""Builds libb200moe.so in-tree with nvcc for sm_100a (ahead of time; there is no JIT and no other architecture)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200moe.so")
SIBLING_INTERMEDIATES = (1536,)  # further builds of the same sources: libb200moe_i<I>.so


def lib_path(inter: int = 768) -> str:
    return LIB if inter == 768 else os.path.join(HERE, f"libb200moe_i{inter}.so")

SOURCES = ["abi.cu", "route_sort.cu", "router_gemm.cu", "router_tc.cu", "quant.cu", "preshuffle.cu", "reduce.cu", "gemm_simt.cu", "gemm_tc.cu", "gemm_pair.cu", "ep_sync.cu", "shared_tc.cu", "sidecar.cu", "tail.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: libb200moe.so cannot be built")
    return path


def needs_build(inter: int = 768) -> bool:
    if not os.path.exists(lib_path(inter)):
        return True
    built = os.path.getmtime(lib_path(inter))
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "b200_moe.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False, inter: int = 768) -> str:
    """Compile every kernel source to an object (in parallel) and link the shared library for intermediate size ``inter``
    (768: libb200moe.so; 1536: libb200moe_i1536.so, the same sources with -DB200MOE_I=1536). Returns its path."""
    lib = lib_path(inter)
    if not force and not needs_build(inter):
        return lib
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build" if inter == 768 else f"build_i{inter}")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *FLAGS, f"-DB200MOE_I={inter}", *(["-Xptxas", "-v"] if verbose else []), "-c", os.path.join(CSRC, src),
               "-o", obj]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose:
            print(out)
        objs.append(obj)
    cmd = [nvcc, "-shared", "-o", lib, *objs, "-lcudart"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return lib


def build_all(force: bool = False, verbose: bool = False) -> list:
    return [build(force, verbose, inter) for inter in (768, *SIBLING_INTERMEDIATES)]


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
