"""Builds ``libember_b200.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m ember_b200.build [--force]

nvcc cross-compiles without a GPU. The shared object lands beside the package
(``ember_b200/libember_b200.so``) so that it travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libember_b200.so")

SOURCES = ["core.cu", "tma_host.cu", "attn_simt.cu", "attn_decode.cu", "attn_fwd_sm100.cu",
           "attn_bwd_sm100.cu", "api.cu", "gemm_simt.cu", "gemm_sm100.cu", "linear_api.cu",
           "softmax_ce.cu", "kv_cache.cu", "comm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _deps_mtime() -> float:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "ember_b200.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr_t = _deps_mtime()
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), r.stderr))
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out)
    if jobs or not os.path.exists(LIB):
        run([_nvcc(), "-shared", "-o", LIB, *objs, "-cudart", "shared", "-ldl"])
    build_binding(force or bool(jobs))
    return LIB


def build_binding(force: bool = False) -> str:
    """Compiles the CPython binding (csrc/tensor_api.c) into ember_b200/_core/, linked against the
    CUDA library beside it (found at run time through an $ORIGIN-relative rpath)."""
    import sysconfig

    src = os.path.join(CSRC, "tensor_api.c")
    out = os.path.join(HERE, "_core", "_tensor" + sysconfig.get_config_var("EXT_SUFFIX"))
    hdr = os.path.join(os.path.dirname(HERE), "include", "ember_b200.h")
    if force or not os.path.exists(out) or os.path.getmtime(out) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        cmd = [os.environ.get("CC", "gcc"), "-O2", "-fPIC", "-shared", "-I", sysconfig.get_paths()["include"], src,
               "-o", out, "-L", HERE, "-lember_b200", "-Wl,-rpath,$ORIGIN/.."]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("binding build failed: %s\n%s" % (" ".join(cmd), r.stderr))
    return out


def build_bounds_checked() -> str:
    """``libember_b200_dbg.so``: the same library with -DEMBER_BOUNDS_CHECK (every global store of the
    tensor-core attention kernels checked against its tensor's extent; see csrc/common.cuh). Objects
    go to build/dbg/. Select it at run time with EMBER_B200_LIB=<path>."""
    obj = os.path.join(OBJ, "dbg")
    os.makedirs(obj, exist_ok=True)
    lib = os.path.join(HERE, "libember_b200_dbg.so")
    hdr_t = _deps_mtime()
    jobs, objs = [], []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj, src.replace(".cu", ".o"))
        objs.append(o)
        if not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-DEMBER_BOUNDS_CHECK", "-c", s, "-o", o])
    for cmd in jobs:
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), r.stderr))
    if jobs or not os.path.exists(lib):
        r = subprocess.run([_nvcc(), "-shared", "-o", lib, *objs, "-cudart", "shared", "-ldl"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: %s" % r.stderr)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--bounds" in sys.argv:
        print(build_bounds_checked())
