"""Builds libsptmm.so (and the rcr / ccc command-line programs) in-tree with nvcc for sm_100a.

    python sptmm_b200/build.py [--force] [--verbose] [--ptxas] [--tuning]

The shared library is the product: a C ABI (include/sptmm.h) over hand-written CUDA kernels.
Objects are rebuilt only when their source, or a shared header, is newer.

--tuning builds a second library beside it, libsptmm_tuning.so, compiled with -DSPTMM_TUNING:
the kernels then carry timestamp hooks for timelines and launch constants can be overridden from
the environment (csrc/tuning.h).  Nothing in the product library reads the environment.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libsptmm.so")
LIB_TUNING = os.path.join(PKG, "libsptmm_tuning.so")
BIN = os.path.join(PKG, "bin")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"] + ARCH
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread"]

LIB_SOURCES = ["host_encode.cpp", "weights_file.cpp", "stack.cpp", "ternarise.cpp", "device_api.cu", "kernels_native.cu", "kernels_compat.cu", "kernels_seq.cu", "kernels_quant.cu", "splitk.cu", "cublas_cmp.cu"]
HEADERS = ["internal.h", "device_common.cuh", "tuning.h", os.path.join(ROOT, "include", "sptmm.h")]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n  %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)


def _build_library(lib: str, obj_dir: str, defines: list[str], force: bool, verbose: bool, ptxas_info: bool) -> None:
    os.makedirs(obj_dir, exist_ok=True)
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    jobs, objs = [], []
    for src in LIB_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            if src.endswith(".cu"):
                cmd = ["nvcc"] + NVCC_FLAGS + defines + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", s, "-o", o]
            else:
                cmd = ["g++"] + CXX_FLAGS + defines + ["-c", s, "-o", o]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        list(ex.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    if force or jobs or not os.path.exists(lib):
        _run(["nvcc", "-shared", "-o", lib] + objs + ARCH + ["-lcublas", "-Xcompiler", "-pthread"], verbose)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, tuning: bool = False) -> str:
    os.makedirs(BIN, exist_ok=True)
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    _build_library(LIB, OBJ, [], force, verbose, ptxas_info)
    if tuning:
        _build_library(LIB_TUNING, OBJ + "_tuning", ["-DSPTMM_TUNING"], force, verbose, False)
    cli = os.path.join(CSRC, "cli.cpp")
    if os.path.exists(cli):
        for name, layout in (("rcr", "-DSPTMM_CLI_RCR"), ("ccc", "-DSPTMM_CLI_CCC")):
            out = os.path.join(BIN, name)
            if force or _newer(out, [cli, LIB] + hdrs):
                _run(["g++"] + CXX_FLAGS + [layout, cli, "-o", out, "-L" + PKG, "-lsptmm",
                      "-Wl,-rpath,$ORIGIN/.."], verbose)
    enc = os.path.join(CSRC, "cli_encode.cpp")
    out = os.path.join(BIN, "sptmm_encode")
    if os.path.exists(enc) and (force or _newer(out, [enc, LIB] + hdrs)):
        _run(["g++"] + CXX_FLAGS + [enc, "-o", out, "-L" + PKG, "-lsptmm", "-Wl,-rpath,$ORIGIN/.."], verbose)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_info="--ptxas" in sys.argv,
                 tuning="--tuning" in sys.argv)
    print(path)
