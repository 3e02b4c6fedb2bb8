"""Builds libneureka_cuda.so in-tree with nvcc for sm_100a.

    python -m neureka_b200.build [--force] [--verbose]

Each translation unit is compiled to an object file (in parallel, only when out of date) and linked
into neureka_b200/lib/libneureka_cuda.so with the static CUDA runtime, so the library has no
dependency on torch or on the toolkit's shared runtime.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(LIBDIR, "libneureka_cuda.so")
# the input generator alone, host code only (no CUDA runtime inside): what a process that must not touch the GPU loads
JRAND_LIB = os.path.join(LIBDIR, "libnk_jrand.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-O2,-fno-fast-math"]

# (source, extra flags). The elementwise family is compiled without multiply-add contraction: the
# reference's CPU implementation is Java, which never fuses a*b+c.
SOURCES = [
    ("nk_runtime.cu", []),
    ("nk_elementwise.cu", ["-fmad=false"]),
    ("nk_ew_unary.cu", ["-fmad=false"]),
    ("nk_conv.cu", []),
    ("nk_conv_gemm.cu", []),
    ("nk_conv_tc.cu", []),
    ("nk_conv_tiled.cu", []),
    ("nk_conv_tiled_inst_f32_ldgsts.cu", []),
    ("nk_conv_tiled_inst_f32_tma4.cu", []),
    ("nk_conv_tiled_inst_f32_tma8.cu", []),
    ("nk_conv_tiled_inst_f64_ldgsts.cu", []),
    ("nk_conv_tiled_inst_f64_tma4.cu", []),
    ("nk_conv_tiled_inst_f64_tma8.cu", []),
    ("nk_conv_wgrad_inst_f32.cu", []),
    ("nk_conv_wgrad_inst_f64.cu", []),
    ("nk_fused.cu", ["-I", OBJDIR]),
    ("nk_group.cu", []),
    ("nk_reduce.cu", []),
    ("nk_probe.cu", []),
    ("nk_sum_static.cu", ["-fmad=false"]),
    ("nk_jrand.cpp", ["-Xcompiler", "-ffp-contract=off"]),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _headers_mtime() -> float:
    t = 0.0
    for d in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return max(t, os.path.getmtime(os.path.abspath(__file__)))


def _write_fused_prelude() -> None:
    """The run-time compiled (NVRTC) fused kernels must use the very scalar functions the precompiled kernels use:
    nk_scalarfun.cuh and the operator / function ids of the public header go into one C++ raw string literal that
    nk_fused.cu includes. Rewritten only when its content changes, so that it does not force a rebuild."""
    import re
    with open(os.path.join(HERE, "..", "include", "neureka_cuda.h")) as f:
        pub = f.read()
    enums = []
    for name in ("nk_op", "nk_fun"):
        m = re.search(r"typedef enum \{[^}]*\} " + name + ";", pub, re.S)
        if not m:
            raise RuntimeError(f"enum {name} not found in include/neureka_cuda.h")
        enums.append(re.sub(r"/\*.*?\*/", "", m.group(0), flags=re.S))
    with open(os.path.join(CSRC, "nk_scalarfun.cuh")) as f:
        body = "".join(line for line in f if not line.startswith("#include") and not line.startswith("#pragma once"))
    text = 'R"NKPRE(\n' + "\n".join(enums) + "\n" + body + '\n)NKPRE"\n'
    path = os.path.join(OBJDIR, "nk_fused_prelude.inc")
    old = None
    if os.path.exists(path):
        with open(path) as f:
            old = f.read()
    if old != text:
        with open(path, "w") as f:
            f.write(text)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    _write_fused_prelude()
    nvcc = _nvcc()
    hdr_t = _headers_mtime()
    jobs = []
    objs = []
    for src, extra in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, os.path.splitext(src)[0] + ".o")
        objs.append(o)
        stale = force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t)
        if stale:
            cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([nvcc, *ARCH, "-shared", "-o", LIB, *objs])
    build_jrand(force)
    return LIB


def build_jrand(force: bool = False) -> str:
    """libnk_jrand.so: nk_jrand.cpp compiled by the host compiler alone."""
    os.makedirs(LIBDIR, exist_ok=True)
    src = os.path.join(CSRC, "nk_jrand.cpp")
    if force or not os.path.exists(JRAND_LIB) or os.path.getmtime(JRAND_LIB) < os.path.getmtime(src):
        cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
               "-o", JRAND_LIB, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("host compiler failed for nk_jrand.cpp")
    return JRAND_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
