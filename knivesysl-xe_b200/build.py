"""Builds libforward_qwen_xpu.so in-tree with nvcc for sm_100a (no torch, no JIT cache).

python knivesysl-xe_b200/build.py [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libforward_qwen_xpu.so")

SOURCES = ["runtime.cu", "quant.cu", "repack.cu", "gemv.cu", "gemv_e2m3.cu", "tqf.cu", "grid_probe.cu", "gemm_mma.cu", "gemm_stream.cu", "gemm_tc.cu", "gemm_dtc.cu", "tc_peak.cu",
           "dispatch.cu", "checks.cu", "comm.cu", "gemv_static.cu", "w8a8.cu", "cxx_linkage.cpp"]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    # no implicit a*b+c contraction: every fused multiply-add in the kernels is an explicit
    # fmaf(), so the fp32 results are the ones the CPU oracle restates
    "-fmad=false",
    "-Xcompiler", "-fPIC,-O2,-fvisibility=default",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "tq_w4a8.h"),
                                                                os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for src in SOURCES:
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- {src} failed ---\n{out}\n")
        elif verbose or "warning" in out:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
            "-lcudart", "-ldl"]
    subprocess.check_call(link)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
