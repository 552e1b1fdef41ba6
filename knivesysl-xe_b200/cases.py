"""Runs one kernel of the library on a named shape, a few launches over rotating weights
(so that weights come from HBM, not L2), or times every named shape.

  python knivesysl-xe_b200/cases.py run <case> [launches]     # e.g. under ncu
  python knivesysl-xe_b200/cases.py time [case ...]           # CUDA-graph replay timing

Cases: cfg1 (GEMV 17408x5120 K32), gemv_down (GEMV 5120x17408), cfg1_from_x / cfg1_one_launch and
gemv_down_from_x / gemv_down_one_launch (the same GEMVs from the fp32 row: x_gemv_w4a8 = staging
launch + GEMV, and x_gemv_w4a8_fused = quantiser in the GEMV's prologue), cfg2 (fused gate+up K64,
T=8), down_t8 / down_t16 / down_t32 / down_t64 (5120x17408 K32), prefill_small (tcgen05 GEMM
2048x5120, T=1024), cfg4 (tcgen05 GEMM 17408x5120 K64, T=4096 in 4 segments), cfg4_w4a4 (the
same shape through x_gemm_w4a4: int4 activations, one promote per K64 group), w8_lm_head (W8A8
GEMV 151936x5120, 803 MB of weights: no rotation needed).
Weights are seeded random codes and scales: timing does not depend on their values.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import __init__ as pkg  # noqa: E402  (the package directory name is not an identifier)

HBM_GBS = 6545.0
ROT = 4


def rand_weight(M, K, k64, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 256, size=M * K // 2, dtype=np.uint8)
    g = 64 if k64 else 32
    scales = (0x2400 + rng.integers(0, 64, size=M * (K // g), dtype=np.uint16) * 16).astype(np.uint16)
    return pkg.PackedWeight(codes, scales, M, K, k64=k64)


class Gemv:
    def __init__(self, lib, M, K, k64):
        self.lib, self.M, self.K = lib, M, K
        self.ws = [rand_weight(M, K, k64, s) for s in range(ROT)]
        x = np.random.default_rng(1).standard_normal(K).astype(np.float32)
        self.dx = pkg.DevBuf.from_numpy(x)
        self.y = pkg.DevBuf(M * 4)
        lib.qwn_x_prepare_gemv_act_s8(self.dx.ptr, K)
        self.bytes = self.ws[0].weight_bytes
        self.ops = 2.0 * M * K

    def launch(self, i):
        assert self.lib.qwn_x_gemv_w4a8_prepared(self.ws[i % ROT].ref, self.y.ptr, None) == 0


class GemvFromX(Gemv):
    """x_gemv_w4a8 from the fp32 row (quantiser + GEMV in one call)."""

    def launch(self, i):
        assert self.lib.qwn_x_gemv_w4a8(self.ws[i % ROT].ref, self.dx.ptr, self.y.ptr) == 0


class GemvOneLaunch(Gemv):
    """x_gemv_w4a8_fused: the quantiser in the GEMV's prologue (one launch)."""

    def launch(self, i):
        assert self.lib.qwn_x_gemv_w4a8_fused(self.ws[i % ROT].ref, self.dx.ptr, None, self.y.ptr) == 0


class Gemm:
    def __init__(self, lib, Ms, K, k64, T, segments=0, rot=ROT):
        self.lib, self.T = lib, T
        self.sets = [[rand_weight(M, K, k64, s * 7 + j) for j, M in enumerate(Ms)] for s in range(rot)]
        self.rot = rot
        self.warr = [pkg.weight_array(p) for p in self.sets]
        x = np.random.default_rng(1).standard_normal((T, K)).astype(np.float32)
        self.dx = pkg.DevBuf.from_numpy(x)
        n = K // 32 * T
        self.aq, self.as_, self.asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
        lib.qwn_x_quantize_act_chunk(self.dx.ptr, K, T, self.aq.ptr, self.as_.ptr, self.asum.ptr)
        self.ys = [pkg.DevBuf(T * M * 4) for M in Ms]
        self.yarr = pkg.ptr_array(self.ys)
        self.n = len(Ms)
        self.offs = ((C.c_int * (segments + 1))(*[T // segments * i for i in range(segments + 1)])
                     if segments else None)
        self.segments = segments
        self.bytes = sum(w.weight_bytes for w in self.sets[0])
        self.ops = 2.0 * T * sum(Ms) * K

    def launch(self, i):
        if self.n == 1:
            rc = self.lib.qwn_x_gemm_w4a8(self.sets[i % self.rot][0].ref, self.aq.ptr, self.as_.ptr,
                                          self.asum.ptr, self.ys[0].ptr, self.T, self.offs, self.segments)
        else:
            rc = self.lib.qwn_x_gemm_w4a8_fanout(self.warr[i % self.rot], self.yarr, self.n, self.aq.ptr,
                                                 self.as_.ptr, self.asum.ptr, self.T, None, 0)
        assert rc == 0, rc


class GemvW8:
    """x_gemv_w8a8_prepared on one int8 weight (random codes, FP16 scales): the lm_head tier."""

    def __init__(self, lib, M, K):
        self.lib = lib
        rng = np.random.default_rng(5)
        codes = rng.integers(0, 256, size=M * K, dtype=np.uint8)
        scales = (0x2400 + rng.integers(0, 64, size=M * (K // 32), dtype=np.uint16) * 16).astype(np.uint16)
        self.codes, self.scales = pkg.DevBuf.from_numpy(codes), pkg.DevBuf.from_numpy(scales)
        self.rec = pkg.TqWeight()
        self.rec.M, self.rec.K, self.rec.Mt, self.rec.Kt = M, K, M // 16, K // 32
        self.rec.d_s8, self.rec.d_s8_scale, self.rec.s8_ready = self.codes.ptr, self.scales.ptr, 1
        x = np.random.default_rng(1).standard_normal(K).astype(np.float32)
        self.dx = pkg.DevBuf.from_numpy(x)
        self.y = pkg.DevBuf(M * 4)
        lib.qwn_x_prepare_gemv_act_s8(self.dx.ptr, K)
        self.bytes = codes.nbytes + scales.nbytes
        self.ops = 2.0 * M * K

    def launch(self, i):
        assert self.lib.qwn_x_gemv_w8a8_prepared(C.byref(self.rec), self.y.ptr, None) == 0


class GemmW4A4:
    """x_gemm_w4a4 on one K64 weight (int4 activations per (token, K64))."""

    def __init__(self, lib, M, K, T):
        self.lib, self.T = lib, T
        self.w = rand_weight(M, K, True, 3)
        x = np.random.default_rng(1).standard_normal((T, K)).astype(np.float32)
        self.dx = pkg.DevBuf.from_numpy(x)
        n = K // 64 * T
        self.aq4, self.as4, self.asum4 = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
        lib.qwn_x_quantize_act_chunk_s4(self.dx.ptr, K, T, self.aq4.ptr, self.as4.ptr, self.asum4.ptr)
        self.y = pkg.DevBuf(T * M * 4)
        self.bytes = self.w.weight_bytes
        self.ops = 2.0 * T * M * K

    def launch(self, i):
        rc = self.lib.qwn_x_gemm_w4a4(self.w.ref, self.aq4.ptr, self.as4.ptr, self.asum4.ptr,
                                      self.y.ptr, self.T)
        assert rc == 0, rc


CASES = {
    "cfg1": lambda lib: Gemv(lib, 17408, 5120, False),
    "gemv_down": lambda lib: Gemv(lib, 5120, 17408, False),
    "cfg1_from_x": lambda lib: GemvFromX(lib, 17408, 5120, False),
    "cfg1_one_launch": lambda lib: GemvOneLaunch(lib, 17408, 5120, False),
    "gemv_down_from_x": lambda lib: GemvFromX(lib, 5120, 17408, False),
    "gemv_down_one_launch": lambda lib: GemvOneLaunch(lib, 5120, 17408, False),
    "cfg2": lambda lib: Gemm(lib, [17408, 17408], 5120, True, 8),
    "down_t8": lambda lib: Gemm(lib, [5120], 17408, False, 8),
    "down_t16": lambda lib: Gemm(lib, [5120], 17408, False, 16),
    "down_t32": lambda lib: Gemm(lib, [5120], 17408, False, 32),
    "down_t64": lambda lib: Gemm(lib, [5120], 17408, False, 64),
    "prefill_small": lambda lib: Gemm(lib, [2048], 5120, True, 1024, rot=1),
    "cfg4": lambda lib: Gemm(lib, [17408], 5120, True, 4096, segments=4, rot=1),
    "cfg4_w4a4": lambda lib: GemmW4A4(lib, 17408, 5120, 4096),
    "w8_lm_head": lambda lib: GemvW8(lib, 151936, 5120),
}


def time_case(lib, case, per=20, reps=10):
    """us per launch: CUDA-graph replay of `per` rotating launches, events on the stream."""
    for i in range(3):
        case.launch(i)
    lib.tq_sync()
    ev0, ev1 = lib.tq_event_create(), lib.tq_event_create()
    assert lib.tq_graph_capture_begin() == 0
    for i in range(per):
        case.launch(i)
    g = lib.tq_graph_capture_end()
    assert g, "graph capture failed"
    lib.tq_graph_launch(g)
    lib.tq_sync()
    lib.tq_event_record(ev0)
    for _ in range(reps):
        lib.tq_graph_launch(g)
    lib.tq_event_record(ev1)
    lib.tq_sync()
    ms = lib.tq_event_elapsed_ms(ev0, ev1)
    lib.tq_graph_destroy(g)
    return ms / (per * reps) * 1e3


def main():
    if len(sys.argv) < 2 or sys.argv[1] not in ("run", "time"):
        print(__doc__)
        return 2
    lib = pkg.load()
    assert lib.tq_set_device(0) == 0
    if sys.argv[1] == "run":
        case = CASES[sys.argv[2]](lib)
        n = int(sys.argv[3]) if len(sys.argv) > 3 else 6
        for i in range(n):
            case.launch(i)
        lib.tq_sync()
        print("done", sys.argv[2], "launches", n, "error", lib.tq_last_error())
        return 0
    for name in (sys.argv[2:] or list(CASES)):
        case = CASES[name](lib)
        big = case.ops > 1e11
        us = time_case(lib, case, per=2 if big else 20, reps=3 if big else 10)
        print(json.dumps({"case": name, "us": round(us, 2),
                          "weight_GBps": round(case.bytes / us / 1e3, 1),
                          "frac_of_hbm_copy": round(case.bytes / us / 1e3 / HBM_GBS, 3),
                          "int8_TOPS": round(case.ops / us / 1e6, 1)}), flush=True)
        del case
    print("error", lib.tq_last_error())
    return 0


if __name__ == "__main__":
    sys.exit(main())
