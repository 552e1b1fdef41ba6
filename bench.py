#!/usr/bin/env python
"""Benchmark of the W4A8 projection path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
  python bench.py --case NAME --launches L       # one kernel, L launches (profiler target)

Prints ONE JSON line on rank 0.

N = 1. Headline ("cfg2"): batched decode fused gate+up projection, K64 scale tier, T = 8
tokens, K = 5120, N = 2 x 17408; seeded N(0, 0.02) weights symmetric-quantised to int4;
N(0, 1) activations with 1% of the channels scaled x20, quantised to int8 per token. One step
= per-token activation staging (1 launch) + ONE fused gate|up GEMM launch over a weight copy
that rotates through `rotate` distinct copies (> L2 in total), so weights come from HBM.
`per_config` holds one record for every other benchmark configuration (single GEMV, the
down-projection sweep, the packed prefill GEMM in each activation mode, the 64-layer stack),
each with its own device time, roofline, end-to-end time through the C ABI with host buffers
and a bounded CPU sample; `prefill_int8_TOPS` is the packed prefill GEMM's throughput and
`int8_peak` the tcgen05 kind::i8 issue peak measured in the same run.

N > 1 (torchrun, one rank per GPU): the 64-layer stack, every projection column-sharded N ways
with x_w4_shard, strong scaling (the same 13.4 GB of weights per step at every N); the line
also carries `weak_cfg2`, the headline projection with per-GPU work fixed. `--scaling weak`
prints that record as the line instead (whole-job weight bytes per second over N GPUs).
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_gemv_weight_GBps"
UNIT = "GB/s"
WORKLOAD_CFG2 = ("cfg2: batched decode fused gate+up, K64 scale tier, T=8, K=5120, N=2x17408, "
                 "int8 per-token activations")
WORKLOAD_CFG5 = ("cfg5: 64-layer projection stack at decode T=8 (5120->10240, 10240->5120, "
                 "5120->2x17408, 17408->5120 per layer, group-32 int4 weights, int8 per-token "
                 "activations), column-sharded over the GPUs, strong scaling")
H, I_FF, QKV = 5120, 17408, 10240          # hidden, MLP width, first projection's width
# DRAM traffic of one launch of the headline kernel, from the profiler capture named here;
# None when the kernel has changed since the capture.
NCU_TRAFFIC = {"bytes_per_launch": 98344448,
               "capture": "profiles/gemm_w4a8_ring_kernel__cfg2.md: ncu --set full --clock-control none "
                          "-k regex:gemm_w4a8_ring -s 3 -c 2 python bench.py --case cfg2 --launches 6 "
                          "(dram__bytes_read.sum 94,822,144 + dram__bytes_write.sum 3,522,304, one launch of "
                          "the full-size cfg2 workload)"}
NOMINAL_INT8_TOPS = 4500.0


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the GPU is under the benchmark's load."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, spans):
        """spans: list of (t0, t1) wall-clock intervals in which the GPU was under load."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            if not any(t0 <= ts <= t1 + 0.06 for t0, t1 in spans):
                continue
            f = [c.strip() for c in line.split(",")]
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except Exception:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


def host_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


# ------------------------------------------------------------------------------------------
# shared state of one benchmark process
# ------------------------------------------------------------------------------------------
class Ctx:
    def __init__(self, rotate: int):
        self.pkg = importlib.import_module("knivesysl-xe_b200")
        self.wl = importlib.import_module("knivesysl-xe_b200.workloads")
        self.lib = self.pkg.load()          # raises if the CUDA library is missing
        self.rotate = rotate
        self.ev = None
        self._host_w = {}
        self.load_spans = []
        self.peak_hbm, self.peak_bf16, self.peak_kind = measured_peaks()

    def events(self):
        if self.ev is None:
            self.ev = [self.lib.tq_event_create() for _ in range(2)]
        return self.ev

    def host_weight(self, M, K, seed, group):
        key = (M, K, seed, group)
        if key not in self._host_w:
            self._host_w[key] = self.wl.make_weight_w4(M, K, seed=seed, group=group)
        return self._host_w[key]

    def rotated(self, M, K, seed, group, n=None):
        """n device copies of one seeded weight, each rolled by a different number of
        row-groups (distinct bytes at every address, same statistics)."""
        codes, scales = self.host_weight(M, K, seed, group)
        out = []
        for c in range(n or self.rotate):
            cc = np.roll(codes.reshape(M // 16, -1), c, axis=0).reshape(-1)
            ss = np.roll(scales.reshape(M // 16, -1), c, axis=0).reshape(-1)
            out.append(self.pkg.PackedWeight(cc, ss, M, K, k64=(group == 64)))
        return out

    def time_loop(self, fn, iters, warmup=3):
        """Mean device time of fn(i) in milliseconds (CUDA events on the library stream)."""
        lib, ev = self.lib, self.events()
        for i in range(warmup):
            fn(i)
        lib.tq_sync()
        t0 = time.time()
        lib.tq_event_record(ev[0])
        for i in range(iters):
            fn(i)
        lib.tq_event_record(ev[1])
        lib.tq_sync()
        self.load_spans.append((t0, time.time()))
        return lib.tq_event_elapsed_ms(ev[0], ev[1]) / iters


def pinned_copy(lib, a):
    a = np.ascontiguousarray(a)
    p = lib.tq_host_alloc_pinned(a.nbytes)
    C.memmove(p, a.ctypes.data, a.nbytes)
    return p


def e2e_loop(ctx, case, iters, warmup=3):
    """The step through the C ABI with HOST buffers: every step uploads its fp32 activations
    from pinned host memory and reads its result back. Uploads and read-backs run on streams
    of their own (one per direction): step n+1's upload and step n's read-back overlap step
    n+1's kernels; tickets order the library stream behind a copy only where a buffer is about
    to be reused (two input and two output buffer sets). Returns seconds per step and the
    number of 32-bit words of the last host result that differ from a synchronous rerun."""
    lib = ctx.lib
    hx = pinned_copy(lib, case.x_host)
    nbx = case.x_host.nbytes
    hy = [lib.tq_host_alloc_pinned(case.out_bytes) for _ in range(2)]
    tickets, up = [-1, -1], [-1, -1]
    up[0] = lib.tq_h2d_overlapped(case.x_dev[0].ptr, hx, nbx)
    n = 0
    last = None

    single = getattr(case, "single_out", False)     # one output buffer: a read-back ends before
                                                    # the next step may rewrite it

    def one(i):
        nonlocal n, last
        b = 0 if single else n & 1
        if tickets[b] >= 0:
            lib.tq_stream_wait_copy(tickets[b])
        up[(n + 1) & 1] = lib.tq_h2d_overlapped(case.x_dev[(n + 1) & 1].ptr, hx, nbx)
        lib.tq_stream_wait_copy(up[n & 1])
        case.run(i, n & 1, b)
        tickets[b] = lib.tq_d2h_overlapped(hy[b], case.out_ptr(b), case.out_bytes)
        last = (i, n & 1, b)
        n += 1

    for i in range(warmup):
        one(i)
    lib.tq_sync()
    t0w = time.time()
    t0 = time.perf_counter()
    for i in range(iters):
        one(i)
    lib.tq_sync()
    dt = time.perf_counter() - t0
    ctx.load_spans.append((t0w, time.time()))
    i, xb, b = last
    got = np.ctypeslib.as_array(C.cast(hy[b], C.POINTER(C.c_uint32)), shape=(case.out_bytes // 4,)).copy()
    lib.tq_h2d(case.x_dev[xb].ptr, hx, nbx)
    case.run(i, xb, b)
    want = np.empty(case.out_bytes // 4, dtype=np.uint32)
    lib.tq_d2h(want.ctypes.data, case.out_ptr(b), case.out_bytes)
    diff = int(np.count_nonzero(got != want))
    lib.tq_host_free_pinned(hx)
    for p in hy:
        lib.tq_host_free_pinned(p)
    return dt / iters, diff


def cpu_sample(fn, units_per_pass, budget_s, unit, what):
    """Time-bounded CPU sample: fn() is one pass of the oracle over `units_per_pass` units."""
    from oracle import oracle as orc
    fn()
    passes, t0 = 0, time.perf_counter()
    while True:
        fn()
        passes += 1
        if time.perf_counter() - t0 >= budget_s:
            break
    dt = time.perf_counter() - t0
    return {"value": units_per_pass * passes / dt, "unit": unit, "cores": orc.num_threads(),
            "kind": "port", "sample": f"{passes} x ({what}) in {dt:.1f} s, OpenMP over all host threads"}


# ------------------------------------------------------------------------------------------
# cases
# ------------------------------------------------------------------------------------------
class DecodeGemm:
    """Chunk staging + batched GEMM over one or two weights that share the staged
    activations (xpu/src/decode.cpp:1856-1871): cfg2 (gate|up, K64) and the T >= 8 points of
    the down-projection sweep (cfg3)."""

    def __init__(self, ctx, name, M, count, K, group, T, mode, seed0, xgen, rows_note=""):
        self.ctx, self.name, self.M, self.count, self.K, self.group, self.T = ctx, name, M, count, K, group, T
        self.mode = mode                       # "pertoken" | "exact" (scale per (token, K32))
        lib, pkg = ctx.lib, ctx.pkg
        self.sets = list(zip(*[ctx.rotated(M, K, seed0 + j, group) for j in range(count)]))
        self.warr = [pkg.weight_array(list(s)) for s in self.sets]
        self.x_host = xgen()
        self.x_dev = [pkg.DevBuf.from_numpy(self.x_host), pkg.DevBuf.from_numpy(self.x_host)]
        nblk = K // 32 * T
        self.nblk = nblk
        self.aq, self.as_, self.asum, self.as_tok = (pkg.DevBuf(nblk * 32), pkg.DevBuf(nblk * 4),
                                                     pkg.DevBuf(nblk * 4), pkg.DevBuf(T * 4))
        self.out_bytes = count * T * M * 4
        self.y = [pkg.DevBuf(self.out_bytes) for _ in range(2)]
        self.yarr = [(C.c_void_p * count)(*[b.ptr + j * T * M * 4 for j in range(count)]) for b in self.y]
        self.weight_bytes = count * ctx.wl.weight_bytes(M, K, group)
        self.algo_bytes = self.weight_bytes + T * K + nblk * 8 + self.out_bytes
        self.ops = 2.0 * T * count * M * K
        self.rows_note = rows_note
        self.launches_per_step = 2

    def stage(self, xb):
        lib = self.ctx.lib
        if self.mode == "pertoken":
            lib.qwn_x_quantize_act_chunk_pertoken(self.x_dev[xb].ptr, self.K, self.T, self.aq.ptr,
                                                  self.as_.ptr, self.asum.ptr, self.as_tok.ptr)
        else:
            lib.qwn_x_quantize_act_chunk(self.x_dev[xb].ptr, self.K, self.T, self.aq.ptr, self.as_.ptr,
                                         self.asum.ptr)

    def kernel(self, i, b=0):
        lib = self.ctx.lib
        if self.mode == "pertoken":
            rc = lib.qwn_x_gemm_w4a8_fanout_pertoken(self.warr[i % len(self.warr)], self.yarr[b], self.count,
                                                     self.aq.ptr, self.as_tok.ptr, self.asum.ptr, self.T)
        else:
            rc = lib.qwn_x_gemm_w4a8_fanout(self.warr[i % len(self.warr)], self.yarr[b], self.count,
                                            self.aq.ptr, self.as_.ptr, self.asum.ptr, self.T, None, 0)
        assert rc == 0, rc

    def _oracle_gemm(self, codes, scales, rows, oq, os_, osm):
        from oracle import oracle as orc
        ksh = int(self.group == 64)
        if self.mode == "pertoken":
            S = self.ctx.lib.qwn_choose_pertoken_splits(self.M // 16, self.T // 8, self.K // 32, ksh)
            at = os_.reshape(self.K // 32, self.T)[0].copy()
            return orc.gemm_w4a8_pertoken(codes, scales, rows, self.K, ksh, oq, at, osm, self.T, splits=S)[1]
        if rows != self.M:
            S = self.ctx.lib.qwn_choose_gemm_splits(self.M // 16, self.T // 8, self.K // 32)
            return orc.gemm_w4a8(codes, scales, rows, self.K, ksh, oq, os_, osm, self.T, forced_splits=S)[1]
        return orc.gemm_w4a8(codes, scales, rows, self.K, ksh, oq, os_, osm, self.T, fma=1)[1]

    def run(self, i, xb, b):
        self.stage(xb)
        self.kernel(i, b)

    def out_ptr(self, b):
        return self.y[b].ptr

    def oracle_diff(self):
        """Words of weight copy 0's output that differ from the CPU oracle (fused variant)."""
        from oracle import oracle as orc
        lib = self.ctx.lib
        lib.tq_h2d(self.x_dev[0].ptr, self.x_host.ctypes.data, self.x_host.nbytes)
        self.run(0, 0, 0)
        lib.tq_sync()
        got = self.y[0].to_numpy(np.uint32).reshape(self.count, self.T, self.M)
        oq, os_, osm = orc.quantize_act_chunk(self.x_host, per_token=(self.mode == "pertoken"))
        diff = 0
        for j in range(self.count):
            codes, scales = self.ctx.host_weight(self.M, self.K, self.seed_of(j), self.group)
            want = self._oracle_gemm(codes, scales, self.M, oq, os_, osm)
            diff += int(np.count_nonzero(got[j] != want.view(np.uint32)))
        return diff

    def seed_of(self, j):
        return self._seed0 + j

    def cpu_pass_fn(self, rows):
        from oracle import oracle as orc
        oq, os_, osm = orc.quantize_act_chunk(self.x_host, per_token=(self.mode == "pertoken"))
        ws = [self.ctx.host_weight(self.M, self.K, self.seed_of(j), self.group) for j in range(self.count)]
        Kt = self.K // 32
        sg = Kt >> int(self.group == 64)

        def fn():
            orc.quantize_act_chunk(self.x_host, per_token=(self.mode == "pertoken"))
            for codes, scales in ws:
                self._oracle_gemm(codes[: rows * self.K // 2], scales[: rows * sg], rows, oq, os_, osm)
        return fn


class DecodeGemv:
    """Single-token staging + prepared GEMV: cfg1 and the T = 1 point of cfg3 (there the
    staging is the fused silu(gate) * up quantiser, xpu/src/decode.cpp:250-258)."""

    def __init__(self, ctx, name, M, K, group, mode, seed0, silu):
        self.ctx, self.name, self.M, self.K, self.group, self.mode, self.silu = ctx, name, M, K, group, mode, silu
        self.T = 1
        pkg = ctx.pkg
        self._seed0 = seed0
        self.ws = ctx.rotated(M, K, seed0, group)
        rng = np.random.Generator(np.random.Philox(key=seed0 + 1000))
        rows = 2 if silu else 1
        self.x_host = rng.standard_normal((rows, K), dtype=np.float32)
        self.x_dev = [pkg.DevBuf.from_numpy(self.x_host), pkg.DevBuf.from_numpy(self.x_host)]
        self.hidden = pkg.DevBuf(K * 4)
        self.out_bytes = M * 4
        self.y = [pkg.DevBuf(M * 4) for _ in range(2)]
        self.weight_bytes = ctx.wl.weight_bytes(M, K, group)
        self.algo_bytes = self.weight_bytes + K + (K // 32) * 8 + M * 4
        self.ops = 2.0 * M * K
        self.launches_per_step = 2

    def stage(self, xb):
        lib, x = self.ctx.lib, self.x_dev[xb].ptr
        if self.silu:
            f = lib.qwn_x_silu_mul_quant_pertoken if self.mode == "pertoken" else lib.qwn_x_silu_mul_quant
            f(self.hidden.ptr, x, x + self.K * 4, self.K)
        elif self.mode == "pertoken":
            lib.qwn_x_prepare_gemv_act_s8_pertoken(x, self.K)
        else:
            lib.qwn_x_prepare_gemv_act_s8(x, self.K)

    def kernel(self, i, b=0):
        rc = self.ctx.lib.qwn_x_gemv_w4a8_prepared(self.ws[i % len(self.ws)].ref, self.y[b].ptr, None)
        assert rc == 0, rc

    def run(self, i, xb, b):
        self.stage(xb)
        self.kernel(i, b)

    def out_ptr(self, b):
        return self.y[b].ptr

    def _oracle_act(self):
        from oracle import oracle as orc
        if self.silu:
            v = orc.silu_mul(self.x_host[0], self.x_host[1])
        else:
            v = self.x_host[0]
        if self.mode == "pertoken":
            q, s, _ = orc.quantize_act_chunk(v[None, :], per_token=True)
            sm = q.astype(np.int32).reshape(-1, 16).sum(axis=1).astype(np.int32)
        else:
            q, s, sm = orc.quantize_act_s8(v)
        return q, s, sm

    def oracle_diff(self):
        from oracle import oracle as orc
        lib = self.ctx.lib
        lib.tq_h2d(self.x_dev[0].ptr, self.x_host.ctypes.data, self.x_host.nbytes)
        self.run(0, 0, 0)
        lib.tq_sync()
        got = self.y[0].to_numpy(np.uint32)
        q, s, sm = self._oracle_act()
        codes, scales = self.ctx.host_weight(self.M, self.K, self._seed0, self.group)
        _, want = orc.gemv_w4a8(codes, scales, self.M, self.K, int(self.group == 64), q, s, sm, fma=1)
        return int(np.count_nonzero(got != want.view(np.uint32)))

    def cpu_pass_fn(self, rows):
        from oracle import oracle as orc
        q, s, sm = self._oracle_act()
        codes, scales = self.ctx.host_weight(self.M, self.K, self._seed0, self.group)

        def fn():
            self._oracle_act()
            orc.gemv_w4a8(codes, scales, self.M, self.K, int(self.group == 64), q, s, sm)
        return fn


class Prefill:
    """cfg4: packed prefill GEMM, 4096 tokens in four segments of 1024, 17408 x 5120, K64."""

    MODES = {"exact_fp32": "scale per (token, K32): the reference's arithmetic, fp32 out",
             "pertoken_fp32": "scale per token, fp32 out", "pertoken_bf16": "scale per token, bf16 out",
             "w4a4_fp32": "int4 activations per (token, K64) (x_gemm_w4a4), fp32 out"}

    def __init__(self, ctx, name, mode, shared=None, M=I_FF, T=4096):
        self.ctx, self.name, self.mode = ctx, name, mode
        self.M, self.K, self.T, self.group = M, H, T, 64
        pkg, lib = ctx.pkg, ctx.lib
        if shared is None:
            shared = {}
            shared["w"] = ctx.rotated(self.M, self.K, 11, 64, n=1)[0]
            shared["x_host"] = ctx.wl.activations_normal(self.T, self.K, seed=7)
            shared["x_dev"] = [pkg.DevBuf.from_numpy(shared["x_host"]) for _ in range(2)]
            n = self.K // 32 * self.T
            shared["stg"] = (pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(self.T * 4))
            shared["y"] = [pkg.DevBuf(self.T * self.M * 4) for _ in range(2)]
        self.shared = shared
        self.w, self.x_host, self.x_dev = shared["w"], shared["x_host"], shared["x_dev"]
        self.aq, self.as_, self.asum, self.as_tok = shared["stg"]
        self.y = shared["y"]
        self.out_bytes = self.T * self.M * (2 if mode.endswith("bf16") else 4)
        self.off = (C.c_int * 5)(0, self.T // 4, self.T // 2, 3 * self.T // 4, self.T)
        self.weight_bytes = ctx.wl.weight_bytes(self.M, self.K, 64)
        self.ops = 2.0 * self.T * self.M * self.K
        self.launches_per_step = 5      # staging, activation image pre-pass, weight image pre-pass, the GEMM
                                        # kernel without and with the zero-point term (the one the weight does
                                        # not need returns at once)

    def stage(self, xb):
        lib, x = self.ctx.lib, self.x_dev[xb].ptr
        if self.mode == "exact_fp32":
            lib.qwn_x_quantize_act_chunk(x, self.K, self.T, self.aq.ptr, self.as_.ptr, self.asum.ptr)
        elif self.mode == "w4a4_fp32":
            lib.qwn_x_quantize_act_chunk_s4(x, self.K, self.T, self.aq.ptr, self.as_.ptr, self.asum.ptr)
        else:
            lib.qwn_x_quantize_act_chunk_pertoken(x, self.K, self.T, self.aq.ptr, self.as_.ptr,
                                                  self.asum.ptr, self.as_tok.ptr)

    def kernel(self, i, b=0):
        lib = self.ctx.lib
        if self.mode == "exact_fp32":
            rc = lib.qwn_x_gemm_w4a8(self.w.ref, self.aq.ptr, self.as_.ptr, self.asum.ptr, self.y[b].ptr,
                                     self.T, self.off, 4)
        elif self.mode == "w4a4_fp32":
            rc = lib.qwn_x_gemm_w4a4(self.w.ref, self.aq.ptr, self.as_.ptr, self.asum.ptr, self.y[b].ptr,
                                     self.T)
        else:
            rc = lib.qwn_x_gemm_w4a8_pertoken(self.w.ref, self.aq.ptr, self.as_tok.ptr, self.asum.ptr,
                                              self.y[b].ptr, self.T, int(self.mode.endswith("bf16")))
        assert rc == 0, rc

    def run(self, i, xb, b):
        self.stage(xb)
        self.kernel(i, b)

    def out_ptr(self, b):
        return self.y[b].ptr

    def cpu_pass_fn(self, rows, tokens=256):
        """A bounded sample: `rows` weight rows x the first `tokens` tokens."""
        from oracle import oracle as orc
        x = self.x_host[:tokens]
        codes, scales = self.ctx.host_weight(self.M, self.K, 11, 64)
        c, s = codes[: rows * self.K // 2], scales[: rows * (self.K // 64)]
        if self.mode == "w4a4_fp32":
            q = orc.quantize_act_chunk_s4(x)
            return lambda: (orc.quantize_act_chunk_s4(x), orc.gemm_w4a4(c, s, rows, self.K, *q, tokens))
        if self.mode == "exact_fp32":
            q = orc.quantize_act_chunk(x)
            return lambda: (orc.quantize_act_chunk(x), orc.gemm_w4a8(c, s, rows, self.K, 1, *q, tokens))
        oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
        at = os_.reshape(self.K // 32, tokens)[0].copy()
        return lambda: (orc.quantize_act_chunk(x, per_token=True),
                        orc.gemm_w4a8_pertoken(c, s, rows, self.K, 1, oq, at, osm, tokens))


class Stack:
    """cfg5: 64 layers x four projections at T = 8, group-32 weights, per-token int8
    activations. Per layer: RMSNorm of the incoming rows (keeps values O(1) through 64
    layers), 5120->10240, 10240->5120, fused 5120->gate|up, silu(gate)*up, 17408->5120; every
    projection is staging + GEMM through the C ABI (the batched path of
    xpu/src/decode.cpp:1856-1871). Layers use distinct weights: five seeded base matrices,
    rolled by a different number of row-groups per layer. With tp > 1 every projection is a
    column shard (x_w4_shard mode 0; gate and up sharded alike, so silu*mul stays local), each
    shard keeps the split count of the whole weight (bit-identical to tp = 1), the projections
    write their output columns into every rank's copy of the next activation matrix, and the
    staging / norm kernel that reads the matrix carries the exchange point."""

    LAYERS = 64

    def __init__(self, ctx, layers=None, tp=1, rank=0, comm=None):
        self.ctx, self.tp, self.rank, self.comm = ctx, tp, rank, comm
        self.L = layers or self.LAYERS
        self.T = 8
        self.name, self.mode = "cfg5", "pertoken"
        pkg, lib, wl = ctx.pkg, ctx.lib, ctx.wl
        shapes = [(QKV, H, 41), (H, QKV, 42), (I_FF, H, 43), (I_FF, H, 44), (H, I_FF, 45)]
        base = [ctx.rotated(M, K, seed, 32, n=1)[0] for M, K, seed in shapes]
        self.shapes = shapes
        self.layers = []
        for l in range(self.L):
            ws = []
            for (M, K, _), b in zip(shapes, base):
                ws.append(self._rolled_shard(b, M, K, (l * 37) % (M // 16)))
            self.layers.append(ws)
        for b in base:
            b.codes.free()
            b.scales.free()
        T = self.T
        self.x_host = wl.activations_normal(T, H, seed=5)
        self.x_dev = [pkg.DevBuf.from_numpy(self.x_host), pkg.DevBuf.from_numpy(self.x_host)]
        self.norm_w = pkg.DevBuf.from_numpy(np.zeros(H, dtype=np.uint16))     # (1 + 0) weights
        nb = I_FF // 32 * T
        self.aq, self.as_, self.asum, self.as_tok = (pkg.DevBuf(nb * 32), pkg.DevBuf(nb * 4),
                                                     pkg.DevBuf(nb * 4), pkg.DevBuf(T * 4))
        self.xn = pkg.DevBuf(T * H * 4)
        self.gu = pkg.DevBuf(2 * T * (I_FF // tp) * 4)          # this rank's gate and up columns
        self.out_bytes = T * H * 4
        # activation matrices between the projections (symmetric buffers when tp > 1)
        self.y1, self.y2, self.h, self.y4 = (pkg.DevBuf(T * QKV * 4), pkg.DevBuf(T * H * 4),
                                             pkg.DevBuf(T * I_FF * 4), pkg.DevBuf(T * H * 4))
        self.sym = [self.y1, self.y2, self.h, self.y4]
        if tp > 1:
            comm.register(self.sym)
        else:
            # a world of one: the same calls, the exchange points wait for this rank's own flag
            self.flags = pkg.DevBuf(4)
            one = (C.c_void_p * 1)
            assert lib.tq_comm_gather_setup(one(self.y1.ptr), one(self.flags.ptr), 1, 0) == 0
            for i, b in enumerate(self.sym):
                assert lib.tq_comm_sym_register(i, one(b.ptr)) == 0
        self.weight_bytes = self.L * sum(wl.weight_bytes(M, K, 32) for M, K, _ in shapes)
        self.algo_bytes = self.weight_bytes
        # per layer: norm+staging, 4 GEMMs, 2 stagings, silu*mul+staging (tp 1: one launch; tp > 1: the
        # scatter and the staging behind the exchange point)
        self.launches_per_step = self.L * (8 if tp == 1 else 9) + (2 if tp > 1 else 0)
        self.single_out = True
        self.graph = None

    def _rolled_shard(self, base, M, K, shift):
        """Device copy of `base` rolled by `shift` row-groups (two runs per array); with
        tp > 1 only this rank's column shard of it is kept."""
        pkg, lib = self.ctx.pkg, self.ctx.lib
        cb, sb = (K // 32) * 256, (K // 32) * 32
        codes, scales = pkg.DevBuf(M // 16 * cb), pkg.DevBuf(M // 16 * sb)
        g = M // 16
        for dst, src, rb in ((codes, base.codes, cb), (scales, base.scales, sb)):
            lib.tq_d2d_async(dst.ptr + shift * rb, src.ptr, (g - shift) * rb)
            if shift:
                lib.tq_d2d_async(dst.ptr, src.ptr + (g - shift) * rb, shift * rb)
        w = pkg.PackedWeight.__new__(pkg.PackedWeight)
        w.codes, w.scales = codes, scales
        w.rec = pkg.TqWeight()
        w.rec.M, w.rec.K, w.rec.Mt, w.rec.Kt = M, K, M // 16, K // 32
        w.rec.d_s4, w.rec.d_s4_scale, w.rec.s4_ready = codes.ptr, scales.ptr, 1
        lib.tq_sync()
        if self.tp > 1:
            sh = pkg.TqWeight()
            assert lib.qwn_x_w4_shard(C.byref(sh), w.ref, self.rank, self.tp, 0, None, 0) == 0
            codes.free()
            scales.free()
            w.codes = w.scales = None
            w.rec = sh
        return w

    def _gemm(self, ws, full_rows, slot, col_off, ld, ys=None):
        lib, pkg, T = self.ctx.lib, self.ctx.pkg, self.T
        n = len(ws)
        warr = (C.POINTER(pkg.TqWeight) * n)(*[C.pointer(w.rec) for w in ws])
        fr = (C.c_int * n)(*full_rows)
        co = (C.c_size_t * n)(*col_off) if col_off is not None else None
        ya = (C.c_void_p * n)(*ys) if ys is not None else None
        rc = lib.qwn_x_gemm_w4a8_fanout_tp(warr, n, self.aq.ptr, None, self.as_tok.ptr, self.asum.ptr, T, fr,
                                           ya, slot, co, ld)
        assert rc == 0, rc

    def _stage(self, x_ptr, K, sync):
        lib, T = self.ctx.lib, self.T
        sync = sync and self.tp > 1              # one GPU: nothing to wait for
        f = lib.qwn_x_quantize_act_chunk_pertoken_sync if sync else lib.qwn_x_quantize_act_chunk_pertoken
        f(x_ptr, K, T, self.aq.ptr, self.as_.ptr, self.asum.ptr, self.as_tok.ptr)

    def _issue(self, x_ptr):
        """One pass: 64 layers, then the exchange point that makes the last output complete on
        every rank, then the step base moves on (so the pass can be replayed)."""
        lib, T, tp, r = self.ctx.lib, self.T, self.tp, self.rank
        n_i = I_FF // tp
        for l, (w1, w2, wg, wu, wd) in enumerate(self.layers):
            # norm and per-token staging in one launch (at tp > 1 it carries the exchange point
            # behind the previous layer's last projection)
            lib.qwn_x_rmsnorm_quant_chunk_pertoken(self.xn.ptr, x_ptr if l == 0 else self.y4.ptr, self.norm_w.ptr,
                                                   H, T, 1e-6, self.aq.ptr, self.as_.ptr, self.asum.ptr,
                                                   self.as_tok.ptr, int(l > 0 and tp > 1))
            self._gemm([w1], [QKV], 0, [r * (QKV // tp)], QKV)
            self._stage(self.y1.ptr, QKV, True)
            self._gemm([w2], [H], 1, [r * (H // tp)], H)
            self._stage(self.y2.ptr, H, True)
            self._gemm([wg, wu], [I_FF, I_FF], -1, None, 0, ys=[self.gu.ptr, self.gu.ptr + T * n_i * 4])
            if tp == 1:
                lib.qwn_x_silu_mul_quant_chunk_pertoken(self.h.ptr, self.gu.ptr, self.gu.ptr + T * n_i * 4, I_FF, T,
                                                        self.aq.ptr, self.as_.ptr, self.asum.ptr, self.as_tok.ptr)
            else:
                assert lib.qwn_x_silu_mul_scatter(self.gu.ptr, self.gu.ptr + T * n_i * 4, T, n_i, 2, r * n_i,
                                                  I_FF) == 0
                self._stage(self.h.ptr, I_FF, True)
            self._gemm([wd], [H], 3, [r * (H // tp)], H)
        if tp > 1:
            assert lib.tq_comm_exchange_sync() == 0
            assert lib.tq_comm_exchange_advance() == 0

    def capture(self):
        """One CUDA graph per input buffer (`launches_per_step` kernels per replay)."""
        lib = self.ctx.lib
        self._issue(self.x_dev[0].ptr)        # warm: all scratch allocated
        lib.tq_sync()
        self.graph = {}
        for xb in range(2):
            assert lib.tq_graph_capture_begin() == 0
            self._issue(self.x_dev[xb].ptr)
            g = lib.tq_graph_capture_end()
            assert g, "graph capture failed"
            self.graph[xb] = g

    def stage(self, xb):
        pass

    def run(self, i, xb, b):
        if self.graph:
            self.ctx.lib.tq_graph_launch(self.graph[xb])
        else:
            self._issue(self.x_dev[xb].ptr)

    def kernel(self, i, b=0):
        self.run(i, 0, b)

    def out_ptr(self, b):
        return self.y4.ptr

    def cpu_pass_fn(self):
        """One projection of each kind of layer 0 on the oracle (1/64 of a step)."""
        from oracle import oracle as orc
        T = self.T
        ws = [self.ctx.host_weight(M, K, seed, 32) for M, K, seed in self.shapes]
        xs = {K: self.ctx.wl.activations_normal(T, K, seed=K) for K in (H, QKV, I_FF)}
        qs = {K: orc.quantize_act_chunk(x, per_token=True) for K, x in xs.items()}

        def fn():
            for (M, K, _), (codes, scales) in zip(self.shapes, ws):
                orc.quantize_act_chunk(xs[K], per_token=True)
                oq, os_, osm = qs[K]
                S = orc.choose_pertoken_splits(M // 16, T // 8, K // 32, 0)
                orc.gemm_w4a8_pertoken(codes, scales, M, K, 0, oq, os_.reshape(K // 32, T)[0].copy(), osm, T,
                                       splits=S)
        return fn


# ------------------------------------------------------------------------------------------
# records
# ------------------------------------------------------------------------------------------
def hbm_record(ctx, case, kernel_name, kernel_ms):
    ach = case.algo_bytes / (kernel_ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": ach, "peak": ctx.peak_hbm, "unit": "GB/s", "frac": ach / ctx.peak_hbm,
            "peak_source": f"{ctx.peak_kind} copy bandwidth", "kernel": kernel_name,
            "us_per_launch": kernel_ms * 1e3, "algorithmic_bytes_per_launch": int(case.algo_bytes),
            "weight_GBps": case.weight_bytes / (kernel_ms * 1e-3) / 1e9, "traffic": None}


def tensor_record(ctx, case, kernel_name, kernel_ms, int8_peak):
    tops = case.ops / (kernel_ms * 1e-3) / 1e12
    peak = int8_peak or NOMINAL_INT8_TOPS
    return {"bound": "tensor", "achieved": tops, "peak": peak, "unit": "TOP/s (int8)", "frac": tops / peak,
            "peak_source": ("tcgen05 kind::i8 issue peak measured in this run" if int8_peak
                            else "nominal dense int8"),
            "frac_of_nominal_4500": tops / NOMINAL_INT8_TOPS,
            "frac_of_2x_measured_bf16": tops / (2.0 * ctx.peak_bf16) if ctx.peak_bf16 else None,
            "kernel": kernel_name, "us_per_launch": kernel_ms * 1e3, "algorithmic_ops_per_launch": case.ops,
            "traffic": None}


def run_case(ctx, case, kernel_name, iters, e2e_iters, cpu_budget, cpu_rows, bound="hbm", int8_peak=None,
             check=True, cpu_units=None, cpu_what=None, cpu_fn=None):
    lib = ctx.lib
    rec = {"name": case.name, "T": case.T, "mode": getattr(case, "mode", None)}
    if check and hasattr(case, "oracle_diff"):
        rec["oracle_words_differing"] = case.oracle_diff()
    step_ms = ctx.time_loop(lambda i: case.run(i, 0, 0), iters)
    case.stage(0)
    k_ms = ctx.time_loop(lambda i: case.kernel(i), iters)
    rec["us"] = step_ms * 1e3
    rec["launches_per_step"] = case.launches_per_step
    rec["roofline"] = (hbm_record(ctx, case, kernel_name, k_ms) if bound == "hbm"
                       else tensor_record(ctx, case, kernel_name, k_ms, int8_peak))
    s, diff = e2e_loop(ctx, case, e2e_iters)
    if bound == "hbm":
        val, unit = case.weight_bytes / s / 1e9, UNIT
        rec["value"], rec["unit"] = case.weight_bytes / (step_ms * 1e-3) / 1e9, UNIT
    else:
        val, unit = case.ops / s / 1e12, "TOP/s (int8)"
        rec["value"], rec["unit"] = case.ops / (step_ms * 1e-3) / 1e12, unit
    rec["e2e"] = {"value": val, "unit": unit, "us_per_step": s * 1e6, "h2d_bytes_per_step": int(case.x_host.nbytes),
                  "d2h_bytes_per_step": int(case.out_bytes), "steps": e2e_iters,
                  "last_result_words_differing": diff}
    if cpu_budget > 0:
        fn = cpu_fn or case.cpu_pass_fn(cpu_rows)
        rec["cpu_baseline"] = cpu_sample(fn, cpu_units, cpu_budget, unit, cpu_what)
    return rec


def int8_peak_tops(ctx):
    """tcgen05 kind::i8 issue peak (TMEM accumulate only, no epilogue), if the library has it."""
    lib = ctx.lib
    if not hasattr(lib, "qwn_tc_int8_peak"):
        return None
    lib.qwn_tc_int8_peak.restype = C.c_double
    lib.qwn_tc_int8_peak.argtypes = [C.c_int]
    t0 = time.time()
    v = float(lib.qwn_tc_int8_peak(4000))
    ctx.load_spans.append((t0, time.time()))
    return v if v > 0 else None


def build_cases(ctx, which):
    """name -> (case, kernel name, bound). Built lazily: only what `which` selects."""
    wl = ctx.wl
    out = {}

    def want(n):
        return which is None or n in which

    if want("cfg2"):
        c = DecodeGemm(ctx, "cfg2", I_FF, 2, H, 64, 8, "pertoken", 11,
                       lambda: wl.activations_normal(8, H, seed=5, outlier_frac=0.01))
        c._seed0 = 11
        out["cfg2"] = (c, "gemm_w4a8_ring_kernel", "hbm")
    if want("cfg2_exact"):
        c = DecodeGemm(ctx, "cfg2_exact", I_FF, 2, H, 64, 8, "exact", 11,
                       lambda: wl.activations_normal(8, H, seed=5, outlier_frac=0.01))
        c._seed0 = 11
        out["cfg2_exact"] = (c, "gemm_w4a8_ring_kernel", "hbm")
    if want("cfg1"):
        out["cfg1"] = (DecodeGemv(ctx, "cfg1", I_FF, H, 32, "pertoken", 21, silu=False), "gemv_w4a8_kernel", "hbm")
    if want("cfg3_T1"):
        out["cfg3_T1"] = (DecodeGemv(ctx, "cfg3_T1", H, I_FF, 32, "pertoken", 23, silu=True),
                          "gemv_w4a8_kernel", "hbm")
    for T in (8, 16, 32, 64):
        n = f"cfg3_T{T}"
        if want(n):
            def xg(T=T):
                rng = np.random.Generator(np.random.Philox(key=31 + T))
                g = rng.standard_normal((T, I_FF))
                u = rng.standard_normal((T, I_FF))
                return (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
            # per-token scales on the ring kernel, a warp carrying all of the call's tokens
            c = DecodeGemm(ctx, n, H, 1, I_FF, 32, T, "pertoken", 23, xg)
            c._seed0 = 23
            out[n] = (c, "gemm_w4a8_ring_kernel", "hbm")
    shared = None
    for mode in Prefill.MODES:
        n = f"cfg4_{mode}"
        if want(n):
            c = Prefill(ctx, n, mode, shared)
            shared = c.shared
            out[n] = (c, "gemm_w4a8_tc_kernel", "tensor")
    # profiler targets only: the same kernel on 4736 x 5120, 1024 tokens (296 tiles, two per SM)
    for mode in Prefill.MODES:
        n = f"prefill_small_{mode}"
        if which is not None and n in which:
            out[n] = (Prefill(ctx, n, mode, None, M=4736, T=1024), "gemm_w4a8_tc_kernel", "tensor")
    return out


# ------------------------------------------------------------------------------------------
# reference arm: the CPU oracle on the host cores
# ------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """The reference's scalar projection semantics (the CPU oracle; the reference's SYCL
    sources cannot be built without Intel's toolchain) on the host cores, on the workload
    the GPU arm runs at this N."""
    if rank != 0:
        return
    from oracle import oracle as orc
    orc.set_num_threads(host_threads())
    wl = importlib.import_module("knivesysl-xe_b200.workloads")
    T = 8
    if world == 1:
        K, M, group = H, I_FF, 64
        host_w = [wl.make_weight_w4(M, K, seed=11 + i, group=group) for i in range(2)]
        x = wl.activations_normal(T, K, seed=5, outlier_frac=0.01)
        aq, as_, asum = orc.quantize_act_chunk(x, per_token=True)

        def cpu_pass(rows):
            orc.quantize_act_chunk(x, per_token=True)
            for codes, scales in host_w:
                orc.gemm_w4a8(codes[: rows * K // 2], scales[: rows * (K // group)], rows, K, 1, aq, as_, asum, T)
        full_rows, per_row_bytes, workload = M, 2 * (K // 2 + (K // group) * 2), WORKLOAD_CFG2
        what = "rows of gate and up per step"
    else:
        shapes = [(QKV, H, 41), (H, QKV, 42), (I_FF, H, 43), (I_FF, H, 44), (H, I_FF, 45)]
        ws = [wl.make_weight_w4(M, K, seed=s, group=32) for M, K, s in shapes]
        xs = {K: wl.activations_normal(T, K, seed=K) for K in (H, QKV, I_FF)}
        qs = {K: orc.quantize_act_chunk(v, per_token=True) for K, v in xs.items()}

        def cpu_pass(frac_rows):
            # frac_rows of 17408 scales every projection of one layer by the same fraction
            for (M, K, _), (codes, scales) in zip(shapes, ws):
                rows = max(16, M * frac_rows // I_FF // 16 * 16)
                orc.quantize_act_chunk(xs[K], per_token=True)
                orc.gemm_w4a8(codes[: rows * K // 2], scales[: rows * (K // 32)], rows, K, 0, *qs[K], T)
        full_rows = I_FF
        per_row_bytes = sum(wl.weight_bytes(M, K, 32) for M, K, _ in shapes) / I_FF
        workload = WORKLOAD_CFG5
        what = "of one layer's five matrices per step (1 of 64 layers)"
    t0 = time.perf_counter()
    cpu_pass(1088)
    t_probe = (time.perf_counter() - t0) * (full_rows / 1088)
    max_seconds = 150.0
    total = args.steps + args.warmup
    rows = full_rows
    if t_probe * total > max_seconds:
        rows = max(16, int(full_rows * max_seconds / (t_probe * total)) // 16 * 16)
    for _ in range(args.warmup):
        cpu_pass(rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(rows)
    dt = time.perf_counter() - t0
    val = per_row_bytes * rows * args.steps / dt / 1e9
    sample = f"{rows} of {full_rows} {what}, T={T}"
    out = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
        "dtype": "s8xs4->s32, fp32 out", "data": "synthetic",
        "config": {"workload": workload},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------
# N = 1
# ------------------------------------------------------------------------------------------
PER_CONFIG = ["cfg1", "cfg2_exact", "cfg3_T1", "cfg3_T8", "cfg3_T16", "cfg3_T32", "cfg3_T64",
              "cfg4_exact_fp32", "cfg4_pertoken_fp32", "cfg4_pertoken_bf16", "cfg4_w4a4_fp32"]


def run_single(args):
    ctx = Ctx(args.rotate)
    lib = ctx.lib
    assert lib.tq_set_device(0) == 0
    sampler = ClockSampler(0)
    cpu_on = not args.no_cpu_baseline
    if cpu_on:
        from oracle import oracle as orc
        orc.set_num_threads(host_threads())

    if args.case:
        # profiler target: L launches of one case's dominant kernel, nothing else timed
        if args.case == "cfg5":
            case = Stack(ctx, layers=args.layers)
            case.run(0, 0, 0)
            lib.tq_sync()
            for i in range(args.launches):
                case.run(i, 0, 0)
        else:
            case, kname, _ = build_cases(ctx, {args.case})[args.case]
            case.stage(0)
            lib.tq_sync()
            for i in range(args.launches):
                case.kernel(i)
        lib.tq_sync()
        print(json.dumps({"case": args.case, "launches": args.launches, "device_error": lib.tq_last_error()}))
        return

    # ---- headline: cfg2 -------------------------------------------------------------------
    head, head_kernel, _ = build_cases(ctx, {"cfg2"})["cfg2"]
    oracle_diff = head.oracle_diff()
    for i in range(args.warmup):
        head.run(i, 0, 0)
    ms = ctx.time_loop(lambda i: head.run(i, 0, 0), args.steps, warmup=0)
    value = head.weight_bytes / (ms * 1e-3) / 1e9
    head.stage(0)
    k_ms = ctx.time_loop(lambda i: head.kernel(i), max(args.steps, 200), warmup=args.warmup)
    roof = hbm_record(ctx, head, head_kernel, k_ms)
    if NCU_TRAFFIC["bytes_per_launch"]:
        roof["traffic"] = NCU_TRAFFIC["bytes_per_launch"]
        roof["traffic_source"] = NCU_TRAFFIC["capture"]
    e_iters = max(min(args.steps, 2000), 50)
    e_s, e_diff = e2e_loop(ctx, head, e_iters, warmup=args.warmup)
    cpu = None
    if cpu_on:
        cpu = cpu_sample(head.cpu_pass_fn(I_FF), head.weight_bytes / 1e9, 10.0, UNIT, "full pass of cfg2")
    head_keep = head          # keep the buffers alive until the line is printed

    # ---- every other configuration ------------------------------------------------------
    per = []
    peak_i8 = int8_peak_tops(ctx)
    if not args.headline_only:
        for name in PER_CONFIG:
            cases = build_cases(ctx, {name})
            case, kname, bound = cases[name]
            it = 300 if bound == "hbm" else 6
            eit = 300 if bound == "hbm" else 4
            if bound == "hbm":
                rows = case.M if case.T <= 8 else max(16, case.M * 8 // case.T // 16 * 16)
                units = case.weight_bytes * rows / case.M / 1e9
                what = f"{rows} of {case.M} rows, T={case.T}"
                rec = run_case(ctx, case, kname, it, eit, 2.0 if cpu_on else 0, rows, cpu_units=units,
                               cpu_what=what)
            else:
                rows, toks = 256, 256
                units = 2.0 * toks * rows * case.K / 1e12
                rec = run_case(ctx, case, kname, it, eit, 2.0 if cpu_on else 0, rows, bound="tensor",
                               int8_peak=peak_i8, check=False, cpu_units=units,
                               cpu_what=f"{rows} rows x {toks} tokens")
            per.append(rec)
            del case, cases
        # cfg5 on one GPU
        st = Stack(ctx, layers=args.layers)
        st.capture()
        st_ms = ctx.time_loop(lambda i: st.run(i, 0, 0), 20)
        s5, d5 = e2e_loop(ctx, st, 20)
        rec5 = {"name": "cfg5_tp1", "T": 8, "mode": "pertoken", "layers": st.L, "us": st_ms * 1e3,
                "launches_per_step": st.launches_per_step, "value": st.weight_bytes / (st_ms * 1e-3) / 1e9,
                "unit": UNIT,
                "roofline": {"bound": "hbm", "achieved": st.weight_bytes / (st_ms * 1e-3) / 1e9,
                             "peak": ctx.peak_hbm, "unit": "GB/s",
                             "frac": st.weight_bytes / (st_ms * 1e-3) / 1e9 / ctx.peak_hbm,
                             "peak_source": f"{ctx.peak_kind} copy bandwidth",
                             "kernel": "whole step (CUDA graph: norm+staging, 4 GEMMs, 2 stagings, silu*mul+staging per layer)",
                             "algorithmic_bytes_per_launch": int(st.weight_bytes), "traffic": None},
                "e2e": {"value": st.weight_bytes / s5 / 1e9, "unit": UNIT, "us_per_step": s5 * 1e6,
                        "h2d_bytes_per_step": int(st.x_host.nbytes), "d2h_bytes_per_step": int(st.out_bytes),
                        "steps": 20, "last_result_words_differing": d5}}
        if cpu_on:
            rec5["cpu_baseline"] = cpu_sample(st.cpu_pass_fn(), st.weight_bytes / st.L / 1e9, 3.0, UNIT,
                                              "the five matrices of one layer")
        per.append(rec5)
        del st

    clocks = sampler.stop(ctx.load_spans)
    prefill = {r["name"]: r["roofline"]["achieved"] for r in per if r["name"].startswith("cfg4")}
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "s8xs4->s32, fp32 out", "data": "synthetic",
        "config": {"workload": WORKLOAD_CFG2, "parallelism": "column shard tp1",
                   "l2": f"inputs larger than L2: {args.rotate} rotating weight copies, "
                         f"{args.rotate * head.weight_bytes / 1e6:.0f} MB",
                   "step": "per-token staging (1 launch) + fused gate|up GEMM"},
        "oracle_words_differing": oracle_diff,
        "roofline": roof,
        "e2e": {"value": head.weight_bytes / e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": int(head.x_host.nbytes),
                "d2h_bytes_per_step": int(head.out_bytes), "steps": e_iters, "us_per_step": e_s * 1e6,
                "last_result_words_differing": e_diff},
        "gpu_launches": head.launches_per_step * args.steps,
        "clocks": clocks,
        "cpu_baseline": cpu,
        "prefill_int8_TOPS": prefill.get("cfg4_pertoken_fp32"),
        "prefill_int8_TOPS_by_mode": prefill,
        "int8_peak": {"measured_tcgen05_kind_i8_TOPS": peak_i8, "nominal_TOPS": NOMINAL_INT8_TOPS},
        "per_config": per,
        "device_error": lib.tq_last_error(),
    }
    del head_keep
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rotate", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true", help="skip the per_config records")
    ap.add_argument("--case", default=None, help="run only this case's dominant kernel (profiler target)")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None, help="layers of the cfg5 stack (default 64)")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world == 1:
        run_single(args)
        return
    multi = importlib.import_module("bench_multi") if os.path.exists(os.path.join(ROOT, "bench_multi.py")) else None
    if multi is None:
        raise SystemExit("multi-GPU bench module missing")
    multi.run(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
