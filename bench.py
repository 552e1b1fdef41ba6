#!/usr/bin/env python
"""Benchmark of the W4A8 projection path.

Workload ("cfg2"): batched decode fused gate+up projection, K64 scale tier, T = 8 tokens,
K = 5120, N = 2 x 17408; seeded N(0, 0.02) weights symmetric-quantised to int4; N(0, 1)
activations with 1% of channels scaled x20, quantised to int8 per token. One step = one pass:
per-token activation staging (1 launch) + ONE fused gate|up GEMM launch over a weight copy
that rotates through `rotate` distinct copies (> L2 in total), so weights come from HBM.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 (torchrun, one rank per GPU): gate and up are column-sharded (x_w4_shard), each rank
computes its slice of every step and the slices are all-gathered over NCCL ("strong").
Prints ONE JSON line on rank 0.
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

T, K, N_EACH, GROUP = 8, 5120, 17408, 64
METRIC = "decode_gemv_weight_GBps"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM launch of this workload, from the
# ncu capture summarised in profiles/ (None until a capture exists)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 100_617_216


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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

    def stop(self, t0: float, t1: float):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            if ts < t0 or ts > t1 + 0.06:
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


def cpu_pass(orc, host_w, aq, as_, asum, rows=None):
    """One pass of the workload on the CPU oracle (all OpenMP threads); rows limits each
    matrix to its first `rows` output rows."""
    for codes, scales in host_w:
        M = N_EACH if rows is None else rows
        orc.gemm_w4a8(codes[: M * K // 2], scales[: M * (K // GROUP)], M, K, 1, aq, as_, asum, T)


def run_reference(args, rank):
    """The reference's scalar projection semantics (the CPU oracle; the reference's SYCL
    sources cannot be built without Intel's toolchain) on the host cores."""
    if rank != 0:
        return
    from oracle import oracle as orc
    # all host threads, also under torchrun (which exports OMP_NUM_THREADS=1 to its workers)
    orc.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity")
                        else (os.cpu_count() or 1))
    wl = importlib.import_module("knivesysl-xe_b200.workloads")
    host_w = [wl.make_weight_w4(N_EACH, K, seed=11 + i, group=GROUP) for i in range(2)]
    x = wl.activations_normal(T, K, seed=5, outlier_frac=0.01)
    aq, as_, asum = orc.quantize_act_chunk(x, per_token=True)
    t0 = time.perf_counter()
    cpu_pass(orc, host_w, aq, as_, asum, rows=1088)
    t_probe = (time.perf_counter() - t0) * 16.0
    max_seconds = 150.0
    frac_rows = N_EACH
    total = args.steps + args.warmup
    if t_probe * total > max_seconds:
        frac_rows = max(16, int(N_EACH * max_seconds / (t_probe * total)) // 16 * 16)
    for _ in range(args.warmup):
        orc.quantize_act_chunk(x, per_token=True)
        cpu_pass(orc, host_w, aq, as_, asum, rows=frac_rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.quantize_act_chunk(x, per_token=True)
        cpu_pass(orc, host_w, aq, as_, asum, rows=frac_rows)
    dt = time.perf_counter() - t0
    wl_bytes = 2 * wl.weight_bytes(frac_rows, K, GROUP)
    val = wl_bytes * args.steps / dt / 1e9
    sample = f"{frac_rows} of {N_EACH} rows of gate and up per step, T={T}, K={K}"
    out = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8xs4->s32",
        "data": "synthetic",
        "config": {"workload": "cfg2: fused gate+up, K64 tier, T=8, K=5120, N=2x17408 (CPU oracle)"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rotate", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N > 1: every rank holds a cfg2-sized column shard of an N-times wider "
                         "projection (weak, default), or cfg2 itself is cut into N shards (strong)")
    ap.add_argument("--quantiser", default="staged", choices=["fused", "staged"],
                    help="activation quantiser as its own launch before the GEMM (the reference's "
                         "two calls; default, faster here), or in the GEMM's prologue (one launch: "
                         "every CTA then reads the same fp32 rows from L2 at once, which costs more "
                         "than the staging launch it saves)")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: all-gather by peer stores from the GEMM epilogue (fused) or by NCCL")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        run_reference(args, rank)
        return

    pkg = importlib.import_module("knivesysl-xe_b200")
    wl = importlib.import_module("knivesysl-xe_b200.workloads")
    lib = pkg.load()                      # raises if the CUDA library is missing
    assert lib.tq_set_device(local_rank) == 0
    dist = None
    if world > 1:
        import torch.distributed as dist   # control plane only: barrier and max-over-ranks
        dist.init_process_group("gloo", rank=rank, world_size=world)
        idbuf = (C.c_char * 128)()
        if rank == 0:
            assert lib.tq_comm_unique_id(idbuf) == 0
        obj = [bytes(idbuf.raw)]
        dist.broadcast_object_list(obj, src=0)
        idbuf = C.create_string_buffer(obj[0], 128)
        assert lib.tq_comm_init(idbuf, rank, world) == 0

    # ---- inputs (same seeds on every rank; a rank keeps only its column shard) ----------
    weak = world > 1 and args.scaling == "weak"
    # weak: this rank's shard is a whole cfg2-sized weight pair of its own (seeded by rank), i.e.
    # the column shard of a projection world times as wide; strong: cfg2 cut with x_w4_shard
    host_w = [wl.make_weight_w4(N_EACH, K, seed=11 + i + (100 * rank if weak else 0), group=GROUP)
              for i in range(2)]
    n_shard = N_EACH if weak else N_EACH // world
    copies = []                      # rotate x [gate, up] PackedWeight (this rank's shard)
    for c in range(args.rotate):
        pair = []
        for codes, scales in host_w:
            cc = np.roll(codes.reshape(N_EACH // 16, -1), c, axis=0).reshape(-1)
            ss = np.roll(scales.reshape(N_EACH // 16, -1), c, axis=0).reshape(-1)
            full = pkg.PackedWeight(cc, ss, N_EACH, K, k64=True)
            if world > 1 and not weak:
                sh = pkg.TqWeight()
                assert lib.qwn_x_w4_shard(C.byref(sh), full.ref, rank, world, 0, None, 0) == 0
                full.codes.free()
                full.scales.free()
                full.rec = sh
            pair.append(full)
        copies.append(pair)
    warr = [pkg.weight_array(p) for p in copies]
    x = wl.activations_normal(T, K, seed=5, outlier_frac=0.01)
    dx = pkg.DevBuf.from_numpy(x)
    nblk = K // 32 * T
    aq, as_, asum, as_tok = (pkg.DevBuf(nblk * 32), pkg.DevBuf(nblk * 4), pkg.DevBuf(nblk * 4),
                             pkg.DevBuf(T * 4))
    # this rank's outputs [gate|up][T][n_shard], contiguous so that they are one send buffer
    block = 2 * T * n_shard                      # floats per rank
    ycat = pkg.DevBuf(block * 4)
    y_ptrs = [ycat.ptr, ycat.ptr + T * n_shard * 4]
    yarr = (C.c_void_p * 2)(*y_ptrs)
    # gathered outputs: [2 halves][world][gate|up][T][n_shard] (NCCL uses the first half)
    gathered = pkg.DevBuf(2 * world * block * 4) if world > 1 else None
    fused = world > 1 and args.exchange == "fused"
    half_off = C.c_size_t(0)
    if world > 1:
        flags = pkg.DevBuf(world * 4)
        lib.tq_dev_zero(flags.ptr, world * 4)
        handles = []
        for buf in (gathered, flags):
            h = (C.c_char * 64)()
            assert lib.tq_comm_ipc_export(buf.ptr, h) == 0
            handles.append(bytes(h.raw))
        allh = [None] * world
        dist.all_gather_object(allh, handles)
        bufs, flgs = (C.c_void_p * world)(), (C.c_void_p * world)()
        for p in range(world):
            if p == rank:
                bufs[p], flgs[p] = gathered.ptr, flags.ptr
            else:
                bufs[p] = lib.tq_comm_ipc_open(C.create_string_buffer(allh[p][0], 64))
                flgs[p] = lib.tq_comm_ipc_open(C.create_string_buffer(allh[p][1], 64))
                if not bufs[p] or not flgs[p]:
                    fused = False
        ok_all = [None] * world
        dist.all_gather_object(ok_all, bool(fused))
        fused = all(ok_all)                      # every rank takes the same path
        if fused:
            assert lib.tq_comm_gather_setup(bufs, flgs, world, rank) == 0

    xin = [dx.ptr]       # the fp32 activations the step reads (the end-to-end loop alternates two)

    def stage():
        lib.qwn_x_quantize_act_chunk_pertoken(xin[0], K, T, aq.ptr, as_.ptr, asum.ptr, as_tok.ptr)

    def gemm(i):
        rc = lib.qwn_x_gemm_w4a8_fanout(warr[i % args.rotate], yarr, 2, aq.ptr, as_.ptr, asum.ptr, T,
                                        None, 0)
        assert rc == 0, rc

    def gemm_gathered(i):
        rc = lib.qwn_x_gemm_w4a8_fanout_gathered(warr[i % args.rotate], 2, aq.ptr, as_.ptr, asum.ptr,
                                                 T, C.byref(half_off))
        assert rc == 0, rc
        assert lib.tq_comm_gather_wait() == 0

    # The step a user runs: ONE call that quantises the fp32 activations per token in the GEMM
    # kernel's prologue, multiplies gate|up and (N > 1) gathers the ranks' slices.
    qfused = args.quantiser == "fused"

    def gemm_fused(i, out=None):
        if qfused:
            rc = lib.qwn_x_gemm_w4a8_fanout_fused(warr[i % args.rotate], out or yarr, 2, xin[0], T, 1)
        else:
            stage()
            rc = lib.qwn_x_gemm_w4a8_fanout(warr[i % args.rotate], out or yarr, 2, aq.ptr, as_.ptr,
                                            asum.ptr, T, None, 0)
        assert rc == 0, rc

    def step(i):
        if fused and qfused:
            rc = lib.qwn_x_gemm_w4a8_fanout_gathered_fused(warr[i % args.rotate], 2, xin[0], T, 1,
                                                           C.byref(half_off))
            assert rc == 0, rc
        elif fused:
            stage()
            gemm_gathered(i)
        else:
            gemm_fused(i)
            if world > 1:
                assert lib.tq_comm_allgather(ycat.ptr, gathered.ptr, ycat.nbytes) == 0

    if fused:
        # the fused gather must deliver exactly what NCCL delivers, on every weight copy and
        # on both halves of the gathered buffer
        stage()
        for i in range(2 * args.rotate):
            gemm(i)
            assert lib.tq_comm_allgather(ycat.ptr, gathered.ptr, ycat.nbytes) == 0
            lib.tq_sync()
            ref = gathered.to_numpy(np.float32)[: world * block].copy()
            dist.barrier()
            step(i)                  # fused quantiser + GEMM + peer-store gather
            lib.tq_sync()
            dist.barrier()
            got = gathered.to_numpy(np.float32)[half_off.value: half_off.value + world * block]
            assert got.tobytes() == ref.tobytes(), f"fused all-gather differs from NCCL (step {i})"
            dist.barrier()

    def barrier():
        lib.tq_sync()
        if dist:
            dist.barrier()

    ev = [lib.tq_event_create() for _ in range(2)]
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_load0 = time.time()

    # ---- timed region: whole steps ----------------------------------------------------
    for i in range(args.warmup):
        step(i)
    barrier()
    lib.tq_event_record(ev[0])
    for i in range(args.steps):
        step(i)
    lib.tq_event_record(ev[1])
    barrier()
    ms = lib.tq_event_elapsed_ms(ev[0], ev[1])
    if dist:
        import torch
        tt = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    # weight bytes the whole job streams per step (all ranks)
    full_weight_bytes = 2 * wl.weight_bytes(N_EACH, K, GROUP) * (world if weak else 1)
    value = full_weight_bytes * args.steps / (ms * 1e-3) / 1e9

    # ---- dominant kernel alone (this rank's shard), for the roofline -----------------------
    stage()
    alone = gemm_fused if qfused else gemm      # staged: the GEMM launch without its staging
    for i in range(args.warmup):
        alone(i)
    lib.tq_sync()
    k_iters = max(args.steps, 200)
    lib.tq_event_record(ev[0])
    for i in range(k_iters):
        alone(i)
    lib.tq_event_record(ev[1])
    lib.tq_sync()
    k_ms = lib.tq_event_elapsed_ms(ev[0], ev[1]) / k_iters
    if fused:
        # diagnostic (stderr): the gathered GEMM with its wait kernel, back to back
        barrier()
        lib.tq_event_record(ev[0])
        for i in range(k_iters):
            step(i)
        lib.tq_event_record(ev[1])
        barrier()
        g_ms = lib.tq_event_elapsed_ms(ev[0], ev[1]) / k_iters
        if rank == 0:
            print(f"[bench] GEMM alone {k_ms * 1e3:.2f} us; gathered GEMM + wait {g_ms * 1e3:.2f} us; "
                  f"step {ms / args.steps * 1e3:.2f} us", file=sys.stderr)
    shard_weight = 2 * wl.weight_bytes(n_shard, K, GROUP)
    # weights + the fp32 activation rows the prologue quantises + the fp32 outputs
    algo_bytes = shard_weight + (T * K * 4 if qfused else T * K + nblk * 8) + block * 4
    achieved = algo_bytes / (k_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()

    # ---- end to end through the C-ABI with host buffers ----------------------------------
    hx = lib.tq_host_alloc_pinned(x.nbytes)
    C.memmove(hx, x.ctypes.data, x.nbytes)
    # strong: every rank reads the whole gathered result back; weak: a rank reads back its own
    # slice of the gathered buffer, so the host receives the (world times larger) result once
    out_bytes = (block * 4 if weak else world * block * 4 if world > 1 else ycat.nbytes)
    hy = [lib.tq_host_alloc_pinned(out_bytes) for _ in range(2)]
    # Two output buffers: the read-back of step i (second stream) overlaps step i+1, and the
    # library stream waits for it only before step i+2 overwrites the same buffer.
    ycat2 = pkg.DevBuf(block * 4)
    yarr2 = (C.c_void_p * 2)(ycat2.ptr, ycat2.ptr + T * n_shard * 4)
    tickets = [-1, -1]
    # Two input buffers as well: step n+1's activations come up from pinned host memory on a
    # third stream while step n computes (one upload per step; the first is queued before the
    # timed loop and the last step's upload is the one nothing reads).
    dx2 = pkg.DevBuf(x.nbytes)
    xbuf = [dx.ptr, dx2.ptr]
    up = [lib.tq_h2d_overlapped(xbuf[0], hx, x.nbytes), -1]
    count = [0]
    e2e_src = [None]

    def e2e_step(i):
        n = count[0]
        count[0] = n + 1
        # N > 1, strong: this rank's next flag tells its peers that they may overwrite the half
        # it is still reading back, so there the previous read-back must finish before the next
        # step. Weak with the fused gather: a rank reads back its own slice only, which no peer
        # writes, so as at N = 1 the read-back of step n must only be over before step n+2
        # writes the same half (NCCL's gather has one buffer, rewritten whole every step).
        b = n & 1 if (world == 1 or (weak and fused)) else 0
        if tickets[b] >= 0:
            lib.tq_stream_wait_copy(tickets[b])
        # the other input buffer was last read by step n-1, which is queued already
        up[(n + 1) & 1] = lib.tq_h2d_overlapped(xbuf[(n + 1) & 1], hx, x.nbytes)
        lib.tq_stream_wait_copy(up[n & 1])
        xin[0] = xbuf[n & 1]
        if world == 1:
            gemm_fused(i, yarr2 if b else yarr)
            src = (ycat2 if b else ycat).ptr
        else:
            step(i)
            src = gathered.ptr + ((half_off.value if fused else 0) + (rank * block if weak else 0)) * 4
        tickets[b] = lib.tq_d2h_overlapped(hy[n & 1], src, out_bytes)
        e2e_src[0] = (src, i, n & 1)
        assert tickets[b] >= 0 and up[(n + 1) & 1] >= 0

    e_iters = max(min(args.steps, 2000), 50)
    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e_iters):
        e2e_step(i)
    lib.tq_sync()
    e_s = time.perf_counter() - t0
    xin[0] = dx.ptr
    # what the host received in the last step is what the device holds; at N = 1 the step is
    # also run again from the input buffer that was uploaded synchronously at the start
    src, last, lb = e2e_src[0]
    got = np.ctypeslib.as_array(C.cast(hy[lb], C.POINTER(C.c_float)), shape=(out_bytes // 4,)).copy()
    if world == 1:
        gemm_fused(last, yarr2 if lb else yarr)
        want = (ycat2 if lb else ycat).to_numpy(np.float32, out_bytes // 4)
    else:
        want = np.empty(out_bytes // 4, dtype=np.float32)
        lib.tq_d2h(want.ctypes.data, src, out_bytes)
    e2e_diff = int(np.count_nonzero(got.view(np.uint32) != want.view(np.uint32)))
    if e2e_diff:
        print(f"[bench] rank {rank}: the end-to-end loop's last result differs from the device's in "
              f"{e2e_diff} of {got.size} words", file=sys.stderr)
    if dist:
        import torch
        tt = torch.tensor([e_s], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e_s = float(tt.item())
    e2e_val = full_weight_bytes * e_iters / e_s / 1e9
    t_load1 = time.time()
    if sampler and (t_load1 - t_load0) < 0.6:
        # too short for nvidia-smi's sampling period: keep the same kernels running a little
        tend = time.time() + 0.6
        i = 0
        while time.time() < tend:
            gemm_fused(i)
            i += 1
            if i % 256 == 0:
                lib.tq_sync()
        lib.tq_sync()
        t_load1 = time.time()
    clocks = sampler.stop(t_load0, t_load1) if sampler else None
    err = lib.tq_last_error()

    # ---- CPU baseline (rank 0, N = 1 only) ----------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as orc
        orc.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity")
                            else (os.cpu_count() or 1))
        oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
        cpu_pass(orc, host_w, oq, os_, osm)      # warm
        passes, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 12.0:
            orc.quantize_act_chunk(x, per_token=True)
            cpu_pass(orc, host_w, oq, os_, osm)
            passes += 1
        dt = time.perf_counter() - t0
        cpu = {"value": full_weight_bytes * passes / dt / 1e9, "unit": UNIT, "cores": orc.num_threads(),
               "kind": "port", "sample": f"{passes} full passes of cfg2 in {dt:.1f} s (OpenMP, all host threads)"}

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak" if (weak or world == 1) else "strong", "vs_baseline": None,
            "dtype": "s8xs4->s32, fp32 out",
            "data": "synthetic",
            "config": {"workload": "cfg2: batched decode fused gate+up, K64 scale tier, T=8, K=5120, "
                                   "N=2x17408, int8 per-token activations" +
                                   (f"; one cfg2-sized column shard per GPU (N={world}x2x17408 in all)"
                                    if weak else ""),
                       "parallelism": f"column shard tp{world}" + (
                           "" if world == 1 else " + all-gather by peer stores from the GEMM epilogue"
                           if fused else " + NCCL all-gather"),
                       "l2": f"inputs larger than L2: {args.rotate} rotating weight copies, "
                             f"{args.rotate * shard_weight / 1e6:.0f} MB per GPU",
                       "step": ("one launch: per-token activation quantiser in the prologue of the "
                                "fused gate|up GEMM" if qfused else
                                "per-token staging (1 launch) + fused gate|up GEMM") +
                               (" + all-gather" if world > 1 else "")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth",
                         "kernel": "gemm_w4a8_ring_kernel", "us_per_launch": k_ms * 1e3,
                         "algorithmic_bytes_per_launch": algo_bytes,
                         # the capture is of the whole-cfg2 launch; a shard's traffic scales with it
                         "traffic": int(NCU_TRAFFIC_BYTES_PER_LAUNCH * algo_bytes / 95_977_472)},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": int(x.nbytes),
                    "d2h_bytes_per_step": int(out_bytes), "steps": e_iters,
                    "us_per_step": e_s / e_iters * 1e6,
                    "last_result_words_differing": e2e_diff},
            "gpu_launches": ((1 if qfused else 2) + (1 if fused else 0) + (1 if world > 1 and not fused else 0)) * args.steps,
            "clocks": clocks,
            "cpu_baseline": cpu,
            "device_error": err,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        lib.tq_comm_destroy()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
