"""Multi-GPU leg of bench.py (one rank per GPU, launched by torchrun): the 64-layer projection
stack with every projection column-sharded over the ranks, strong scaling (the same 13.4 GB of
weights per step at every N). torch.distributed (gloo) is the control plane only: barriers,
the exchange of IPC handles, max-over-ranks of the device times.

Rank 0 also runs the unsharded stack on its own GPU in the same process: the sharded result
must be byte-identical to it (`tp1_words_differing`), and its time is the strong-scaling
baseline measured in the same run (`tp1_ms_per_step`).
"""
from __future__ import annotations

import ctypes as C
import json
import time

import numpy as np

import bench as B


class Comm:
    """World set-up for the fused exchange: flag arrays and symmetric buffers mapped into
    every rank through CUDA IPC."""

    def __init__(self, ctx, dist, rank, world):
        self.ctx, self.dist, self.rank, self.world = ctx, dist, rank, world
        lib, pkg = ctx.lib, ctx.pkg
        self.flags = pkg.DevBuf(world * 4)
        lib.tq_dev_zero(self.flags.ptr, world * 4)
        self.flag_ptrs = self._map(self.flags)
        self.slots = 0

    def _map(self, buf):
        lib = self.ctx.lib
        h = (C.c_char * 64)()
        assert lib.tq_comm_ipc_export(buf.ptr, h) == 0
        allh = [None] * self.world
        self.dist.all_gather_object(allh, bytes(h.raw))
        ptrs = (C.c_void_p * self.world)()
        for p in range(self.world):
            ptrs[p] = buf.ptr if p == self.rank else lib.tq_comm_ipc_open(C.create_string_buffer(allh[p], 64))
            assert ptrs[p], f"rank {self.rank}: cannot map rank {p}'s buffer"
        return ptrs

    def register(self, bufs):
        lib = self.ctx.lib
        maps = [self._map(b) for b in bufs]
        assert lib.tq_comm_gather_setup(maps[0], self.flag_ptrs, self.world, self.rank) == 0
        for i, m in enumerate(maps):
            assert lib.tq_comm_sym_register(i, m) == 0
        self.maps = maps
        self.dist.barrier()          # every rank has cleared its flags before anyone publishes


class WeakCfg2:
    """Weak scaling of the headline projection: every rank multiplies its own cfg2 weights
    (2 x 17408 x 5120, K64 - columns [rank * 34816, (rank + 1) * 34816) of a global
    [8][world * 34816] output); the GEMM epilogue stores its columns into every rank's copy of
    that matrix, and an exchange point closes the step. Per-GPU work is fixed, so the ideal
    time per step is the single-GPU time."""

    def __init__(self, ctx, comm, rank, world):
        self.ctx, self.rank, self.world = ctx, rank, world
        pkg, lib = ctx.pkg, ctx.lib
        self.T, self.N2 = 8, 2 * B.I_FF
        self.gate = ctx.rotated(B.I_FF, B.H, 11 + 2 * rank, 64)
        self.up = ctx.rotated(B.I_FF, B.H, 12 + 2 * rank, 64)
        self.x = pkg.DevBuf.from_numpy(ctx.wl.activations_normal(self.T, B.H, seed=5, outlier_frac=0.01))
        nb = B.H // 32 * self.T
        self.aq, self.as_, self.asum, self.as_tok = (pkg.DevBuf(nb * 32), pkg.DevBuf(nb * 4), pkg.DevBuf(nb * 4),
                                                     pkg.DevBuf(self.T * 4))
        self.out = pkg.DevBuf(self.T * world * self.N2 * 4)
        comm.register([self.out])
        self.weight_bytes = 2 * ctx.wl.weight_bytes(B.I_FF, B.H, 64)
        self.steps_per_pass = len(self.gate)
        # staging (with the exchange point) and GEMM per step; exchange point + advance per pass
        self.launches_per_pass = 2 * self.steps_per_pass + 2
        self.graph = None

    def _step(self, c, first):
        """Staging + GEMM on weight copy c. The staging kernel carries the exchange point that
        orders the previous step's peer stores (as the consumer of a gathered matrix does in a
        model), so no launch is spent on the exchange itself."""
        lib, pkg, T = self.ctx.lib, self.ctx.pkg, self.T
        f = lib.qwn_x_quantize_act_chunk_pertoken if first else lib.qwn_x_quantize_act_chunk_pertoken_sync
        f(self.x.ptr, B.H, T, self.aq.ptr, self.as_.ptr, self.asum.ptr, self.as_tok.ptr)
        warr = (C.POINTER(pkg.TqWeight) * 2)(C.pointer(self.gate[c].rec), C.pointer(self.up[c].rec))
        fr = (C.c_int * 2)(B.I_FF, B.I_FF)
        co = (C.c_size_t * 2)(self.rank * self.N2, self.rank * self.N2 + B.I_FF)
        rc = lib.qwn_x_gemm_w4a8_fanout_tp(warr, 2, self.aq.ptr, None, self.as_tok.ptr, self.asum.ptr, T, fr,
                                           None, 0, co, self.world * self.N2)
        assert rc == 0, rc

    def _issue_pass(self):
        """One pass = one step per weight copy, then the exchange point of the last step and the
        step-base advance that makes the pass replayable."""
        lib = self.ctx.lib
        for c in range(len(self.gate)):
            self._step(c, c == 0)
        assert lib.tq_comm_exchange_sync() == 0
        assert lib.tq_comm_exchange_advance() == 0

    def capture(self):
        lib = self.ctx.lib
        self._issue_pass()
        lib.tq_sync()
        assert lib.tq_graph_capture_begin() == 0
        self._issue_pass()
        self.graph = lib.tq_graph_capture_end()
        assert self.graph, "graph capture failed"

    def run_pass(self):
        if self.graph:
            self.ctx.lib.tq_graph_launch(self.graph)
        else:
            self._issue_pass()


def run_weak(args, ctx, dist, rank, world, barrier, max_over_ranks):
    """The weak cfg2 record of the multi-GPU line."""
    lib = ctx.lib
    single_us = None
    if rank == 0:
        head, _, _ = B.build_cases(ctx, {"cfg2"})["cfg2"]
        single_us = ctx.time_loop(lambda i: head.run(i, 0, 0), 200, warmup=20) * 1e3
        del head
    dist.barrier()
    comm = Comm(ctx, dist, rank, world)
    wk = WeakCfg2(ctx, comm, rank, world)
    barrier()
    wk.run_pass()
    barrier()
    full = wk.out.to_numpy(np.uint32)
    sums = [None] * world
    dist.all_gather_object(sums, (int(full.astype(np.uint64).sum()), int(np.bitwise_xor.reduce(full))))
    differ = sum(1 for v in sums if v != sums[0])
    wk.capture()
    barrier()
    for i in range(5):
        wk.run_pass()
    barrier()
    ev, passes = ctx.events(), 50
    t0 = time.time()
    lib.tq_event_record(ev[0])
    for i in range(passes):
        wk.run_pass()
    lib.tq_event_record(ev[1])
    barrier()
    ctx.load_spans.append((t0, time.time()))
    steps = passes * wk.steps_per_pass
    us = max_over_ranks(lib.tq_event_elapsed_ms(ev[0], ev[1])) / steps * 1e3
    err = lib.tq_last_error()
    rec = {"workload": B.WORKLOAD_CFG2, "scaling": "weak",
           "us_per_step": us, "single_gpu_us_per_step": single_us,
           "value": world * wk.weight_bytes / (us * 1e-6) / 1e9, "unit": B.UNIT,
           "per_gpu_weight_bytes": int(wk.weight_bytes), "launches_per_pass": wk.launches_per_pass,
           "steps_per_pass": wk.steps_per_pass,
           "ranks_with_a_different_result": differ, "steps": steps, "device_error": err,
           "step": "per-token staging (its prologue is the exchange point behind the previous step's peer "
                   "stores), fused gate|up GEMM storing its columns into every rank's [8][N x 34816] matrix; "
                   "a pass of one step per weight copy is one CUDA graph"}
    barrier()
    del wk
    lib.tq_comm_destroy()
    dist.barrier()
    return rec


def run(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    ctx = B.Ctx(args.rotate)
    lib, pkg = ctx.lib, ctx.pkg
    assert lib.tq_set_device(local_rank) == 0
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sampler = B.ClockSampler(local_rank) if rank == 0 else None

    def barrier():
        lib.tq_sync()
        dist.barrier()

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- weak scaling of the headline projection (a record inside the line) --------------------
    weak = run_weak(args, ctx, dist, rank, world, barrier, max_over_ranks)
    if args.scaling == "weak":
        # the weak record as the line: cfg2 on every rank, whole-job weight bytes per second
        clocks = sampler.stop(ctx.load_spans) if sampler else None
        if rank == 0:
            print(json.dumps({
                "metric": B.METRIC, "value": weak["value"], "unit": B.UNIT, "n_gpus": world,
                "steps": weak["steps"], "warmup": 5 * weak["steps_per_pass"], "ms_per_step": weak["us_per_step"] / 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "s8xs4->s32, fp32 out", "data": "synthetic",
                "config": {"workload": B.WORKLOAD_CFG2, "parallelism": f"one cfg2-sized column shard per GPU ({world} "
                           "GPUs), outputs stored into every rank's matrix by the GEMM epilogue",
                           "l2": "inputs larger than L2: rotating weight copies", "step": weak["step"]},
                "single_gpu_us_per_step": weak["single_gpu_us_per_step"],
                "ranks_with_a_different_result": weak["ranks_with_a_different_result"],
                "roofline": {"bound": "hbm", "achieved": weak["value"] / world, "peak": ctx.peak_hbm, "unit": "GB/s",
                             "frac": weak["value"] / world / ctx.peak_hbm, "peak_source": f"{ctx.peak_kind} copy bandwidth",
                             "kernel": "whole step, per GPU", "traffic": None},
                "e2e": None, "gpu_launches": weak["launches_per_pass"] * weak["steps"] // weak["steps_per_pass"],
                "clocks": clocks, "cpu_baseline": None, "device_error": weak["device_error"]}), flush=True)
        dist.destroy_process_group()
        return

    # ---- the unsharded stack on rank 0: result to match, time to scale from ------------------
    tp1 = {"ms": None, "out": None}
    if rank == 0:
        st1 = B.Stack(ctx, layers=args.layers)
        st1.capture()
        tp1["ms"] = ctx.time_loop(lambda i: st1.run(i, 0, 0), 10)
        lib.tq_sync()
        tp1["out"] = st1.y4.to_numpy(np.uint32).copy()
        del st1
    dist.barrier()

    # ---- the sharded stack -------------------------------------------------------------------
    comm = Comm(ctx, dist, rank, world)
    st = B.Stack(ctx, layers=args.layers, tp=world, rank=rank, comm=comm)
    barrier()
    st.run(0, 0, 0)                      # eager pass: warm-up, all scratch allocated
    barrier()
    out = st.y4.to_numpy(np.uint32).copy()
    diff = int(np.count_nonzero(out != tp1["out"])) if rank == 0 else 0
    # every rank must hold the same gathered result
    outs = [None] * world
    dist.all_gather_object(outs, out.tobytes())
    ranks_differ = sum(1 for o in outs if o != outs[0])
    barrier()
    st.capture()
    barrier()
    for i in range(args.warmup):
        st.run(i, 0, 0)
    barrier()
    ev = ctx.events()
    t0 = time.time()
    lib.tq_event_record(ev[0])
    for i in range(args.steps):
        st.run(i, 0, 0)
    lib.tq_event_record(ev[1])
    barrier()
    ctx.load_spans.append((t0, time.time()))
    ms = max_over_ranks(lib.tq_event_elapsed_ms(ev[0], ev[1])) / args.steps
    out2 = st.y4.to_numpy(np.uint32)
    replay_diff = int(np.count_nonzero(out2 != out))       # graph replays give the eager result

    # ---- this rank's GEMMs alone (no staging, no exchange): where the step's time is not ------
    lib.qwn_x_quantize_act_chunk_pertoken(st.xn.ptr, B.H, 8, st.aq.ptr, st.as_.ptr, st.asum.ptr, st.as_tok.ptr)

    # (the four GEMM kinds read different K; time each kind with its own staging below)
    kinds = []
    for name, K, pick, full in (("5120->10240", B.H, lambda l: [l[0]], [B.QKV]),
                                ("10240->5120", B.QKV, lambda l: [l[1]], [B.H]),
                                ("5120->gate|up", B.H, lambda l: [l[2], l[3]], [B.I_FF, B.I_FF]),
                                ("17408->5120", B.I_FF, lambda l: [l[4]], [B.H])):
        src = {B.H: st.xn, B.QKV: st.y1, B.I_FF: st.h}[K]
        lib.qwn_x_quantize_act_chunk_pertoken(src.ptr, K, 8, st.aq.ptr, st.as_.ptr, st.asum.ptr, st.as_tok.ptr)
        scratch = [st.gu.ptr, st.gu.ptr + 8 * (B.I_FF // world) * 4]

        def one(i, pick=pick, full=full):
            ws = pick(st.layers[i % st.L])
            st._gemm(ws, full, -1, None, 0, ys=scratch[: len(ws)])
        kinds.append((name, ctx.time_loop(one, 4 * st.L, warmup=8) * 1e3))
    gemm_us = sum(us for _, us in kinds) * st.L
    gemm_us = max_over_ranks(gemm_us)

    # ---- end to end with host buffers ------------------------------------------------------
    barrier()
    e_iters = max(min(args.steps, 200), 10)
    e_s, e_diff = B.e2e_loop(ctx, st, e_iters, warmup=3)
    e_s = max_over_ranks(e_s)
    barrier()
    clocks = sampler.stop(ctx.load_spans) if sampler else None
    err = lib.tq_last_error()
    errs = [None] * world
    dist.all_gather_object(errs, err)

    if rank == 0:
        wb = st.weight_bytes
        line = {
            "metric": B.METRIC, "value": wb / (ms * 1e-3) / 1e9, "unit": B.UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "s8xs4->s32, fp32 out", "data": "synthetic",
            "config": {"workload": B.WORKLOAD_CFG5,
                       "parallelism": f"column shard tp{world}; projections store their output columns into "
                                      "every rank's activation matrix (peer stores from the GEMM epilogue), "
                                      "the next staging kernel carries the exchange point",
                       "l2": f"inputs larger than L2: {wb / world / 1e9:.2f} GB of distinct weights per GPU "
                             "per step",
                       "step": f"{st.L} layers x (norm+staging, 4 GEMMs, 3 stagings, silu*mul scatter) replayed as one CUDA "
                               f"graph; {4 * st.L} exchange points per step"},
            "tp1_ms_per_step": tp1["ms"],
            "tp1_words_differing": diff,
            "ranks_with_a_different_result": ranks_differ,
            "graph_replay_words_differing": replay_diff,
            "step_split_us": {"step": ms * 1e3, "gemm_kernels_alone": gemm_us,
                              "staging_exchange_and_gaps": ms * 1e3 - gemm_us,
                              "gemm_kinds_us_per_launch": dict(kinds)},
            "roofline": {"bound": "hbm", "achieved": wb / world / (ms * 1e-3) / 1e9, "peak": ctx.peak_hbm,
                         "unit": "GB/s", "frac": wb / world / (ms * 1e-3) / 1e9 / ctx.peak_hbm,
                         "peak_source": f"{ctx.peak_kind} copy bandwidth", "kernel": "whole step, per GPU",
                         "algorithmic_bytes_per_launch": int(wb / world), "traffic": None},
            "e2e": {"value": wb / e_s / 1e9, "unit": B.UNIT, "h2d_bytes_per_step": int(st.x_host.nbytes),
                    "d2h_bytes_per_step": int(st.out_bytes), "steps": e_iters, "us_per_step": e_s * 1e6,
                    "last_result_words_differing": e_diff},
            "weak_cfg2": weak,
            "gpu_launches": st.launches_per_step * args.steps,
            "clocks": clocks, "cpu_baseline": None, "device_error": max(errs),
        }
        print(json.dumps(line), flush=True)
    lib.tq_comm_destroy()
    dist.destroy_process_group()
