"""The N > 1 path on CPU: two gloo ranks column-shard a packed weight the way bench.py and
x_w4_shard (mode 0) do, run the projection on their shard (CPU oracle in the role of the
device kernel), all-gather the output slices and compare with the unsharded result. Mirrors
the reference's shard gate (xpu/src/kernels_dpas.cpp:2544-2599): the concatenation of column
shards must be bit-identical to the full projection."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, groups, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import oracle as orc
    import refgen
    wl = importlib.import_module("knivesysl-xe_b200.workloads")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, T, ksh = 256, 512, 8, 1
        codes, scales = wl.random_packed_weight(M, K, seed=5, ksh=ksh)     # same on every rank
        x = refgen.gemm_check_rows(T, K)
        aq, as_, asum = orc.quantize_act_chunk(x)
        rc, sc, ss = orc.w4_shard_column(codes, scales, M, K, ksh, rank, world, groups=groups)
        assert rc == 0
        Mn = M // world
        _, y_local = orc.gemm_w4a8(sc, ss, Mn, K, ksh, aq, as_, asum, T, fma=1)
        y_local = torch.from_numpy(np.ascontiguousarray(y_local.reshape(T, Mn)))
        gathered = [torch.empty_like(y_local) for _ in range(world)]
        dist.all_gather(gathered, y_local)                                  # [rank][T][Mn]
        if rank == 0:
            _, y_full = orc.gemm_w4a8(codes, scales, M, K, ksh, aq, as_, asum, T, fma=1)
            y_full = y_full.reshape(T, M)
            # rebuild the row order: within every group, rank r owns the r-th run of rows
            gs = groups or [M]
            out = np.empty((T, M), dtype=np.float32)
            src_off = [0] * world
            dst = 0
            for gsz in gs:
                per = gsz // world
                for r in range(world):
                    out[:, dst:dst + per] = gathered[r].numpy()[:, src_off[r]:src_off[r] + per]
                    src_off[r] += per
                    dst += per
            q.put(out.tobytes() == y_full.tobytes())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("groups", [None, [128, 128]])
def test_two_rank_column_shard_allgather_bit_identical(groups):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, groups, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert q.get(timeout=5) is True


def test_max_over_ranks_timing_reduction():
    """bench.py reports the slowest rank: the MAX all-reduce it uses, on two gloo ranks."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_max_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    assert q.get(timeout=5) == 7.0


def _max_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    t = torch.tensor([3.0 if rank == 0 else 7.0], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        q.put(float(t.item()))
    dist.barrier()
    dist.destroy_process_group()


def _row_main(rank, world, port, q):
    """Row-parallel (K) shard, x_w4_shard mode 1: every rank multiplies its K range and the
    partial outputs are summed (gloo all-reduce in the role of tq_comm_allreduce_sum)."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import oracle as orc
    import refgen
    wl = importlib.import_module("knivesysl-xe_b200.workloads")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, ksh = 128, 1024, 1
        codes, scales = wl.random_packed_weight(M, K, seed=9, ksh=ksh)
        x = refgen.shard_check_row(K)
        Kt, Kn = K // 32, K // world
        cs = codes.reshape(M // 16, Kt, 256)[:, rank * (Kt // world):(rank + 1) * (Kt // world)]
        g = (Kt // world) >> ksh
        ss = scales.reshape(M // 16, Kt >> ksh, 16)[:, rank * g:(rank + 1) * g]
        xs = np.ascontiguousarray(x[rank * Kn:(rank + 1) * Kn])
        q8, sc, sm = orc.quantize_act_s8(xs)
        _, part = orc.gemv_w4a8(np.ascontiguousarray(cs).reshape(-1), np.ascontiguousarray(ss).reshape(-1),
                                M, Kn, ksh, q8, sc, sm, fma=1)
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        if rank == 0:
            qf, scf, smf = orc.quantize_act_s8(x)       # per-K32 scales: the same codes as the shards'
            _, full = orc.gemv_w4a8(codes, scales, M, K, ksh, qf, scf, smf, fma=1)
            err = np.abs(t.numpy() - full).max() / max(np.abs(full).max(), 1e-6)
            q.put(float(err))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_row_shard_allreduce_within_tolerance():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_row_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert q.get(timeout=5) <= 1e-3       # the stated fp32 tolerance; not bit-exact by design


def _chain_main(rank, world, port, q):
    """Two column-sharded projections in a row with per-token activation scales, the way the
    tensor-parallel decode chain runs them: a shard is split like the whole projection
    (the split count comes from the unsharded row count), every rank ends up with the full
    output matrix, quantises it per token and multiplies its shard of the next weight."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import oracle as orc
    wl = importlib.import_module("knivesysl-xe_b200.workloads")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, K0, N1, N2, ksh = 8, 512, 640, 384, 0
        w1 = wl.random_packed_weight(N1, K0, seed=21, ksh=ksh)              # same on every rank
        w2 = wl.random_packed_weight(N2, N1, seed=22, ksh=ksh)
        x = wl.activations_normal(T, K0, seed=3, outlier_frac=0.01)

        def project(weight, M, K, xin, sharded):
            codes, scales = weight
            aq, as_, asum = orc.quantize_act_chunk(xin, per_token=True)
            as_tok = as_.reshape(K // 32, T)[0].copy()
            S = orc.choose_pertoken_splits(M // 16, T // 8, K // 32, ksh)   # of the WHOLE projection
            if not sharded:
                return orc.gemm_w4a8_pertoken(codes, scales, M, K, ksh, aq, as_tok, asum, T, splits=S)[1].reshape(T, M), S
            rc, sc, ss = orc.w4_shard_column(codes, scales, M, K, ksh, rank, world, groups=None)
            assert rc == 0
            Mn = M // world
            y = orc.gemm_w4a8_pertoken(sc, ss, Mn, K, ksh, aq, as_tok, asum, T, splits=S)[1].reshape(T, Mn)
            y = torch.from_numpy(np.ascontiguousarray(y))
            parts = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(parts, y)
            return np.concatenate([p.numpy() for p in parts], axis=1), S   # columns [r * Mn, (r + 1) * Mn)

        y1, S1 = project(w1, N1, K0, x, True)
        y2, S2 = project(w2, N2, N1, y1, True)
        if rank == 0:
            f1, _ = project(w1, N1, K0, x, False)
            f2, _ = project(w2, N2, N1, f1, False)
            # the rule under test matters: a shard on its own would pick another split count
            own = orc.choose_pertoken_splits(N1 // world // 16, T // 8, K0 // 32, ksh)
            q.put((y1.tobytes() == f1.tobytes(), y2.tobytes() == f2.tobytes(), S1, own))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_per_token_chain_bit_identical():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_chain_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    same1, same2, s_full, s_shard = q.get(timeout=5)
    assert same1 and same2
    assert s_full != s_shard or s_full == 16, (s_full, s_shard)
