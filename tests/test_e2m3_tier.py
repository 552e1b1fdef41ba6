"""The tier a weight is in before it is repacked: the TQF record reader, the scalar E2M3 GEMV
behind x_gemv_qmma, the absolute quality gate qwn_w4_check, the repack policy, and
qwn_shard_check_all over a synthetic projection family."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

FLAGS = (1 << 5) | (1 << 8)            # block-scaled QMMA, dense E2M3 (xpu/src/tq_common.hpp:40-43)


def make_record(orc, M, K, seed, k32_scales=False):
    rng = np.random.default_rng(seed)
    codes6 = rng.integers(0, 64, size=(M, K), dtype=np.uint8)
    rows, cols = (M + 127) // 128, (K // 32 if k32_scales else (K + 127) // 128)
    bs = (rng.random((rows, cols)) * 0.01 + 0.002).astype(np.float32)
    payload = orc.e2m3_payload_from_codes_fast(codes6)
    blob = struct.pack("<II", rows, cols) + bs.tobytes() + payload.tobytes()
    return blob, payload, bs, cols


def test_selector_grammar_and_tier_policy(pkg):
    lib = pkg.load()
    has = lambda s, k: lib.tq_selector_has(s.encode() if s is not None else None, k.encode())
    assert has("gate,up,down", "up") and has(" gate , up ", "gate") and has("all", "in_qkv")
    assert has("q, all", "lm_head") and not has("gate,up", "down") and not has("", "gate")
    assert not has(None, "gate") and not has("gateway", "gate") and not has("ga", "gate")
    keep = {k: os.environ.get(k) for k in ("TQ_XPU_W4A8", "TQ_XPU_W8", "TQ_XPU_W4_K16", "TQ_XPU_K64")}
    try:
        for k in keep:
            os.environ.pop(k, None)
        tier = lambda k: lib.tq_repack_tier_for(k.encode())
        assert tier("lm_head") == 8 and tier("gate") == 0          # default: only lm_head is int8
        os.environ["TQ_XPU_K64"] = "gate,up,down"
        assert tier("gate") == 2 and tier("q") == 0
        os.environ["TQ_XPU_K64"] = "1"                             # "1" means every matrix
        assert tier("q") == 2 and tier("lm_head") == 8             # W8 wins over K64
        os.environ["TQ_XPU_W4_K16"] = "all"
        assert tier("gate") == 1                                   # K16 wins over K64
        os.environ["TQ_XPU_W8"] = ""                               # empty: no int8 matrix
        assert tier("lm_head") == 1
        os.environ["TQ_XPU_W4A8"] = "0"
        assert tier("gate") == -1                                  # keep the E2M3 payload
    finally:
        for k, v in keep.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,k32", [(128, 512, False), (272, 1024, True), (1088, 5120, False)])
def test_record_reader_and_scalar_gemv(lib, pkg, orc, M, K, k32):
    blob, payload, bs, cols = make_record(orc, M, K, seed=M + K, k32_scales=k32)
    w = pkg.TqWeight()
    used = C.c_size_t(0)
    buf = np.frombuffer(blob + b"tail", dtype=np.uint8)
    assert lib.qwn_tqf_read_qmma(buf.ctypes.data, buf.size, M, K, FLAGS, C.byref(w), C.byref(used)) == 0
    assert used.value == len(blob) and w.scale_cols == cols and w.Mt == M // 16 and w.e2m3 == 1
    got_payload = np.empty_like(payload)
    lib.tq_d2h(got_payload.ctypes.data, w.d_A, payload.nbytes)
    assert np.array_equal(got_payload, payload)
    x = np.random.default_rng(1).standard_normal(K).astype(np.float32)
    res = np.linspace(-1, 1, M).astype(np.float32)
    dx, dr, y = pkg.DevBuf.from_numpy(x), pkg.DevBuf.from_numpy(res), pkg.DevBuf(M * 4)
    assert lib.qwn_x_gemv_qmma(C.byref(w), dx.ptr, y.ptr) == 0
    lib.tq_sync()
    want = orc.gemv_e2m3(payload, bs, cols, M, K, x)
    assert y.to_numpy(np.float32).tobytes() == want.tobytes()
    assert lib.qwn_x_gemv_qmma_add(C.byref(w), dx.ptr, dr.ptr, y.ptr) == 0
    lib.tq_sync()
    assert y.to_numpy(np.float32).tobytes() == (want + res).astype(np.float32).tobytes()
    assert lib.qwn_x_gemv_qmma_prepared(C.byref(w), dx.ptr, y.ptr, None) == 0
    lib.tq_sync()
    assert y.to_numpy(np.float32).tobytes() == want.tobytes()
    # validation of the scalar tier (xpu/src/kernels_core.cpp:170-182)
    w.row_major = 1
    assert lib.qwn_x_gemv_qmma(C.byref(w), dx.ptr, y.ptr) == -4
    w.row_major = 0
    w.scale_rows = 0
    assert lib.qwn_x_gemv_qmma(C.byref(w), dx.ptr, y.ptr) == -6
    w.scale_rows = (M + 127) // 128
    # reader errors
    bad = pkg.TqWeight()
    assert lib.qwn_tqf_read_qmma(buf.ctypes.data, len(blob) - 1, M, K, FLAGS, C.byref(bad), None) == -1
    assert lib.qwn_tqf_read_qmma(buf.ctypes.data, buf.size, M, K, 1 << 5, C.byref(bad), None) == -1
    assert lib.qwn_tqf_read_qmma(buf.ctypes.data, buf.size, M + 8, K, FLAGS, C.byref(bad), None) == -1
    assert lib.qwn_tqf_read_qmma(buf.ctypes.data, buf.size, M, 2 * K, FLAGS, C.byref(bad), None) == -1
    lib.qwn_tqf_free_qmma(C.byref(w))
    assert lib.tq_last_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_w4_check_gate_on_every_repack_mode(lib, pkg, orc, mode):
    """Scalar E2M3 GEMV against the W4A8 GEMV of the repacked weight: cos >= 0.99 in all
    three scale tiers (the reference observed 0.997 on a real matrix)."""
    M, K = 1088, 5120
    blob, *_ = make_record(orc, M, K, seed=40 + mode)
    w = pkg.TqWeight()
    buf = np.frombuffer(blob, dtype=np.uint8)
    assert lib.qwn_tqf_read_qmma(buf.ctypes.data, buf.size, M, K, FLAGS, C.byref(w), None) == 0
    cos, rel = C.c_double(), C.c_double()
    assert lib.qwn_w4_check(C.byref(w), mode, C.byref(cos), C.byref(rel)) == 0
    assert cos.value >= 0.99
    assert w.s4_ready == 1 and w.s4_k16 == (mode == 1) and w.s4_k64 == (mode == 2) and not w.d_A
    assert lib.qwn_w4_check(C.byref(w), mode, None, None) == -2       # already repacked
    lib.qwn_tqf_free_qmma(C.byref(w))


@pytest.mark.gpu
def test_repack_by_policy_and_shard_check_all(lib, pkg, orc):
    """A small projection family read as records, repacked by the environment policy, then
    qwn_shard_check_all in each projection's intended mode (column with row blocks, plain
    column, replicate, row)."""
    shapes = [("in_qkv", 1024, 1024), ("gate", 2176, 1024), ("in_b", 48, 1024), ("down", 1024, 2176 - 128)]
    keep = os.environ.get("TQ_XPU_K64")
    os.environ["TQ_XPU_K64"] = "gate,down"
    ws = []
    try:
        for i, (kind, M, K) in enumerate(shapes):
            blob, *_ = make_record(orc, M, K, seed=70 + i)
            w = pkg.TqWeight()
            buf = np.frombuffer(blob, dtype=np.uint8)
            assert lib.qwn_tqf_read_qmma(buf.ctypes.data, buf.size, M, K, FLAGS, C.byref(w), None) == 0
            tier = lib.qwn_repack_by_policy(C.byref(w), kind.encode())
            assert tier == (2 if kind in ("gate", "down") else 0), (kind, tier)
            assert w.s4_ready == 1 and w.s4_k64 == (tier == 2)
            ws.append(w)
    finally:
        if keep is None:
            os.environ.pop("TQ_XPU_K64", None)
        else:
            os.environ["TQ_XPU_K64"] = keep
    arr = (C.POINTER(pkg.TqWeight) * len(ws))(*[C.pointer(w) for w in ws])
    modes = (C.c_int * 4)(0, 0, 2, 1)
    groups = (C.c_int * 12)(512, 256, 256, 0, 0, 0, 0, 0, 0, 0, 0, 0)
    ngroups = (C.c_int * 4)(3, 0, 0, 0)
    assert lib.qwn_shard_check_all(arr, modes, groups, ngroups, 4) == 0
    # a column shard of the 48-row matrix is impossible (24 rows per rank): counted as a failure
    modes[2] = 0
    assert lib.qwn_shard_check_all(arr, modes, groups, ngroups, 4) == 1
    assert lib.qwn_shard_check(C.byref(ws[1]), 2) == 0           # column + row legs on `gate`
    for w in ws:
        lib.qwn_tqf_free_qmma(C.byref(w))
    assert lib.tq_last_error() == 0


def _gaussian_record(orc, M, K, seed):
    """A record whose decoded weights look like a trained matrix: N(0, 1) values snapped to the
    nearest E2M3 code under one block scale per (128 rows, 128 columns)."""
    rng = np.random.default_rng(seed)
    rows, cols = (M + 127) // 128, (K + 127) // 128
    bs = (rng.random((rows, cols)) * 0.004 + 0.004).astype(np.float32)
    grid = np.array([orc.e2m3f(c) for c in range(64)], dtype=np.float32)
    target = rng.standard_normal((M, K)).astype(np.float32) * 2.0          # in units of the block scale
    codes6 = np.abs(target[..., None] - grid[None, None, :]).argmin(axis=-1).astype(np.uint8)
    payload = orc.e2m3_payload_from_codes_fast(codes6)
    blob = struct.pack("<II", rows, cols) + bs.tobytes() + payload.tobytes()
    return blob, payload, bs, cols


def test_grid_probe_oracle_orders_the_formats(orc):
    """CPU only: on a Gaussian-like matrix more bits reconstruct better, the K16 fit beats the
    K32 fit beats the K64 fit, and asymmetric int4 beats symmetric int4 at the same budget."""
    M, K = 128, 512
    blob, payload, bs, cols = _gaussian_record(orc, M, K, seed=3)
    W = orc.e2m3_decode(payload, bs, cols, M, K)
    cos, rel, bits, verdict = orc.w4_grid_probe(W)
    assert cos[4] > cos[2] > cos[1] > cos[10] and cos[1] > cos[0] and cos[1] > cos[8] and cos[0] > cos[7]
    assert 3.5 <= bits[9] <= 4.5 and cos[8] <= cos[9] <= cos[1] + 1e-12
    assert np.all(rel > 0) and np.all(cos > 0.9) and verdict in (0, 1)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,gauss", [(256, 512, True), (144, 1024, False)])
def test_grid_probe_matches_oracle(lib, pkg, orc, M, K, gauss):
    """Floating-point report: cosine and relative error per format agree with the CPU
    restatement to 2e-5 and 5e-4 (the device sums each row in fp32, the oracle in double); bits per
    weight of the mixed format to 0.01; the verdict whenever the oracle's margin exceeds
    that tolerance."""
    blob, payload, bs, cols = (_gaussian_record if gauss else make_record)(orc, M, K, 5)
    w = pkg.TqWeight()
    buf = np.frombuffer(blob, dtype=np.uint8)
    assert lib.qwn_tqf_read_qmma(buf.ctypes.data, buf.size, M, K, FLAGS, C.byref(w), None) == 0
    cos, rel, bits = (C.c_double * 11)(), (C.c_double * 11)(), (C.c_double * 11)()
    rc = lib.qwn_w4_grid_probe(C.byref(w), cos, rel, bits)
    assert rc in (0, 1) and lib.tq_last_error() == 0
    W = orc.e2m3_decode(payload, bs, cols, M, K)
    ocos, orel, obits, overdict = orc.w4_grid_probe(W)
    assert np.abs(np.array(cos[:]) - ocos).max() <= 2e-5, (list(cos), ocos)
    # |w - w_hat|^2 comes out of fp32 row sums as na - 2 dot + nb: for the int8 format it is 3e-5 of
    # na, so the row sums' rounding shows in the fourth digit of its relative error
    assert np.abs(np.array(rel[:]) - orel).max() <= 5e-4, (list(rel), orel)
    assert np.abs(np.array(bits[:]) - obits).max() <= 0.01
    rivals = [k for k in range(11) if k != 1 and obits[k] <= obits[1] + 1e-9]
    if min(abs(ocos[1] - ocos[k]) for k in rivals) > 1e-4:
        assert rc == overdict
    assert w.d_A and not w.s4_ready                                   # a pure read
    # validation
    w.row_major = 1
    assert lib.qwn_w4_grid_probe(C.byref(w), None, None, None) == -3
    w.row_major = 0
    assert lib.qwn_x_w4_repack_weight_mode(C.byref(w), 0) == 0
    assert lib.qwn_w4_grid_probe(C.byref(w), None, None, None) == -2   # the source is gone
    lib.qwn_tqf_free_qmma(C.byref(w))
