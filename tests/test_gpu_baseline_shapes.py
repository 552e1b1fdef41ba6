"""Parity at the benchmark's own shapes: the five configurations the headline metric is quoted
on, CUDA through the C ABI against the CPU oracle on the same seeded inputs.

Integer layers (codes, code sums, per-(row, k-tile) int32 dots) must be bit-exact; fp32
outputs must be byte-identical to the oracle's fused-multiply-add variant and within 1e-3 of
its separate-multiply-add variant (the tolerance stated for fp32 outputs). Weights are the
benchmark's: seeded N(0, 0.02), symmetric int4 with one FP16 scale per 32 (K32) or 64 (K64)
reduction elements. Shapes follow the reference's naming: M output rows, K reduction, T
tokens (xpu/src/kernels_dpas.cpp:586-675 GEMV, 1334-1490 GEMM).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = 1e-3


def close_1e3(got, want):
    scale = np.abs(want).max() + 1e-30
    return np.abs(got - want).max() <= RTOL * scale


def dev(pkg, a):
    return pkg.DevBuf.from_numpy(np.ascontiguousarray(a))


@pytest.fixture(scope="module")
def w_gate_k32(wl):
    """cfg1 weight: 17408 x 5120, one scale per K32."""
    return wl.make_weight_w4(17408, 5120, seed=11, group=32)


@pytest.fixture(scope="module")
def w_down_k32(wl):
    """cfg3 weight: 5120 x 17408, one scale per K32."""
    return wl.make_weight_w4(5120, 17408, seed=13, group=32)


@pytest.fixture(scope="module")
def w_gate_up_k64(wl):
    """cfg2 / cfg4 weights: gate and up, 17408 x 5120 each, one scale per K64."""
    return [wl.make_weight_w4(17408, 5120, seed=11 + i, group=64) for i in range(2)]


def silu_mul_rows(T, K, seed):
    """cfg3 activations: silu(g) * u with g, u ~ N(0, 1), computed on the host in float64 and
    rounded once (inputs to the quantiser; the fused device SiLU has its own test)."""
    rng = np.random.Generator(np.random.Philox(key=seed))
    g = rng.standard_normal((T, K))
    u = rng.standard_normal((T, K))
    return (g / (1.0 + np.exp(-g)) * u).astype(np.float32)


# ------------------------------------------------------------------------------- cfg1
@pytest.mark.parametrize("per_token", [False, True])
def test_cfg1_gemv_17408x5120(lib, pkg, orc, wl, w_gate_k32, per_token):
    M, K = 17408, 5120
    codes, scales = w_gate_k32
    w = pkg.PackedWeight(codes, scales, M, K)
    assert lib.qwn_choose_gemv_splits(M // 16) == 8
    x = wl.activations_normal(1, K, seed=5)[0]
    dx = dev(pkg, x)
    y = pkg.DevBuf(M * 4)
    y.fill(0xA5)
    if per_token:
        lib.qwn_x_prepare_gemv_act_s8_pertoken(dx.ptr, K)
        assert lib.qwn_x_gemv_w4a8_prepared(w.ref, y.ptr, None) == 0
        q, s, _ = orc.quantize_act_chunk(x[None, :], per_token=True)
        sm = q.astype(np.int32).reshape(-1, 16).sum(axis=1).astype(np.int32)
    else:
        assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y.ptr) == 0
        q, s, sm = orc.quantize_act_s8(x)
    lib.tq_sync()
    # the staging the GEMV consumed
    dq, ds, dsm = pkg.DevBuf(K), pkg.DevBuf(K // 32 * 4), pkg.DevBuf(K // 16 * 4)
    assert lib.qwn_dbg_prepared_act(K, dq.ptr, ds.ptr, dsm.ptr) == 0
    lib.tq_sync()
    assert np.array_equal(dq.to_numpy(np.int8), q)
    assert ds.to_numpy(np.float32).tobytes() == s.tobytes()
    assert np.array_equal(dsm.to_numpy(np.int32), sm)
    # int32 dots of every (row, k-tile)
    dd = pkg.DevBuf((M // 16) * (K // 32) * 16 * 4)
    dd.fill(0xA5)
    assert lib.qwn_dbg_tile_dots_gemv(w.ref, dd.ptr) == 0
    lib.tq_sync()
    assert np.array_equal(dd.to_numpy(np.int32), orc.tile_dots_gemv(codes, M, K, q))
    got = y.to_numpy(np.float32)
    _, want = orc.gemv_w4a8(codes, scales, M, K, 0, q, s, sm, fma=1)
    _, want_sep = orc.gemv_w4a8(codes, scales, M, K, 0, q, s, sm, fma=0)
    assert got.tobytes() == want.tobytes()
    assert close_1e3(got, want_sep)
    assert lib.tq_last_error() == 0


# ------------------------------------------------------------------------------- cfg3
@pytest.mark.parametrize("residual", [False, True])
def test_cfg3_down_gemv_t1(lib, pkg, orc, w_down_k32, residual):
    """T = 1: x_silu_mul_quant then the prepared GEMV (xpu/src/decode.cpp:250-258)."""
    M, K = 5120, 17408
    codes, scales = w_down_k32
    w = pkg.PackedWeight(codes, scales, M, K)
    rng = np.random.Generator(np.random.Philox(key=21))
    gate = rng.standard_normal(K, dtype=np.float32)
    up = rng.standard_normal(K, dtype=np.float32)
    dg, du, hid = dev(pkg, gate), dev(pkg, up), pkg.DevBuf(K * 4)
    lib.qwn_x_silu_mul_quant(hid.ptr, dg.ptr, du.ptr, K)
    res = rng.standard_normal(M, dtype=np.float32) if residual else None
    dr = dev(pkg, res) if residual else None
    y = pkg.DevBuf(M * 4)
    y.fill(0xA5)
    assert lib.qwn_x_gemv_qmma_prepared(w.ref, hid.ptr, y.ptr, dr.ptr if residual else None) == 0
    lib.tq_sync()
    oh, q, s, sm = orc.silu_mul_quant(gate, up)
    assert hid.to_numpy(np.float32).tobytes() == oh.tobytes()
    if not residual:
        dd = pkg.DevBuf((M // 16) * (K // 32) * 16 * 4)
        assert lib.qwn_dbg_tile_dots_gemv(w.ref, dd.ptr) == 0
        lib.tq_sync()
        assert np.array_equal(dd.to_numpy(np.int32), orc.tile_dots_gemv(codes, M, K, q))
    got = y.to_numpy(np.float32)
    _, want = orc.gemv_w4a8(codes, scales, M, K, 0, q, s, sm, residual=res, fma=1)
    _, want_sep = orc.gemv_w4a8(codes, scales, M, K, 0, q, s, sm, residual=res, fma=0)
    assert got.tobytes() == want.tobytes()
    assert close_1e3(got, want_sep)
    assert lib.tq_last_error() == 0


@pytest.mark.parametrize("T,splits", [(8, 8), (16, 4), (32, 2), (64, 1)])
def test_cfg3_down_gemm(lib, pkg, orc, w_down_k32, T, splits):
    """T = 8..64 (T = 2 and 4 are padded to 8 rows by the caller, xpu/src/decode.cpp:2785-2790):
    chunk staging + x_gemm_w4a8 with the split count the reference's rule gives."""
    M, K = 5120, 17408
    codes, scales = w_down_k32
    w = pkg.PackedWeight(codes, scales, M, K)
    assert lib.qwn_choose_gemm_splits(M // 16, T // 8, K // 32) == splits
    x = silu_mul_rows(T, K, seed=31)
    if T == 8:
        x[2:] = 0.0            # a batch of two real rows padded to eight
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    y = pkg.DevBuf(T * M * 4)
    y.fill(0xA5)
    assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, y.ptr, T, None, 0) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x)
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)
    if T == 8:
        dd = pkg.DevBuf(n * M * 4)
        assert lib.qwn_dbg_tile_dots_gemm(w.ref, aq.ptr, T, dd.ptr) == 0
        assert np.array_equal(dd.to_numpy(np.int32), orc.tile_dots_gemm(codes, M, K, oq, T))
    got = y.to_numpy(np.float32).reshape(T, M)
    _, want = orc.gemm_w4a8(codes, scales, M, K, 0, oq, os_, osm, T, fma=1)
    _, want_sep = orc.gemm_w4a8(codes, scales, M, K, 0, oq, os_, osm, T, fma=0)
    assert got.tobytes() == want.tobytes()
    assert close_1e3(got, want_sep)
    # per-token activation scales (what the configuration names): own staging, own kernel mode
    at = pkg.DevBuf(T * 4)
    lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    y.fill(0xA5)
    assert lib.qwn_x_gemm_w4a8_pertoken(w.ref, aq.ptr, at.ptr, asum.ptr, y.ptr, T, 0) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    as_tok = os_.reshape(K // 32, T)[0].copy()
    pt_splits = lib.qwn_choose_pertoken_splits(M // 16, T // 8, K // 32, 0)
    assert pt_splits == {8: 8, 16: 8, 32: 8, 64: 16}[T]      # own rule: see qwn_choose_pertoken_splits
    _, want = orc.gemm_w4a8_pertoken(codes, scales, M, K, 0, oq, as_tok, osm, T, splits=pt_splits)
    assert y.to_numpy(np.float32).tobytes() == want.tobytes()
    assert lib.tq_last_error() == 0


# ------------------------------------------------------------------------------- cfg2
@pytest.mark.parametrize("per_token", [False, True])
def test_cfg2_fused_gate_up_k64_t8(lib, pkg, orc, wl, w_gate_up_k64, per_token):
    """Fused gate|up launch, K64 tier, 8 tokens with 1% outlier channels; the reference's
    per-(token, K32) staging and the per-token staging (scale replicated per K32 block), both
    through x_gemm_w4a8_fanout, each weight keeping the split count it has alone (2)."""
    M, K, T = 17408, 5120, 8
    ws = [pkg.PackedWeight(c, s, M, K, k64=True) for c, s in w_gate_up_k64]
    assert lib.qwn_choose_gemm_splits(M // 16, 1, K // 32) == 2
    x = wl.activations_normal(T, K, seed=5, outlier_frac=0.01)
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    if per_token:
        lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    else:
        lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    ys = [pkg.DevBuf(T * M * 4) for _ in ws]
    for b in ys:
        b.fill(0xA5)
    assert lib.qwn_x_gemm_w4a8_fanout(pkg.weight_array(ws), pkg.ptr_array(ys), 2, aq.ptr, as_.ptr,
                                      asum.ptr, T, None, 0) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x, per_token=per_token)
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)
    for (codes, scales), w, yb in zip(w_gate_up_k64, ws, ys):
        got = yb.to_numpy(np.float32).reshape(T, M)
        _, want = orc.gemm_w4a8(codes, scales, M, K, 1, oq, os_, osm, T, fma=1)
        _, want_sep = orc.gemm_w4a8(codes, scales, M, K, 1, oq, os_, osm, T, fma=0)
        assert got.tobytes() == want.tobytes()
        assert close_1e3(got, want_sep)
    if per_token:
        # the per-token kernel proper: one promote per K64 group, as_tok applied at the end
        for b in ys:
            b.fill(0xA5)
        assert lib.qwn_x_gemm_w4a8_fanout_pertoken(pkg.weight_array(ws), pkg.ptr_array(ys), 2, aq.ptr,
                                                   at.ptr, asum.ptr, T) == 0
        lib.tq_sync()
        as_tok = os_.reshape(K // 32, T)[0].copy()
        for (codes, scales), yb in zip(w_gate_up_k64, ys):
            _, want = orc.gemm_w4a8_pertoken(codes, scales, M, K, 1, oq, as_tok, osm, T, splits=2)
            assert yb.to_numpy(np.float32).tobytes() == want.tobytes()
    # int32 layer of the gate matrix
    dd = pkg.DevBuf(n * M * 4)
    assert lib.qwn_dbg_tile_dots_gemm(ws[0].ref, aq.ptr, T, dd.ptr) == 0
    assert np.array_equal(dd.to_numpy(np.int32),
                          orc.tile_dots_gemm(w_gate_up_k64[0][0], M, K, oq, T))
    assert lib.tq_last_error() == 0


# ------------------------------------------------------------------------------- cfg4
CFG4_OFFSETS = [0, 1024, 2048, 3072, 4096]
CFG4_SAMPLE_GROUPS = 40        # 40 row-groups = 640 rows of the 17408 are checked, all tokens


def _bf16_rne(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _sample(codes, scales, M, K, ksh, seed):
    """A seeded sample of whole 16-row groups of a packed weight as a smaller packed weight
    (rows are independent, so the oracle on the sample gives those rows of the full result)."""
    rng = np.random.default_rng(seed)
    groups = np.sort(rng.choice(M // 16, size=CFG4_SAMPLE_GROUPS, replace=False))
    Kt = K // 32
    c = codes.reshape(M // 16, Kt * 256)[groups].reshape(-1)
    s = scales.reshape(M // 16, (Kt >> ksh) * 16)[groups].reshape(-1)
    rows = (groups[:, None] * 16 + np.arange(16)[None, :]).reshape(-1)
    return c, s, rows


@pytest.fixture(scope="module")
def cfg4_inputs(wl):
    return wl.activations_normal(4096, 5120, seed=7)


@pytest.mark.parametrize("mode", ["exact_fp32", "pertoken_fp32", "pertoken_bf16", "w4a4"])
def test_cfg4_prefill_4096_tokens(lib, pkg, orc, w_gate_up_k64, cfg4_inputs, mode):
    """Packed prefill: 4096 tokens in four segments of 1024, K64 weights, on the tcgen05
    kernel. The oracle checks a seeded sample of 640 rows x all 4096 tokens (each segment is
    unsplit for the sample exactly as for the full weight, asserted below)."""
    M, K, T, ksh = 17408, 5120, 4096, 1
    codes, scales = w_gate_up_k64[0]
    w = pkg.PackedWeight(codes, scales, M, K, k64=True)
    x = cfg4_inputs
    dx = dev(pkg, x)
    sc, ss, rows = _sample(codes, scales, M, K, ksh, seed=3)
    Ms = rows.size
    for rg in (M // 16, Ms // 16):
        assert lib.qwn_choose_gemm_splits(rg, 1024 // 8, K // 32) == 1
    off = (C.c_int * 5)(*CFG4_OFFSETS)
    if mode == "w4a4":
        n = K // 64 * T
        aq4, as4, asum4 = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
        lib.qwn_x_quantize_act_chunk_s4(dx.ptr, K, T, aq4.ptr, as4.ptr, asum4.ptr)
        y = pkg.DevBuf(T * M * 4)
        assert lib.qwn_x_gemm_w4a4(w.ref, aq4.ptr, as4.ptr, asum4.ptr, y.ptr, T) == 0
        lib.tq_sync()
        oq, os_, osm = orc.quantize_act_chunk_s4(x)
        assert np.array_equal(aq4.to_numpy(np.uint8), oq)
        assert as4.to_numpy(np.float32).tobytes() == os_.tobytes()
        assert np.array_equal(asum4.to_numpy(np.int32), osm)
        got = y.to_numpy(np.float32).reshape(T, M)[:, rows]
        _, want = orc.gemm_w4a4(sc, ss, Ms, K, oq, os_, osm, T, fma=1)
        _, want_sep = orc.gemm_w4a4(sc, ss, Ms, K, oq, os_, osm, T, fma=0)
        assert got.tobytes() == want.tobytes()
        assert close_1e3(got, want_sep)
    else:
        n = K // 32 * T
        aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
        if mode == "exact_fp32":
            lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
            y = pkg.DevBuf(T * M * 4)
            assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, y.ptr, T, off, 4) == 0
            lib.tq_sync()
            oq, os_, osm = orc.quantize_act_chunk(x)
            assert np.array_equal(aq.to_numpy(np.int8), oq)
            assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
            assert np.array_equal(asum.to_numpy(np.int32), osm)
            got = y.to_numpy(np.float32).reshape(T, M)[:, rows]
            _, want = orc.gemm_w4a8(sc, ss, Ms, K, ksh, oq, os_, osm, T, offsets=CFG4_OFFSETS, fma=1)
            _, want_sep = orc.gemm_w4a8(sc, ss, Ms, K, ksh, oq, os_, osm, T, offsets=CFG4_OFFSETS,
                                        fma=0)
            assert got.tobytes() == want.tobytes()
            assert close_1e3(got, want_sep)
        else:
            bf16 = mode.endswith("bf16")
            lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
            y = pkg.DevBuf(T * M * (2 if bf16 else 4))
            assert lib.qwn_x_gemm_w4a8_pertoken(w.ref, aq.ptr, at.ptr, asum.ptr, y.ptr, T,
                                                int(bf16)) == 0
            lib.tq_sync()
            oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
            as_tok = os_.reshape(K // 32, T)[0].copy()
            assert np.array_equal(aq.to_numpy(np.int8), oq)
            assert at.to_numpy(np.float32).tobytes() == as_tok.tobytes()
            _, want = orc.gemm_w4a8_pertoken(sc, ss, Ms, K, ksh, oq, as_tok, osm, T)
            if bf16:
                got = y.to_numpy(np.uint16).reshape(T, M)[:, rows]
                assert np.array_equal(got, _bf16_rne(want).reshape(T, Ms))
            else:
                got = y.to_numpy(np.float32).reshape(T, M)[:, rows]
                assert got.tobytes() == want.tobytes()
    assert lib.tq_last_error() == 0
