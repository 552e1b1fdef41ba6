"""GPU parity: every CUDA entry point against the CPU oracle on the same seeded inputs,
called through the C-ABI. Integer layers (codes, sums, tile dots) must be bit-exact. fp32
outputs are compared bit-for-bit with the oracle's fused-multiply-add variant (the kernels
use explicit fmaf in the same order) and within 1e-3 of its separate-multiply-add variant
(the tolerance stated for fp32 outputs)."""
import ctypes as C

import numpy as np
import pytest

import refgen

pytestmark = pytest.mark.gpu

RTOL = 1e-3   # stated fp32 tolerance against the reference semantics


def close_1e3(got, want):
    scale = np.abs(want).max() + 1e-30
    return np.abs(got - want).max() <= RTOL * scale


def dev(pkg, a):
    return pkg.DevBuf.from_numpy(np.ascontiguousarray(a))


def prepared(lib, pkg, K):
    q, s, sm = pkg.DevBuf(K), pkg.DevBuf(K // 32 * 4), pkg.DevBuf(K // 16 * 4)
    assert lib.qwn_dbg_prepared_act(K, q.ptr, s.ptr, sm.ptr) == 0
    lib.tq_sync()
    return q.to_numpy(np.int8), s.to_numpy(np.float32), sm.to_numpy(np.int32)


# ---------------------------------------------------------------- quantisers
@pytest.mark.parametrize("K", [32, 5120, 17408])
def test_quantize_act_s8(lib, pkg, orc, K):
    x = refgen.lcg_floats(K)[0] if K <= 5120 else np.random.default_rng(K).standard_normal(K).astype(np.float32)
    x[:32] = 0.0
    dx = dev(pkg, x)
    q, s, sm = pkg.DevBuf(K), pkg.DevBuf(K // 32 * 4), pkg.DevBuf(K // 16 * 4)
    for b in (q, s, sm):
        b.fill(0xA5)
    lib.qwn_x_quantize_act_s8(dx.ptr, K, q.ptr, s.ptr, sm.ptr)
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_s8(x)
    assert np.array_equal(q.to_numpy(np.int8), oq)
    assert s.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(sm.to_numpy(np.int32), osm)
    lib.qwn_x_prepare_gemv_act_s8(dx.ptr, K)
    pq, ps, psm = prepared(lib, pkg, K)
    assert np.array_equal(pq, oq) and ps.tobytes() == os_.tobytes() and np.array_equal(psm, osm)


@pytest.mark.parametrize("K,T,exceptional", [(128, 16, True), (128, 16, False), (5120, 8, False),
                                             (256, 40, True),
                                             # 64 tokens and more: the wide kernel (K % 128 == 0) ...
                                             (128, 67, True), (5120, 136, False), (17408, 64, False),
                                             # ... and the block-per-warp one where a row does not split
                                             (160, 70, True)])
def test_quantize_act_chunk(lib, pkg, orc, K, T, exceptional):
    x = refgen.chunk_quant_probe_input(K, T, exceptional)
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    for b in (aq, as_, asum):
        b.fill(0xA5)                      # poison: a missed store fails the comparison
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x)
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)


# one fused launch up to 64 tokens; above, one CTA per token with the row in registers (rows up
# to 8192 values) or the row maxima and then the wide kernel
@pytest.mark.parametrize("T,K", [(8, 5120), (16, 5120), (40, 5120), (72, 5120), (136, 5120), (65, 17408),
                                 (70, 8224)])
def test_quantize_act_chunk_pertoken(lib, pkg, orc, wl, T, K):
    x = wl.activations_normal(T, K, seed=2, outlier_frac=0.01)
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)
    assert at.to_numpy(np.float32).tobytes() == os_.reshape(K // 32, T)[0].tobytes()


def test_chunk_staging_from_a_row_that_is_not_16_byte_aligned(lib, pkg, orc, wl):
    """The wide kernels load 16 bytes per lane; rows that start 4 bytes off go to the kernels
    that do not, with the same result."""
    K, T = 256, 80
    x = wl.activations_normal(T, K, seed=4, outlier_frac=0.01)
    buf = pkg.DevBuf.from_numpy(np.concatenate([np.zeros(1, np.float32), x.reshape(-1), np.zeros(3, np.float32)]))
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    lib.qwn_x_quantize_act_chunk(buf.ptr + 4, K, T, aq.ptr, as_.ptr, asum.ptr)
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x)
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)
    lib.qwn_x_quantize_act_chunk_pertoken(buf.ptr + 4, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)
    assert lib.tq_last_error() == 0


# a cluster of 8 / 4 / 2 CTAs where the row divides into K32-aligned slices of at most 1024
# values (one launch), two launches elsewhere (352, 17408). Rows stay below 32768 values: a
# later test needs the library's staging scratch to be smaller than that.
@pytest.mark.parametrize("K", [64, 128, 352, 5120, 8192, 17408])
@pytest.mark.parametrize("silu", [False, True])
def test_single_row_pertoken_staging_and_gemv(lib, pkg, orc, wl, K, silu):
    """One scale for the whole row: codes, scale slots and K16 sums against the oracle; the
    permuted tile and the K32 sums through the GEMV that reads them."""
    rng = np.random.default_rng(K + silu)
    x = rng.standard_normal(K).astype(np.float32)
    x[:32] = 0.0
    x[K // 2] = -37.5
    if silu:
        up = rng.standard_normal(K).astype(np.float32)
        dg, du, hid = dev(pkg, x), dev(pkg, up), pkg.DevBuf(K * 4)
        hid.fill(0xFF)
        lib.qwn_x_silu_mul_quant_pertoken(hid.ptr, dg.ptr, du.ptr, K)
        row = orc.silu_mul(x, up)
        lib.tq_sync()
        assert hid.to_numpy(np.float32).tobytes() == row.tobytes()
    else:
        dx = dev(pkg, x)
        lib.qwn_x_prepare_gemv_act_s8_pertoken(dx.ptr, K)
        row = x
    q, s, sm = prepared(lib, pkg, K)
    oq, os_, _ = orc.quantize_act_chunk(row[None, :], per_token=True)
    osm = oq.astype(np.int32).reshape(-1, 16).sum(axis=1).astype(np.int32)
    assert np.array_equal(q, oq.reshape(-1))
    assert s.tobytes() == os_.tobytes()
    assert np.array_equal(sm, osm)
    if K % 128 == 0:
        M = 32
        codes, scales = wl.random_packed_weight(M, K, seed=K, ksh=0)
        w = pkg.PackedWeight(codes, scales, M, K)
        y = pkg.DevBuf(M * 4)
        y.fill(0xFF)
        assert lib.qwn_x_gemv_w4a8_prepared(w.ref, y.ptr, None) == 0
        lib.tq_sync()
        _, want = orc.gemv_w4a8(codes, scales, M, K, 0, oq.reshape(-1), os_.reshape(-1), osm, fma=1)
        assert y.to_numpy(np.float32).tobytes() == want.tobytes()
    assert lib.tq_last_error() == 0


def test_silu_mul_quant_fused_equals_unfused_and_oracle(lib, pkg, orc):
    rng = np.random.default_rng(5)
    K = 17408
    gate = ((rng.random(K) * 2 - 1) * 8).astype(np.float32)
    up = ((rng.random(K) * 2 - 1) * 4).astype(np.float32)
    gate[:32] = 0.0
    gate[0] = -0.0
    gate[32], gate[33] = -100.0, 100.0
    up[64:96] *= np.float32(1e-20)
    dg, du = dev(pkg, gate), dev(pkg, up)
    h0, h1 = pkg.DevBuf(K * 4), pkg.DevBuf(K * 4)
    lib.qwn_x_silu_mul(h0.ptr, dg.ptr, du.ptr, K)
    lib.qwn_x_prepare_gemv_act_s8(h0.ptr, K)
    a = prepared(lib, pkg, K)
    lib.qwn_x_silu_mul_quant(h1.ptr, dg.ptr, du.ptr, K)
    b = prepared(lib, pkg, K)
    assert h0.to_numpy(np.float32).tobytes() == h1.to_numpy(np.float32).tobytes()
    assert all(np.array_equal(u, v) for u, v in zip(a, b))
    oh, oq, os_, osm = orc.silu_mul_quant(gate, up)
    assert h1.to_numpy(np.float32).tobytes() == oh.tobytes()
    assert np.array_equal(b[0], oq) and b[1].tobytes() == os_.tobytes() and np.array_equal(b[2], osm)


@pytest.mark.parametrize("H", [5120, 352])
def test_rmsnorm_quant(lib, pkg, orc, H):
    rng = np.random.default_rng(6)
    x = (rng.standard_normal(H) * 3).astype(np.float32)
    w = ((rng.standard_normal(H) * 0.1).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    dx, dw, out = dev(pkg, x), dev(pkg, w), pkg.DevBuf(H * 4)
    lib.qwn_x_rmsnorm_quant(out.ptr, dx.ptr, dw.ptr, H, 1e-6)
    q, s, sm = prepared(lib, pkg, H)
    oo, oq, os_, osm = orc.rmsnorm_quant(x, w, 1e-6)
    assert out.to_numpy(np.float32).tobytes() == oo.tobytes()
    assert np.array_equal(q, oq) and s.tobytes() == os_.tobytes() and np.array_equal(sm, osm)


# ---------------------------------------------------------------- repack / shard
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("k32_scales", [False, True])
def test_repack_bit_exact(lib, pkg, orc, mode, k32_scales):
    rng = np.random.default_rng(7 + mode)
    M, K = 128, 512
    codes6 = rng.integers(0, 64, size=(M, K), dtype=np.uint8)
    Kt = K // 32
    sc = Kt if k32_scales else Kt // 4
    bs = (rng.random(((M + 127) // 128, sc)) * 0.01 + 0.002).astype(np.float32)
    payload = orc.e2m3_payload_from_codes_fast(codes6)
    w = pkg.TqWeight()
    w.M, w.K, w.Mt, w.Kt = M, K, M // 16, Kt
    w.block_scaled, w.e2m3, w.scale_rows, w.scale_cols = 1, 1, (M + 127) // 128, sc
    w.d_A = lib.tq_dev_alloc(payload.nbytes, b"t.payload")
    w.d_block_scale_inv = lib.tq_dev_alloc(bs.nbytes, b"t.bs")
    lib.tq_h2d(w.d_A, payload.ctypes.data, payload.nbytes)
    lib.tq_h2d(w.d_block_scale_inv, bs.ctypes.data, bs.nbytes)
    assert lib.qwn_x_w4_repack_weight_mode(C.byref(w), mode) == 0
    assert w.s4_ready == 1 and w.s4_k16 == (mode == 1) and w.s4_k64 == (mode == 2)
    assert not w.d_A and not w.d_block_scale_inv
    rc, oc, osc = orc.w4_repack(payload, bs, sc, M, K, mode)
    assert rc == 0
    gc = np.empty_like(oc)
    gs = np.empty_like(osc)
    lib.tq_d2h(gc.ctypes.data, w.d_s4, gc.nbytes)
    lib.tq_d2h(gs.ctypes.data, w.d_s4_scale, gs.nbytes)
    assert np.array_equal(gs, osc)
    assert np.array_equal(gc, oc)
    lib.qwn_x_w4_shard_free(C.byref(w))


def test_repack_errors(lib, pkg):
    w = pkg.TqWeight()
    assert lib.qwn_x_w4_repack_weight_mode(C.byref(w), 0) == -1
    w.d_A = w.d_block_scale_inv = 1
    w.block_scaled = w.e2m3 = 1
    w.M, w.K, w.Mt, w.Kt = 24, 128, 1, 4
    assert lib.qwn_x_w4_repack_weight(C.byref(w)) == -2
    w.M, w.K, w.Kt = 32, 96, 3
    assert lib.qwn_x_w4_repack_weight(C.byref(w)) == -2


@pytest.mark.parametrize("tp,groups", [(2, None), (4, None), (8, None), (2, [512, 256, 256])])
def test_shard_matches_oracle_and_concat_bit_identical(lib, pkg, orc, wl, tp, groups):
    M, K, ksh = 1024, 1024, 1   # every shard keeps > 4 row-groups, so the split count is unchanged
    codes, scales = wl.random_packed_weight(M, K, seed=21, ksh=ksh)
    w = pkg.PackedWeight(codes, scales, M, K, k64=True)
    x = refgen.shard_check_row(K)
    dx = dev(pkg, x)
    lib.qwn_x_prepare_gemv_act_s8(dx.ptr, K)
    full = pkg.DevBuf(M * 4)
    assert lib.qwn_x_gemv_w4a8_prepared(w.ref, full.ptr, None) == 0
    got = pkg.DevBuf(M * 4)
    garr = (C.c_int * len(groups))(*groups) if groups else None
    for r in range(tp):
        s = pkg.TqWeight()
        assert lib.qwn_x_w4_shard(C.byref(s), w.ref, r, tp, 0, garr, len(groups) if groups else 0) == 0
        rc, oc, osc = orc.w4_shard_column(codes, scales, M, K, ksh, r, tp, groups)
        gc, gs = np.empty_like(oc), np.empty_like(osc)
        lib.tq_d2h(gc.ctypes.data, s.d_s4, gc.nbytes)
        lib.tq_d2h(gs.ctypes.data, s.d_s4_scale, gs.nbytes)
        assert np.array_equal(gc, oc) and np.array_equal(gs, osc) and s.M == M // tp
        assert lib.qwn_x_gemv_w4a8_prepared(C.byref(s), got.ptr + r * (M // tp) * 4, None) == 0
        lib.tq_sync()
        lib.qwn_x_w4_shard_free(C.byref(s))
    part = got.to_numpy(np.float32)
    gsz = groups or [M]
    out = np.empty(M, np.float32)
    base = 0
    cur = [r * (M // tp) for r in range(tp)]
    for g in gsz:
        per = g // tp
        for r in range(tp):
            out[base + r * per: base + (r + 1) * per] = part[cur[r]: cur[r] + per]
            cur[r] += per
        base += g
    assert out.tobytes() == full.to_numpy(np.float32).tobytes()
    if not groups:
        assert lib.qwn_shard_check(w.ref, tp) == 0
    s = pkg.TqWeight()
    assert lib.qwn_x_w4_shard(C.byref(s), w.ref, 0, 3, 0, None, 0) == -6
    assert lib.qwn_x_w4_shard(C.byref(s), w.ref, 5, 2, 0, None, 0) == -2
    assert lib.qwn_x_w4_shard(C.byref(s), w.ref, 0, 2, 3, None, 0) == -9


# ---------------------------------------------------------------- GEMV
GEMV_SHAPES = [(64, 256, 0), (48, 384, 1), (16, 128, 0), (16, 128, 1), (272, 5120, 0),
               (5120, 1024, 1), (65536 + 16, 64, 0)]


@pytest.mark.parametrize("M,K,ksh", GEMV_SHAPES)
def test_gemv_int32_dots_and_fp32(lib, pkg, orc, wl, M, K, ksh):
    codes, scales = wl.random_packed_weight(M, K, seed=M * 7 + K, ksh=ksh)
    w = pkg.PackedWeight(codes, scales, M, K, k64=bool(ksh))
    x = refgen.lcg_floats(K, seed=391 + M)[0]
    x[:32] = 0.0
    dx = dev(pkg, x)
    y = pkg.DevBuf(M * 4)
    y.fill(0xA5)
    assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y.ptr) == 0
    lib.tq_sync()
    q, s, sm = orc.quantize_act_s8(x)
    # int32 layer, from the same unpack + dp4a code path
    dd = pkg.DevBuf((M // 16) * (K // 32) * 16 * 4)
    dd.fill(0xA5)
    assert lib.qwn_dbg_tile_dots_gemv(w.ref, dd.ptr) == 0
    lib.tq_sync()
    assert np.array_equal(dd.to_numpy(np.int32), orc.tile_dots_gemv(codes, M, K, q))
    got = y.to_numpy(np.float32)
    _, want_fma = orc.gemv_w4a8(codes, scales, M, K, ksh, q, s, sm, fma=1)
    _, want_sep = orc.gemv_w4a8(codes, scales, M, K, ksh, q, s, sm, fma=0)
    assert got.tobytes() == want_fma.tobytes()
    assert close_1e3(got, want_sep)
    # residual forms
    res = np.linspace(-3, 3, M).astype(np.float32)
    dr = dev(pkg, res)
    assert lib.qwn_x_gemv_w4a8_add(w.ref, dx.ptr, dr.ptr, y.ptr) == 0
    lib.tq_sync()
    _, want_res = orc.gemv_w4a8(codes, scales, M, K, ksh, q, s, sm, residual=res, fma=1)
    assert y.to_numpy(np.float32).tobytes() == want_res.tobytes()
    assert lib.qwn_x_gemv_qmma_prepared(w.ref, dx.ptr, y.ptr, dr.ptr) == 0
    lib.tq_sync()
    assert y.to_numpy(np.float32).tobytes() == want_res.tobytes()
    assert lib.tq_last_error() == 0


@pytest.mark.parametrize("Ms,K,ksh", [([64, 64], 256, 0), ([160, 96, 48, 48], 384, 1),
                                      ([16, 48], 128, 0), ([1088, 1088], 1024, 1)])
def test_gemv_fanout(lib, pkg, orc, wl, Ms, K, ksh):
    ws, host = [], []
    for i, M in enumerate(Ms):
        c, s = wl.random_packed_weight(M, K, seed=100 + i, ksh=ksh)
        host.append((c, s, M))
        ws.append(pkg.PackedWeight(c, s, M, K, k64=bool(ksh)))
    x = refgen.lcg_floats(K)[0]
    dx = dev(pkg, x)
    lib.qwn_x_prepare_gemv_act_s8(dx.ptr, K)
    ys = [pkg.DevBuf(M * 4) for M in Ms]
    for b in ys:
        b.fill(0xA5)
    assert lib.qwn_x_gemv_w4a8_fanout(pkg.weight_array(ws), pkg.ptr_array(ys), len(ws)) == 0
    lib.tq_sync()
    q, s, sm = orc.quantize_act_s8(x)
    rc, want = orc.gemv_w4a8_fanout(host, K, ksh, q, s, sm, fma=1)
    rc2, want_sep = orc.gemv_w4a8_fanout(host, K, ksh, q, s, sm, fma=0)
    for b, w1, w0 in zip(ys, want, want_sep):
        got = b.to_numpy(np.float32)
        assert got.tobytes() == w1.tobytes()
        assert close_1e3(got, w0)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,res", [(64, 256, False), (48, 384, True), (16, 128, True), (272, 5120, False),
                                     (5120, 1056, True), (65536 + 16, 64, True)])
def test_gemv_k16_tier(lib, pkg, orc, wl, M, K, res):
    """K16 scale tier (x_gemv_w4a8_core_k16): one scale, zero point and code sum per 16 codes,
    one accumulator per split; x_gemv_w4a8(_add) and the x_gemv_qmma shim route to it.
    Bit-identical to the oracle (contracted form), within 1e-3 of the uncontracted one."""
    codes, scales = wl.random_packed_weight(M, K, seed=M + K, k16=True)
    w = pkg.PackedWeight(codes, scales, M, K, k16=True)
    x = refgen.lcg_floats(K, seed=17 + M)[0]
    x[:16] = 0.0
    dx = dev(pkg, x)
    r = refgen.lcg_floats(M, seed=5)[0] if res else None
    dr = dev(pkg, r) if res else None
    y = pkg.DevBuf(M * 4)
    y.fill(0xA5)
    if res:
        assert lib.qwn_x_gemv_w4a8_add(w.ref, dx.ptr, dr.ptr, y.ptr) == 0
    else:
        assert lib.qwn_x_gemv_qmma(w.ref, dx.ptr, y.ptr) == 0
    lib.tq_sync()
    q, s, sm = orc.quantize_act_s8(x)
    want = orc.gemv_w4a8_k16(codes, scales, M, K, q, s, sm, residual=r, fma=1)
    want0 = orc.gemv_w4a8_k16(codes, scales, M, K, q, s, sm, residual=r, fma=0)
    got = y.to_numpy(np.float32)
    assert got.tobytes() == want.tobytes()
    assert close_1e3(got, want0)
    # the prepared form gives the same bits; the GEMM does not take this tier
    y2 = pkg.DevBuf(M * 4)
    assert lib.qwn_x_gemv_w4a8_prepared(w.ref, y2.ptr, dr.ptr if res else None) == 0
    lib.tq_sync()
    assert y2.to_numpy(np.float32).tobytes() == want.tobytes()
    assert lib.tq_last_error() == 0


def test_gemv_errors(lib, pkg, wl):
    M, K = 32, 128
    c, s = wl.random_packed_weight(M, K, seed=1)
    w = pkg.PackedWeight(c, s, M, K)
    y = pkg.DevBuf(M * 4)
    x = pkg.DevBuf(K * 4)
    assert lib.qwn_x_gemv_w4a8(None, x.ptr, y.ptr) == -1
    assert lib.qwn_x_gemv_w4a8(w.ref, None, y.ptr) == -1
    w.rec.s4_ready = 0
    assert lib.qwn_x_gemv_w4a8_prepared(w.ref, y.ptr, None) == -1
    w.rec.s4_ready = 1
    big = pkg.PackedWeight(c, s, 16, 1 << 20)        # K larger than anything prepared
    assert lib.qwn_x_gemv_w4a8_prepared(big.ref, y.ptr, None) == -2
    w2 = pkg.PackedWeight(c, s, M, 256)
    assert lib.qwn_x_gemv_w4a8_fanout(pkg.weight_array([w, w2]), pkg.ptr_array([y, y]), 2) == -2
    assert lib.qwn_x_gemv_w4a8_fanout(pkg.weight_array([w]), pkg.ptr_array([y]), 5) == -1
    w.rec.s8_ready = 1                                   # flagged W8A8 but no W8 buffers
    assert lib.qwn_x_gemv_qmma(w.ref, x.ptr, y.ptr) == -1
    w.rec.s8_ready = w.rec.s4_ready = 0                  # scalar E2M3 tier, but no payload
    assert lib.qwn_x_gemv_qmma(w.ref, x.ptr, y.ptr) == -3


# ---------------------------------------------------------------- GEMM
GEMM_CASES = [
    (64, 512, 0, 8, None), (64, 512, 1, 16, None), (48, 384, 0, 24, None),
    (64, 512, 0, 32, [0, 8, 32]), (64, 512, 1, 64, [0, 8, 16, 40, 64]),
    (320, 1024, 0, 8, None), (2176, 256, 1, 8, None), (16, 128, 0, 8, None),
    (128, 256, 0, 136, None), (5120, 512, 0, 64, None),
    (2048, 512, 0, 64, [0, 8, 64]),      # segments with different split counts (16 and 4)
    # streaming kernel: several row-groups per warp team, a ragged last ring stage
    (40000, 320, 1, 8, None),
    # K64 splits that start on an odd k-tile, odd tile counts, two token groups
    (4800, 2112, 1, 16, None),
    # five token groups, 8 splits of 4..5 tiles
    (1600, 1056, 0, 40, None),
    (1088, 5120, 1, 8, None),
    # T = 8 ring kernel: K64 splits that start on odd k-tiles (a tile pair then has two scale
    # lines), K32 with full stages plus a one-tile last stage, 17-tile splits
    (4800, 2112, 1, 8, None), (320, 2112, 0, 8, None), (1088, 1056, 0, 8, None),
    # tcgen05 path: unsplit, T >= 128, rows a multiple of 128; ragged token tail; segments
    (2048, 512, 0, 128, None), (1024, 1024, 1, 256, None), (2048, 256, 0, 136, None),
    (2048, 512, 1, 256, [0, 128, 256]),
]


@pytest.mark.parametrize("M,K,ksh,T,offsets", GEMM_CASES)
def test_gemm_int32_dots_and_fp32(lib, pkg, orc, wl, M, K, ksh, T, offsets):
    codes, scales = wl.random_packed_weight(M, K, seed=M + K + T, ksh=ksh)
    w = pkg.PackedWeight(codes, scales, M, K, k64=bool(ksh))
    x = refgen.gemm_check_rows(T, K)
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    y = pkg.DevBuf(T * M * 4)
    y.fill(0xA5)
    off = (C.c_int * len(offsets))(*offsets) if offsets else None
    nseg = len(offsets) - 1 if offsets else 0
    assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, y.ptr, T, off, nseg) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x)
    dd = pkg.DevBuf(n * M * 4)
    dd.fill(0xA5)
    assert lib.qwn_dbg_tile_dots_gemm(w.ref, aq.ptr, T, dd.ptr) == 0
    assert np.array_equal(dd.to_numpy(np.int32), orc.tile_dots_gemm(codes, M, K, oq, T))
    got = y.to_numpy(np.float32).reshape(T, M)
    _, want = orc.gemm_w4a8(codes, scales, M, K, ksh, oq, os_, osm, T, offsets=offsets, fma=1)
    _, want_sep = orc.gemm_w4a8(codes, scales, M, K, ksh, oq, os_, osm, T, offsets=offsets, fma=0)
    assert got.tobytes() == want.tobytes()
    assert close_1e3(got, want_sep)
    assert lib.tq_last_error() == 0


def test_gemm_fanout_equals_per_weight(lib, pkg, orc, wl):
    K, T, ksh = 512, 8, 1
    Ms = [1088, 1088]
    ws = [pkg.PackedWeight(*wl.random_packed_weight(M, K, seed=40 + i, ksh=ksh), M, K, k64=True)
          for i, M in enumerate(Ms)]
    x = wl.activations_normal(T, K, seed=4, outlier_frac=0.01)
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    ys = [pkg.DevBuf(T * M * 4) for M in Ms]
    assert lib.qwn_x_gemm_w4a8_fanout(pkg.weight_array(ws), pkg.ptr_array(ys), 2, aq.ptr, as_.ptr,
                                      asum.ptr, T, None, 0) == 0
    for w, yb, M in zip(ws, ys, Ms):
        y1 = pkg.DevBuf(T * M * 4)
        assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, y1.ptr, T, None, 0) == 0
        lib.tq_sync()
        assert yb.to_numpy(np.float32).tobytes() == y1.to_numpy(np.float32).tobytes()


def test_gemm_errors(lib, pkg, wl):
    M, K = 16, 128
    w = pkg.PackedWeight(*wl.random_packed_weight(M, K, seed=1), M, K)
    b = pkg.DevBuf(8 * K * 4)
    bad = (C.c_int * 3)(0, 4, 8)
    assert lib.qwn_x_gemm_w4a8(w.ref, b.ptr, b.ptr, b.ptr, b.ptr, 12, None, 0) == -2
    assert lib.qwn_x_gemm_w4a8(w.ref, b.ptr, b.ptr, b.ptr, b.ptr, 8, bad, 2) == -2
    assert lib.qwn_x_gemm_w4a8(w.ref, b.ptr, b.ptr, b.ptr, b.ptr, 8, None, 1) == -2
    assert lib.qwn_x_gemm_w4a8(w.ref, None, b.ptr, b.ptr, b.ptr, 8, None, 0) == -2
    w.rec.s4_k16 = 1
    assert lib.qwn_x_gemm_w4a8(w.ref, b.ptr, b.ptr, b.ptr, b.ptr, 8, None, 0) == -1


def test_reference_gates_on_synthetic_weight(lib, pkg, wl):
    """qwn_gemm_check (cos >= 0.9999), qwn_specwave_check (byte-identical prefix rows)."""
    M, K = 1088, 5120
    for ksh in (0, 1):
        c, s = wl.make_weight_w4(M, K, seed=9, group=32 << ksh)
        w = pkg.PackedWeight(c, s, M, K, k64=bool(ksh))
        cos, rel = C.c_double(), C.c_double()
        for T in (8, 32):
            assert lib.qwn_gemm_check(w.ref, T, C.byref(cos), C.byref(rel)) == 0
            assert cos.value >= 0.9999
        assert lib.qwn_specwave_check(w.ref) == 0
        assert lib.qwn_gemv_bench(w.ref, 5) > 0 and lib.qwn_gemm_bench(w.ref, 8, 5) > 0


# ---------------------------------------------------------------- fused all-gather (1 rank)
@pytest.mark.gpu
def test_gathered_gemm_single_rank(lib, pkg, orc, wl):
    """World of one: the peer-store epilogue, the step flag and the bounded wait kernel run
    against this GPU's own buffers; both halves of the gathered buffer are exercised and
    the result is bit-identical to the plain fan-out call."""
    K, T, ksh = 512, 8, 1
    Ms = [1088, 544]
    ws = [pkg.PackedWeight(*wl.random_packed_weight(M, K, seed=70 + i, ksh=ksh), M, K, k64=True)
          for i, M in enumerate(Ms)]
    x = refgen.gemm_check_rows(T, K)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    dx = dev(pkg, x)          # stays alive until the asynchronous calls below have run
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    ys = [pkg.DevBuf(T * M * 4) for M in Ms]
    assert lib.qwn_x_gemm_w4a8_fanout(pkg.weight_array(ws), pkg.ptr_array(ys), 2, aq.ptr, as_.ptr,
                                      asum.ptr, T, None, 0) == 0
    want = np.concatenate([y.to_numpy(np.float32) for y in ys])
    block = T * sum(Ms)
    gathered = pkg.DevBuf(2 * block * 4)
    gathered.fill(0xA5)
    flags = pkg.DevBuf(4)
    lib.tq_dev_zero(flags.ptr, 4)
    bufs = (C.c_void_p * 1)(gathered.ptr)
    flg = (C.c_void_p * 1)(flags.ptr)
    assert lib.tq_comm_gather_setup(bufs, flg, 1, 0) == 0
    halves = []
    for step in range(3):
        off = C.c_size_t(0)
        if step == 2:      # the fused-quantiser form of the same call (per-block scales)
            assert lib.qwn_x_gemm_w4a8_fanout_gathered_fused(pkg.weight_array(ws), 2, dx.ptr, T, 0,
                                                             C.byref(off)) == 0
        else:
            assert lib.qwn_x_gemm_w4a8_fanout_gathered(pkg.weight_array(ws), 2, aq.ptr, as_.ptr,
                                                       asum.ptr, T, C.byref(off)) == 0
        assert lib.tq_comm_gather_wait() == 0
        lib.tq_sync()
        halves.append(off.value)
        got = gathered.to_numpy(np.float32)[off.value: off.value + block]
        assert got.tobytes() == want.tobytes()
        assert flags.to_numpy(np.int32)[0] == step + 1
    assert sorted(set(halves)) == [0, block]
    assert lib.tq_last_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,ksh", [(1088, 5120, 0), (320, 1024, 1), (64, 256, 0)])
def test_gemv_fused_quant_prologue(lib, pkg, orc, wl, M, K, ksh):
    """x_gemv_w4a8_fused quantises the row inside the GEMV launch: same bits as the oracle and
    as the two-launch x_gemv_w4a8, and the prepared scratch it leaves behind serves a following
    *_prepared call like the reference's x_prepare_gemv_act_s8 would."""
    codes, scales = wl.random_packed_weight(M, K, seed=3 * M + K, ksh=ksh)
    w = pkg.PackedWeight(codes, scales, M, K, k64=bool(ksh))
    x = refgen.shard_check_row(K)
    y = pkg.DevBuf(M * 4)
    y.fill(0xA5)
    dx = dev(pkg, x)
    y0 = pkg.DevBuf(M * 4)
    assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y0.ptr) == 0          # two launches
    lib.qwn_x_prepare_gemv_act_s8(dev(pkg, np.zeros(K, np.float32)).ptr, K)   # scratch overwritten
    assert lib.qwn_x_gemv_w4a8_fused(w.ref, dx.ptr, None, y.ptr) == 0
    lib.tq_sync()
    q, s, sm = orc.quantize_act_s8(x)
    _, want = orc.gemv_w4a8(codes, scales, M, K, ksh, q, s, sm, fma=1)
    assert y.to_numpy(np.float32).tobytes() == want.tobytes()
    assert y0.to_numpy(np.float32).tobytes() == want.tobytes()
    dq, ds, dsum = pkg.DevBuf(K), pkg.DevBuf(K // 32 * 4), pkg.DevBuf(K // 16 * 4)
    assert lib.qwn_dbg_prepared_act(K, dq.ptr, ds.ptr, dsum.ptr) == 0
    lib.tq_sync()
    assert np.array_equal(dq.to_numpy(np.int8), q)
    assert ds.to_numpy(np.float32).tobytes() == s.tobytes()
    assert np.array_equal(dsum.to_numpy(np.int32), sm)
    y2 = pkg.DevBuf(M * 4)
    assert lib.qwn_x_gemv_w4a8_prepared(w.ref, y2.ptr, None) == 0
    lib.tq_sync()
    assert y2.to_numpy(np.float32).tobytes() == want.tobytes()
    assert lib.tq_last_error() == 0


def _bf16_rne(a):
    """fp32 -> bfloat16 bits, round to nearest even (what __float2bfloat16_rn does)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,ksh,T,bf16", [(2048, 512, 1, 128, False), (1024, 1024, 0, 256, False),
                                            (2048, 256, 1, 136, False), (1024, 512, 1, 128, True),
                                            # one tile of two steps; more tiles than SMs with ragged tokens
                                            (128, 128, 1, 128, False), (2560, 640, 0, 1000, False)])
def test_gemm_pertoken_tcgen05(lib, pkg, orc, wl, M, K, ksh, T, bf16):
    """Per-token activation scales: the int32 dot runs over a whole weight-scale group in
    TMEM (two k-tiles under K64) before one fp32 promote; y = acc * as_tok. Bit-identical to
    the oracle's restatement of that formula."""
    codes, scales = wl.random_packed_weight(M, K, seed=M + K + T, ksh=ksh)
    w = pkg.PackedWeight(codes, scales, M, K, k64=bool(ksh))
    x = wl.activations_normal(T, K, seed=9, outlier_frac=0.01)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    dx = dev(pkg, x)
    lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    y = pkg.DevBuf(T * M * (2 if bf16 else 4))
    y.fill(0xA5)
    assert lib.qwn_x_gemm_w4a8_pertoken(w.ref, aq.ptr, at.ptr, asum.ptr, y.ptr, T, int(bf16)) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
    as_tok = os_.reshape(K // 32, T)[0].copy()
    rc, want = orc.gemm_w4a8_pertoken(codes, scales, M, K, ksh, oq, as_tok, osm, T)
    assert rc == 0
    if bf16:
        assert np.array_equal(y.to_numpy(np.uint16), _bf16_rne(want).reshape(-1))
    else:
        assert y.to_numpy(np.float32).tobytes() == np.ascontiguousarray(want).tobytes()
    assert lib.tq_last_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("K,T", [(256, 8), (5120, 40), (128, 136), (5120, 72), (17408, 64), (192, 70)])
def test_quantize_act_chunk_s4(lib, pkg, orc, wl, K, T):
    """W4A4 staging: packed int4 codes, scales and sums bit-identical to the oracle."""
    x = wl.activations_normal(T, K, seed=K + T, outlier_frac=0.01)
    x[0, :64] = 0.0
    n = K // 64 * T
    aq4, as4, asum4 = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    for b in (aq4, as4, asum4):
        b.fill(0xA5)
    dx = dev(pkg, x)
    lib.qwn_x_quantize_act_chunk_s4(dx.ptr, K, T, aq4.ptr, as4.ptr, asum4.ptr)
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk_s4(x)
    assert np.array_equal(aq4.to_numpy(np.uint8), oq)
    assert as4.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum4.to_numpy(np.int32), osm)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,T", [(2048, 512, 128), (1024, 1024, 256), (2048, 256, 136)])
def test_gemm_w4a4_tcgen05(lib, pkg, orc, wl, M, K, T):
    """W4A4 GEMM: both k-tiles of a K64 group accumulate in TMEM, one fp32 promote per group
    with the (token, K64) activation scale; bit-identical to the oracle (contracted
    multiply-add), within 1e-3 of the uncontracted form. Error codes as the reference."""
    codes, scales = wl.random_packed_weight(M, K, seed=M + K + T, ksh=1)
    w = pkg.PackedWeight(codes, scales, M, K, k64=True)
    x = wl.activations_normal(T, K, seed=11, outlier_frac=0.01)
    n = K // 64 * T
    aq4, as4, asum4 = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    dx = dev(pkg, x)
    lib.qwn_x_quantize_act_chunk_s4(dx.ptr, K, T, aq4.ptr, as4.ptr, asum4.ptr)
    y = pkg.DevBuf(T * M * 4)
    y.fill(0xA5)
    assert lib.qwn_x_gemm_w4a4(w.ref, aq4.ptr, as4.ptr, asum4.ptr, y.ptr, T) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk_s4(x)
    rc, want = orc.gemm_w4a4(codes, scales, M, K, oq, os_, osm, T, fma=1)
    rc0, want0 = orc.gemm_w4a4(codes, scales, M, K, oq, os_, osm, T, fma=0)
    assert rc == 0 and rc0 == 0
    got = y.to_numpy(np.float32).reshape(T, M)
    assert got.tobytes() == np.ascontiguousarray(want).tobytes()
    assert close_1e3(got, want0)
    assert lib.tq_last_error() == 0
    # argument errors and the shapes this build does not cover
    assert lib.qwn_x_gemm_w4a4(w.ref, aq4.ptr, as4.ptr, asum4.ptr, y.ptr, 12) == -2
    assert lib.qwn_x_gemm_w4a4(w.ref, aq4.ptr, as4.ptr, asum4.ptr, y.ptr, 8) == -3
    c32, s32 = wl.random_packed_weight(M, K, seed=1, ksh=0)
    w32 = pkg.PackedWeight(c32, s32, M, K, k64=False)
    assert lib.qwn_x_gemm_w4a4(w32.ref, aq4.ptr, as4.ptr, asum4.ptr, y.ptr, T) == -1


@pytest.mark.gpu
def test_overlapped_readback(lib, pkg):
    """tq_d2h_overlapped: the copy runs behind what was queued before it, tickets come in
    turn, tq_stream_wait_copy orders a later overwrite after the copy, tq_sync covers both
    streams."""
    n = 1 << 20
    a = np.arange(n, dtype=np.int32)
    d = dev(pkg, a)
    host = [lib.tq_host_alloc_pinned(n * 4) for _ in range(2)]
    try:
        t0 = lib.tq_d2h_overlapped(host[0], d.ptr, n * 4)
        assert 0 <= t0 < 16
        lib.tq_stream_wait_copy(t0)          # the fill below must not overtake the copy
        d.fill(0x11)
        t1 = lib.tq_d2h_overlapped(host[1], d.ptr, n * 4)
        assert t1 == (t0 + 1) % 16
        lib.tq_sync()
        got0 = np.ctypeslib.as_array(C.cast(host[0], C.POINTER(C.c_int32)), shape=(n,))
        got1 = np.ctypeslib.as_array(C.cast(host[1], C.POINTER(C.c_int32)), shape=(n,))
        assert np.array_equal(got0, a)
        assert np.all(got1 == 0x11111111)
        lib.tq_stream_wait_copy(-1)          # out of range: ignored
        assert lib.tq_last_error() == 0
    finally:
        for h in host:
            lib.tq_host_free_pinned(h)


@pytest.mark.gpu
def test_overlapped_upload(lib, pkg):
    """tq_h2d_overlapped: the upload starts behind what was queued before it (so it may
    replace a buffer that an earlier call reads), a later call that reads the buffer is
    ordered behind it by tq_stream_wait_copy, and it shares the tickets of the read-back."""
    n = 1 << 20
    a = np.arange(n, dtype=np.int32)
    b = a[::-1].copy()
    d = dev(pkg, a)
    e = pkg.DevBuf(n * 4)
    hb = lib.tq_host_alloc_pinned(n * 4)
    ho = lib.tq_host_alloc_pinned(n * 4)
    try:
        C.memmove(hb, b.ctypes.data, n * 4)
        lib.tq_d2d_async(e.ptr, d.ptr, n * 4)          # reads d before the upload replaces it
        t0 = lib.tq_h2d_overlapped(d.ptr, hb, n * 4)
        assert 0 <= t0 < 16
        lib.tq_stream_wait_copy(t0)
        t1 = lib.tq_d2h_overlapped(ho, d.ptr, n * 4)   # queued behind the wait: sees b
        assert t1 == (t0 + 1) % 16
        lib.tq_sync()
        got = np.ctypeslib.as_array(C.cast(ho, C.POINTER(C.c_int32)), shape=(n,))
        assert np.array_equal(got, b)
        assert np.array_equal(e.to_numpy(np.int32), a)
        assert lib.tq_last_error() == 0
    finally:
        lib.tq_host_free_pinned(hb)
        lib.tq_host_free_pinned(ho)


# ---------------------------------------------------------------- W8A8 tier
def _w8_weight(pkg, orc, M, K, seed):
    """A W8A8 record repacked on the device from a random E2M3 payload, plus the oracle's
    codes and scales of the same payload."""
    rng = np.random.default_rng(seed)
    codes6 = rng.integers(0, 64, size=(M, K), dtype=np.uint8)
    Kt = K // 32
    sc = Kt // 4
    bs = (rng.random(((M + 127) // 128, sc)) * 0.01 + 0.002).astype(np.float32)
    payload = orc.e2m3_payload_from_codes_fast(codes6)
    lib = pkg.load()
    w = pkg.TqWeight()
    w.M, w.K, w.Mt, w.Kt = M, K, M // 16, Kt
    w.block_scaled, w.e2m3, w.scale_rows, w.scale_cols = 1, 1, (M + 127) // 128, sc
    w.d_A = lib.tq_dev_alloc(payload.nbytes, b"t.payload")
    w.d_block_scale_inv = lib.tq_dev_alloc(bs.nbytes, b"t.bs")
    lib.tq_h2d(w.d_A, payload.ctypes.data, payload.nbytes)
    lib.tq_h2d(w.d_block_scale_inv, bs.ctypes.data, bs.nbytes)
    assert lib.qwn_x_w8_repack_weight(C.byref(w)) == 0
    assert w.s8_ready == 1 and not w.d_A and not w.d_block_scale_inv
    rc, oc, osc = orc.w8_repack(payload, bs, sc, M, K)
    assert rc == 0
    return w, oc, osc


def _w8_free(lib, w):
    lib.tq_dev_free(w.d_s8)
    lib.tq_dev_free(w.d_s8_scale)


@pytest.mark.gpu
def test_w8_repack_bit_exact(lib, pkg, orc):
    M, K = 128, 512
    w, oc, osc = _w8_weight(pkg, orc, M, K, seed=31)
    gc, gs = np.empty_like(oc), np.empty_like(osc)
    lib.tq_d2h(gc.ctypes.data, w.d_s8, gc.nbytes)
    lib.tq_d2h(gs.ctypes.data, w.d_s8_scale, gs.nbytes)
    assert np.array_equal(gs, osc)
    assert np.array_equal(gc, oc)
    _w8_free(lib, w)
    bad = pkg.TqWeight()
    assert lib.qwn_x_w8_repack_weight(C.byref(bad)) == -1


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,res", [(64, 256, False), (48, 384, True), (272, 5120, True),
                                     (65536 + 16, 128, False)])
def test_gemv_w8a8(lib, pkg, orc, M, K, res):
    """W8A8 GEMV through the tier dispatcher: bit-identical to the oracle (contracted form),
    within 1e-3 of the uncontracted one; split counts 16, 8 and 1."""
    w, oc, osc = _w8_weight(pkg, orc, M, K, seed=M + K)
    x = refgen.lcg_floats(K, seed=3 + M)[0]
    dx = dev(pkg, x)
    r = refgen.lcg_floats(M, seed=9)[0] if res else None
    dr = dev(pkg, r) if res else None
    y = pkg.DevBuf(M * 4)
    y.fill(0xA5)
    if res:
        assert lib.qwn_x_gemv_qmma_add(C.byref(w), dx.ptr, dr.ptr, y.ptr) == 0
    else:
        assert lib.qwn_x_gemv_qmma(C.byref(w), dx.ptr, y.ptr) == 0
    lib.tq_sync()
    q, s, _ = orc.quantize_act_s8(x)
    want = orc.gemv_w8a8(oc, osc, M, K, q, s, residual=r, fma=1)
    want0 = orc.gemv_w8a8(oc, osc, M, K, q, s, residual=r, fma=0)
    got = y.to_numpy(np.float32)
    assert got.tobytes() == want.tobytes()
    assert close_1e3(got, want0)
    assert lib.qwn_x_gemv_w8a8_prepared(C.byref(w), None, None) == -1
    assert lib.tq_last_error() == 0
    _w8_free(lib, w)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,T", [(64, 256, 8), (272, 512, 24), (1024, 1024, 128)])
def test_gemm_w8a8(lib, pkg, orc, M, K, T):
    w, oc, osc = _w8_weight(pkg, orc, M, K, seed=M + K + T)
    x = refgen.gemm_check_rows(T, K)
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    y = pkg.DevBuf(T * M * 4)
    y.fill(0xA5)
    assert lib.qwn_x_gemm_w8a8(C.byref(w), aq.ptr, as_.ptr, y.ptr, T) == 0
    lib.tq_sync()
    oq, os_, _ = orc.quantize_act_chunk(x)
    rc, want = orc.gemm_w8a8(oc, osc, M, K, oq, os_, T, fma=1)
    rc0, want0 = orc.gemm_w8a8(oc, osc, M, K, oq, os_, T, fma=0)
    assert rc == 0 and rc0 == 0
    got = y.to_numpy(np.float32).reshape(T, M)
    assert got.tobytes() == np.ascontiguousarray(want).tobytes()
    assert close_1e3(got, want0)
    assert lib.qwn_x_gemm_w8a8(C.byref(w), aq.ptr, as_.ptr, y.ptr, 12) == -2
    assert lib.tq_last_error() == 0
    _w8_free(lib, w)


@pytest.mark.gpu
@pytest.mark.parametrize("ksh,tp", [(0, 2), (1, 4), (0, 8)])
def test_row_parallel_and_replicate_shards(lib, pkg, orc, wl, ksh, tp):
    """x_w4_shard modes 1 and 2 (kernels_dpas.cpp:501-546). Mode 1: a rank's shard is the
    weight restricted to its K range, so its GEMV equals the oracle's GEMV of that slice bit
    for bit, and the ranks' partial outputs add up to the full projection within 1e-3
    (tq_comm_allreduce_sum is that sum; with one rank it is a copy). Mode 2: a full copy."""
    M, K = 256, 2048
    codes, scales = wl.random_packed_weight(M, K, seed=5 + ksh, ksh=ksh)
    w = pkg.PackedWeight(codes, scales, M, K, k64=bool(ksh))
    x = refgen.shard_check_row(K)
    q, sc, sm = orc.quantize_act_s8(x)
    _, full = orc.gemv_w4a8(codes, scales, M, K, ksh, q, sc, sm, fma=1)
    Kt, Kn = K // 32, K // tp
    cs = codes.reshape(M // 16, Kt, 256)
    ss = scales.reshape(M // 16, Kt >> ksh, 16)
    total = np.zeros(M, np.float64)
    for r in range(tp):
        s = pkg.TqWeight()
        assert lib.qwn_x_w4_shard(C.byref(s), w.ref, r, tp, 1, None, 0) == 0
        assert s.K == Kn and s.Kt == Kt // tp and s.M == M
        want_c = np.ascontiguousarray(cs[:, r * (Kt // tp):(r + 1) * (Kt // tp)]).reshape(-1)
        g = (Kt // tp) >> ksh
        want_s = np.ascontiguousarray(ss[:, r * g:(r + 1) * g]).reshape(-1)
        gc, gs = np.empty_like(want_c), np.empty_like(want_s)
        lib.tq_d2h(gc.ctypes.data, s.d_s4, gc.nbytes)
        lib.tq_d2h(gs.ctypes.data, s.d_s4_scale, gs.nbytes)
        assert np.array_equal(gc, want_c) and np.array_equal(gs, want_s)
        xs = np.ascontiguousarray(x[r * Kn:(r + 1) * Kn])
        dxs = dev(pkg, xs)
        y = pkg.DevBuf(M * 4)
        assert lib.qwn_x_gemv_w4a8(C.byref(s), dxs.ptr, y.ptr) == 0
        y2 = pkg.DevBuf(M * 4)
        assert lib.tq_comm_allreduce_sum(y.ptr, y2.ptr, M) == 0      # world of one: a copy
        lib.tq_sync()
        qs, scs, sms = orc.quantize_act_s8(xs)
        _, part = orc.gemv_w4a8(want_c, want_s, M, Kn, ksh, qs, scs, sms, fma=1)
        assert y.to_numpy(np.float32).tobytes() == part.tobytes()
        assert y2.to_numpy(np.float32).tobytes() == part.tobytes()
        total += part
        lib.qwn_x_w4_shard_free(C.byref(s))
    assert close_1e3(total.astype(np.float32), full)
    rep = pkg.TqWeight()
    assert lib.qwn_x_w4_shard(C.byref(rep), w.ref, 1, tp, 2, None, 0) == 0
    gc, gs = np.empty_like(codes), np.empty_like(scales)
    lib.tq_d2h(gc.ctypes.data, rep.d_s4, gc.nbytes)
    lib.tq_d2h(gs.ctypes.data, rep.d_s4_scale, gs.nbytes)
    assert np.array_equal(gc, codes) and np.array_equal(gs, scales) and rep.M == M and rep.K == K
    lib.qwn_x_w4_shard_free(C.byref(rep))
    bad = pkg.TqWeight()
    assert lib.qwn_x_w4_shard(C.byref(bad), w.ref, 0, 3, 1, None, 0) == -7
    if ksh:
        assert lib.qwn_x_w4_shard(C.byref(bad), w.ref, 0, 64, 1, None, 0) == -8


@pytest.mark.gpu
@pytest.mark.parametrize("H,T", [(5120, 8), (352, 3), (256, 40)])
def test_rmsnorm_chunk(lib, pkg, orc, H, T):
    rng = np.random.default_rng(H + T)
    x = (rng.standard_normal((T, H)) * 3).astype(np.float32)
    w = ((rng.standard_normal(H) * 0.1).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    dx, dw, out = dev(pkg, x), dev(pkg, w), pkg.DevBuf(T * H * 4)
    out.fill(0xA5)
    lib.qwn_x_rmsnorm_chunk(out.ptr, dx.ptr, dw.ptr, H, T, 1e-6)
    lib.tq_sync()
    want = orc.rmsnorm_chunk(x, w, 1e-6)
    assert out.to_numpy(np.float32).tobytes() == want.tobytes()
    wf = (w.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    x64 = x.astype(np.float64)
    ref = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-6) * (1.0 + wf)
    assert np.abs(want - ref).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.gpu
@pytest.mark.parametrize("Ms,K,ksh,T,per_token", [
    ([1088, 1088], 5120, 1, 8, True), ([1088, 544], 512, 1, 8, False), ([320], 2112, 0, 8, True),
    ([4800], 2112, 1, 8, False), ([64, 64], 512, 0, 16, True), ([48], 384, 0, 24, False)])
def test_gemm_fanout_fused_quantiser(lib, pkg, orc, wl, Ms, K, ksh, T, per_token):
    """x_gemm_w4a8_fanout_fused: the quantiser in the GEMM's prologue (T = 8) or staged by the
    library (other T) gives the bits of staging first and calling x_gemm_w4a8_fanout, which in
    turn are the oracle's."""
    ws, host = [], []
    for i, M in enumerate(Ms):
        c, s = wl.random_packed_weight(M, K, seed=300 + i + T, ksh=ksh)
        host.append((c, s, M))
        ws.append(pkg.PackedWeight(c, s, M, K, k64=bool(ksh)))
    x = wl.activations_normal(T, K, seed=K + T, outlier_frac=0.01)
    x[1, :32] = 0.0
    dx = dev(pkg, x)
    ys = [pkg.DevBuf(T * M * 4) for M in Ms]
    for y in ys:
        y.fill(0xA5)
    assert lib.qwn_x_gemm_w4a8_fanout_fused(pkg.weight_array(ws), pkg.ptr_array(ys), len(Ms), dx.ptr, T,
                                            int(per_token)) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x, per_token=per_token)
    for (c, s, M), y in zip(host, ys):
        _, want = orc.gemm_w4a8(c, s, M, K, ksh, oq, os_, osm, T, fma=1)
        assert y.to_numpy(np.float32).tobytes() == np.ascontiguousarray(want).tobytes()
    assert lib.qwn_x_gemm_w4a8_fanout_fused(pkg.weight_array(ws), pkg.ptr_array(ys), len(Ms), None, T, 0) == -2
    assert lib.tq_last_error() == 0


# ---------------------------------------------------------------- per-token decode batches
PERTOKEN_DECODE = [
    # Ms, K, ksh, T
    ([1088, 1088], 5120, 1, 8), ([320], 1024, 0, 8), ([48], 384, 0, 8), ([16, 272], 128, 1, 8),
    ([5120], 2112, 0, 16), ([4800], 2112, 1, 16), ([1600], 1056, 0, 40), ([2048], 512, 0, 64),
    ([640, 128], 2048, 1, 32), ([144], 4096, 1, 24), ([34816], 256, 0, 8), ([4096], 64, 1, 64),
]


@pytest.mark.gpu
@pytest.mark.parametrize("Ms,K,ksh,T", PERTOKEN_DECODE)
def test_gemm_pertoken_decode(lib, pkg, orc, wl, Ms, K, ksh, T):
    """x_gemm_w4a8_fanout_pertoken (tcgen05 decode kernel, per-token activation scales): one
    promote per weight-scale group, splits over groups summed in order, bit-identical to the
    oracle; arbitrary zero points, zero scales, partial 128-row blocks, odd group counts."""
    host = [wl.random_packed_weight(M, K, seed=900 + i + M + T, ksh=ksh) for i, M in enumerate(Ms)]
    ws = [pkg.PackedWeight(c, s, M, K, k64=bool(ksh)) for (c, s), M in zip(host, Ms)]
    x = wl.activations_normal(T, K, seed=T + K, outlier_frac=0.01)
    dx = dev(pkg, x)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    ys = [pkg.DevBuf(T * M * 4) for M in Ms]
    for b in ys:
        b.fill(0xA5)
    assert lib.qwn_x_gemm_w4a8_fanout_pertoken(pkg.weight_array(ws), pkg.ptr_array(ys), len(Ms), aq.ptr,
                                               at.ptr, asum.ptr, T) == 0
    lib.tq_sync()
    oq, os_, osm = orc.quantize_act_chunk(x, per_token=True)
    as_tok = os_.reshape(K // 32, T)[0].copy()
    for (c, s), M, yb in zip(host, Ms, ys):
        S = lib.qwn_choose_pertoken_splits(M // 16, T // 8, K // 32, ksh)
        assert S == orc.choose_pertoken_splits(M // 16, T // 8, K // 32, ksh)
        _, want = orc.gemm_w4a8_pertoken(c, s, M, K, ksh, oq, as_tok, osm, T, splits=S)
        got = yb.to_numpy(np.float32).reshape(T, M)
        assert got.tobytes() == want.tobytes(), (M, S)
    # the single-weight entry point routes decode batches to the same kernel
    y1 = pkg.DevBuf(T * Ms[0] * 4)
    assert lib.qwn_x_gemm_w4a8_pertoken(ws[0].ref, aq.ptr, at.ptr, asum.ptr, y1.ptr, T, 0) == 0
    lib.tq_sync()
    assert y1.to_numpy(np.float32).tobytes() == ys[0].to_numpy(np.float32).tobytes()
    assert lib.qwn_x_gemm_w4a8_pertoken(ws[0].ref, aq.ptr, at.ptr, asum.ptr, y1.ptr, T, 1) == -3
    assert lib.tq_last_error() == 0


@pytest.mark.gpu
def test_gemm_cases_on_the_tcgen05_decode_kernel():
    """The decode-batch cases of test_gemm_int32_dots_and_fp32 once more with the tcgen05 decode
    kernel forced for every batch of 8..64 tokens (TQ_XPU_DTC_MIN_TOKENS=8, read once per
    process, hence the child process): byte-identical to the oracle there too."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, TQ_XPU_DTC_MIN_TOKENS="8")
    out = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-q", "-m", "gpu", "-x",
                          "-k", "test_gemm_int32_dots_and_fp32 or test_gemm_fanout_equals_per_weight"],
                         env=env, capture_output=True, text=True, timeout=1200)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]


# ---- decode-batch fusions: the two calls' bits in one launch ---------------------------------
# (5120, 8): clusters of 8 CTAs per token; (1280, 16): clusters of 8 over short slices;
# (96, 8): no K32-aligned split into 2, 4 or 8 - the two separate launches
@pytest.mark.gpu
@pytest.mark.parametrize("H,T", [(5120, 8), (1280, 16), (17408, 8), (96, 8), (5120, 40), (5120, 64), (5120, 72)])
def test_rmsnorm_quant_chunk_pertoken(lib, pkg, orc, H, T):
    rng = np.random.default_rng(H + T)
    x = (rng.standard_normal((T, H)) * 3).astype(np.float32)
    x[0, :] = 0.0                                           # a zero row: scale 1, codes 0
    w = ((rng.standard_normal(H) * 0.1).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    dx, dw, out = dev(pkg, x), dev(pkg, w), pkg.DevBuf(T * H * 4)
    n = H // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    for b in (out, aq, as_, asum, at):
        b.fill(0xA5)
    lib.qwn_x_rmsnorm_quant_chunk_pertoken(out.ptr, dx.ptr, dw.ptr, H, T, 1e-6, aq.ptr, as_.ptr, asum.ptr,
                                           at.ptr, 0)
    lib.tq_sync()
    xn = orc.rmsnorm_chunk(x, w, 1e-6)
    oq, os_, osm = orc.quantize_act_chunk(xn, per_token=True)
    assert out.to_numpy(np.float32).tobytes() == xn.tobytes()
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)
    assert at.to_numpy(np.float32).tobytes() == os_.reshape(H // 32, T)[0].tobytes()
    assert lib.tq_last_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("K,T", [(17408, 8), (8704, 8), (160, 8), (5120, 40), (17408, 64), (17408, 66)])
def test_silu_mul_quant_chunk_pertoken(lib, pkg, orc, K, T):
    rng = np.random.default_rng(K + T)
    g = (rng.standard_normal((T, K)) * 2).astype(np.float32)
    u = rng.standard_normal((T, K)).astype(np.float32)
    dg, du, out = dev(pkg, g), dev(pkg, u), pkg.DevBuf(T * K * 4)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    for b in (out, aq, as_, asum, at):
        b.fill(0xA5)
    lib.qwn_x_silu_mul_quant_chunk_pertoken(out.ptr, dg.ptr, du.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    lib.tq_sync()
    h = orc.silu_mul(g, u).reshape(T, K)
    oq, os_, osm = orc.quantize_act_chunk(h, per_token=True)
    assert out.to_numpy(np.float32).tobytes() == h.tobytes()
    assert np.array_equal(aq.to_numpy(np.int8), oq)
    assert as_.to_numpy(np.float32).tobytes() == os_.tobytes()
    assert np.array_equal(asum.to_numpy(np.int32), osm)
    assert at.to_numpy(np.float32).tobytes() == os_.reshape(K // 32, T)[0].tobytes()
    assert lib.tq_last_error() == 0
