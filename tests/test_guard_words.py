"""Out-of-bounds writes: every output of the hot path's kernels sits between two guard regions
filled with 0xFF bytes (a NaN as fp32) that must survive the call (compute-sanitizer is not available on the
GPUs this is tested on; the oracle comparisons elsewhere check what is inside the buffers)."""
import ctypes as C

import numpy as np
import pytest

GUARD = 4096


class Guarded:
    """nbytes of output at .ptr inside an allocation with GUARD bytes of 0xFF before and after."""

    def __init__(self, pkg, nbytes):
        self.pkg, self.nbytes = pkg, int(nbytes)
        pad = (-self.nbytes) % 256
        self.total = GUARD + self.nbytes + pad + GUARD
        self.buf = pkg.DevBuf(self.total)
        self.buf.fill(0xFF)
        self.ptr = self.buf.ptr + GUARD

    def check(self, what):
        raw = self.buf.to_numpy(np.uint8)
        assert np.all(raw[:GUARD] == 0xFF), f"{what}: bytes before the buffer were written"
        assert np.all(raw[GUARD + self.nbytes:] == 0xFF), f"{what}: bytes behind the buffer were written"
        body = raw[GUARD:GUARD + self.nbytes]
        return body


def staging(pkg, K, T):
    n = K // 32 * T
    return Guarded(pkg, n * 32), Guarded(pkg, n * 4), Guarded(pkg, n * 4), Guarded(pkg, T * 4)


@pytest.mark.gpu
@pytest.mark.parametrize("K,T", [(5120, 8), (1280, 16), (96, 8), (17408, 8), (2048, 40)])
def test_stagings_stay_inside_their_buffers(lib, pkg, K, T):
    rng = np.random.default_rng(K + T)
    x = rng.standard_normal((T, K)).astype(np.float32)
    u = rng.standard_normal((T, K)).astype(np.float32)
    wn = ((rng.standard_normal(K) * 0.1).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    dx, du, dw = pkg.DevBuf.from_numpy(x), pkg.DevBuf.from_numpy(u), pkg.DevBuf.from_numpy(wn)
    for name, call in (
        ("chunk", lambda a, s, m, t, o: lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, a.ptr, s.ptr, m.ptr)),
        ("pertoken", lambda a, s, m, t, o: lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, a.ptr, s.ptr, m.ptr, t.ptr)),
        ("rmsnorm+pertoken", lambda a, s, m, t, o: lib.qwn_x_rmsnorm_quant_chunk_pertoken(
            o.ptr, dx.ptr, dw.ptr, K, T, 1e-6, a.ptr, s.ptr, m.ptr, t.ptr, 0)),
        ("silu*up+pertoken", lambda a, s, m, t, o: lib.qwn_x_silu_mul_quant_chunk_pertoken(
            o.ptr, dx.ptr, du.ptr, K, T, a.ptr, s.ptr, m.ptr, t.ptr)),
    ):
        aq, as_, asum, at = staging(pkg, K, T)
        out = Guarded(pkg, T * K * 4)
        call(aq, as_, asum, at, out)
        lib.tq_sync()
        for g in (aq, as_, asum, at, out):
            g.check(name)
        assert not np.all(aq.check(name) == 0xFF), name          # the call did write its codes
    assert lib.tq_last_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("T", [8, 16, 32, 64])
@pytest.mark.parametrize("ksh", [0, 1])
def test_decode_gemms_stay_inside_their_buffers(lib, pkg, wl, T, ksh):
    Ms, K = [272, 144], 2048            # partial 128-row blocks, two weights in one launch
    host = [wl.random_packed_weight(M, K, seed=50 + i + T, ksh=ksh) for i, M in enumerate(Ms)]
    ws = [pkg.PackedWeight(c, s, M, K, k64=bool(ksh)) for (c, s), M in zip(host, Ms)]
    x = wl.activations_normal(T, K, seed=T, outlier_frac=0.01)
    dx = pkg.DevBuf.from_numpy(x)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    for mode in ("exact", "pertoken"):
        ys = [Guarded(pkg, T * M * 4) for M in Ms]
        ya = (C.c_void_p * 2)(*[g.ptr for g in ys])
        if mode == "exact":
            lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
            assert lib.qwn_x_gemm_w4a8_fanout(pkg.weight_array(ws), ya, 2, aq.ptr, as_.ptr, asum.ptr, T, None, 0) == 0
        else:
            lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
            assert lib.qwn_x_gemm_w4a8_fanout_pertoken(pkg.weight_array(ws), ya, 2, aq.ptr, at.ptr, asum.ptr, T) == 0
        lib.tq_sync()
        for g, M in zip(ys, Ms):
            body = g.check(f"{mode} T={T}")
            assert np.isfinite(body.view(np.float32)).all()       # every output word was written
    assert lib.tq_last_error() == 0


@pytest.mark.gpu
def test_gemv_and_prefill_stay_inside_their_buffers(lib, pkg, wl):
    M, K = 1088, 1024
    codes, scales = wl.make_weight_w4(M, K, seed=1, group=64)
    w = pkg.PackedWeight(codes, scales, M, K, k64=True)
    x = wl.activations_normal(136, K, seed=2)
    dx = pkg.DevBuf.from_numpy(x)
    y = Guarded(pkg, M * 4)
    assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y.ptr) == 0
    lib.tq_sync()
    assert np.isfinite(y.check("gemv").view(np.float32)).all()
    # prefill kernel: 136 tokens = one full and one partial 128-token block; rows a multiple of 128
    Mp, T = 256, 136
    cp, sp = wl.make_weight_w4(Mp, K, seed=3, group=64)
    wp = pkg.PackedWeight(cp, sp, Mp, K, k64=True)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    yp = Guarded(pkg, T * Mp * 4)
    assert lib.qwn_x_gemm_w4a8(wp.ref, aq.ptr, as_.ptr, asum.ptr, yp.ptr, T, None, 0) == 0
    lib.tq_sync()
    assert np.isfinite(yp.check("prefill fp32").view(np.float32)).all()
    lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    for bf16 in (0, 1):
        yq = Guarded(pkg, T * Mp * (2 if bf16 else 4))
        assert lib.qwn_x_gemm_w4a8_pertoken(wp.ref, aq.ptr, at.ptr, asum.ptr, yq.ptr, T, bf16) == 0
        lib.tq_sync()
        body = yq.check(f"prefill per-token bf16={bf16}")
        assert not np.all(body == 0xFF)
    assert lib.tq_last_error() == 0
