"""Committed golden vectors (tests/golden/w4a8_golden.npz, made by tests/golden/make_golden.py
from the reference's closed-form check inputs): the CPU oracle must reproduce them bit for
bit, and so must the CUDA library through its C ABI (marked gpu)."""
import ctypes as C
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "w4a8_golden.npz")


@pytest.fixture(scope="module")
def g():
    return dict(np.load(GOLDEN))


def same(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.dtype == b.dtype and a.shape == b.shape and a.tobytes() == b.tobytes()


def test_generator_is_deterministic(g):
    """Re-running the committed generator gives the committed bytes."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(GOLDEN), "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.cases()
    assert sorted(fresh) == sorted(g)
    for k in g:
        assert same(fresh[k], g[k]), k


def test_oracle_quantisers_match_golden(g, orc):
    q, s, sm = orc.quantize_act_s8(g["q1_x"])
    assert same(q, g["q1_q"]) and same(s, g["q1_scale"]) and same(sm, g["q1_sum16"])
    aq, as_, asum = orc.quantize_act_chunk(g["qc_x"])
    assert same(aq, g["qc_aq"]) and same(as_, g["qc_as"]) and same(asum, g["qc_asum"])
    hid, hq, hs, hsm = orc.silu_mul_quant(g["silu_gate"], g["silu_up"])
    assert same(hid, g["silu_hidden"]) and same(hq, g["silu_q"]) and same(hs, g["silu_scale"])
    # hand-checkable facts of the first block: scale = absmax/127, codes within [-127, 127]
    x = g["q1_x"][:32]
    assert g["q1_scale"][0] == np.float32(np.abs(x).max()) / np.float32(127.0)
    assert np.abs(g["q1_q"]).max() <= 127
    assert g["q1_sum16"][0] == int(g["q1_q"][:16].astype(np.int32).sum())


def test_oracle_repack_gemv_gemm_match_golden(g, orc):
    K = g["qc_x"].shape[1]
    for mode in (0, 1, 2):
        rc, c, sc = orc.w4_repack(g["rp_payload"], g["rp_bs"], K // 128, 32, K, mode)
        assert rc == 0 and same(c, g[f"rp_codes_m{mode}"]) and same(sc, g[f"rp_scales_m{mode}"])
    for ksh in (0, 1):
        q, s, sm = orc.quantize_act_s8(g[f"gv{ksh}_x"])
        _, y = orc.gemv_w4a8(g[f"gv{ksh}_codes"], g[f"gv{ksh}_scales"], 48, 512, ksh, q, s, sm,
                             residual=g[f"gv{ksh}_res"], fma=1)
        assert same(y, g[f"gv{ksh}_y"])
        assert same(orc.tile_dots_gemv(g[f"gv{ksh}_codes"], 48, 512, q), g[f"gv{ksh}_dots"])
    aq, as_, asum = orc.quantize_act_chunk(g["gm_x"])
    _, y = orc.gemm_w4a8(g["gm_codes"], g["gm_scales"], 64, 512, 1, aq, as_, asum, 32,
                         offsets=[int(v) for v in g["gm_offsets"]], fma=1)
    assert same(y, g["gm_y"])
    # per-token mode
    aq, as_, asum = orc.quantize_act_chunk(g["gm_x"][:16], per_token=True)
    assert same(aq, g["pt_aq"]) and same(asum, g["pt_asum"]) and same(as_.reshape(16, 16)[0].copy(), g["pt_as_tok"])
    S = orc.choose_pertoken_splits(64 // 16, 2, 512 // 32, 1)
    assert S == int(g["pt_splits"][0])
    _, y = orc.gemm_w4a8_pertoken(g["gm_codes"], g["gm_scales"], 64, 512, 1, aq, g["pt_as_tok"], asum, 16, splits=S)
    assert same(y, g["pt_y"])


# ------------------------------------------------------------------ CUDA library vs golden
@pytest.mark.gpu
def test_cuda_matches_golden(g, lib, pkg):
    def dev(a):
        return pkg.DevBuf.from_numpy(np.ascontiguousarray(a))

    # decode quantiser
    K = g["q1_x"].size
    dq, ds, dsum = pkg.DevBuf(K), pkg.DevBuf(K // 32 * 4), pkg.DevBuf(K // 16 * 4)
    dx = dev(g["q1_x"])       # inputs stay alive until the asynchronous calls have run
    lib.qwn_x_quantize_act_s8(dx.ptr, K, dq.ptr, ds.ptr, dsum.ptr)
    lib.tq_sync()
    assert same(dq.to_numpy(np.int8), g["q1_q"]) and same(ds.to_numpy(np.float32), g["q1_scale"])
    assert same(dsum.to_numpy(np.int32), g["q1_sum16"])
    # GEMV with residual, both tiers
    for ksh in (0, 1):
        w = pkg.PackedWeight(g[f"gv{ksh}_codes"], g[f"gv{ksh}_scales"], 48, 512, k64=bool(ksh))
        y = pkg.DevBuf(48 * 4)
        dxv, dres = dev(g[f"gv{ksh}_x"]), dev(g[f"gv{ksh}_res"])
        assert lib.qwn_x_gemv_w4a8_add(w.ref, dxv.ptr, dres.ptr, y.ptr) == 0
        lib.tq_sync()
        assert same(y.to_numpy(np.float32), g[f"gv{ksh}_y"])
    # segmented GEMM
    T, Kg, M = 32, 512, 64
    n = Kg // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    dgx = dev(g["gm_x"])
    lib.qwn_x_quantize_act_chunk(dgx.ptr, Kg, T, aq.ptr, as_.ptr, asum.ptr)
    w = pkg.PackedWeight(g["gm_codes"], g["gm_scales"], M, Kg, k64=True)
    y = pkg.DevBuf(T * M * 4)
    offs = (C.c_int * 3)(*[int(v) for v in g["gm_offsets"]])
    assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, y.ptr, T, offs, 2) == 0
    lib.tq_sync()
    assert same(y.to_numpy(np.float32).reshape(T, M), g["gm_y"].reshape(T, M))
    # per-token staging and GEMM (16 tokens: two token groups on one warp of the ring kernel)
    Tp = 16
    npt = Kg // 32 * Tp
    paq, pas, pasum, pat = pkg.DevBuf(npt * 32), pkg.DevBuf(npt * 4), pkg.DevBuf(npt * 4), pkg.DevBuf(Tp * 4)
    dpx = dev(g["gm_x"][:Tp])
    lib.qwn_x_quantize_act_chunk_pertoken(dpx.ptr, Kg, Tp, paq.ptr, pas.ptr, pasum.ptr, pat.ptr)
    ypt = pkg.DevBuf(Tp * M * 4)
    assert lib.qwn_x_gemm_w4a8_pertoken(w.ref, paq.ptr, pat.ptr, pasum.ptr, ypt.ptr, Tp, 0) == 0
    lib.tq_sync()
    assert same(paq.to_numpy(np.int8).reshape(g["pt_aq"].shape), g["pt_aq"])
    assert same(pat.to_numpy(np.float32), g["pt_as_tok"])
    assert lib.qwn_choose_pertoken_splits(M // 16, Tp // 8, Kg // 32, 1) == int(g["pt_splits"][0])
    assert same(ypt.to_numpy(np.float32).reshape(g["pt_y"].shape), g["pt_y"])
    # column shard
    sh = pkg.TqWeight()
    grp = (C.c_int * 2)(32, 32)
    assert lib.qwn_x_w4_shard(C.byref(sh), w.ref, 1, 2, 0, grp, 2) == 0
    gc = np.empty_like(g["sh_codes"])
    gs = np.empty_like(g["sh_scales"])
    lib.tq_d2h(gc.ctypes.data, sh.d_s4, gc.nbytes)
    lib.tq_d2h(gs.ctypes.data, sh.d_s4_scale, gs.nbytes)
    assert same(gc, g["sh_codes"]) and same(gs, g["sh_scales"])
    lib.qwn_x_w4_shard_free(C.byref(sh))
    assert lib.tq_last_error() == 0
