"""Generates tests/golden/w4a8_golden.npz: small input/output vectors of the W4A8 projection path.

The reference ships no golden vectors for this path and cannot be built or run without
Intel's SYCL toolchain and GPU, so these vectors are produced by the CPU oracle
(oracle/w4a8_oracle.c, a restatement of the reference's source text) from the reference's own
closed-form check inputs (tests/refgen.py). They pin the oracle and the CUDA kernels to one
committed set of bits: a change in either shows up as a diff against this file.

  python tests/golden/make_golden.py          # rewrites the .npz beside this script
"""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

OUT = os.path.join(HERE, "w4a8_golden.npz")


def cases():
    from oracle import oracle as orc
    import refgen
    wl = importlib.import_module("knivesysl-xe_b200.workloads")
    g = {}

    # decode quantiser on the reference's check row (kernels_dpas.cpp:2705-2710)
    K = 256
    x = refgen.w4_check_row(K)
    q, s, sm = orc.quantize_act_s8(x)
    g.update(q1_x=x, q1_q=q, q1_scale=s, q1_sum16=sm)

    # chunk quantiser, k-tile-major staging (kernels_dpas.cpp:1149-1207)
    T = 8
    xc = refgen.gemm_check_rows(T, K)
    aq, as_, asum = orc.quantize_act_chunk(xc)
    g.update(qc_x=xc, qc_aq=aq, qc_as=as_, qc_asum=asum)

    # fused SiLU*up staging (kernels_dpas.cpp:199-202)
    gate = refgen.shard_check_row(K)
    up = refgen.w4_check_row(K)
    hid, hq, hs, hsm = orc.silu_mul_quant(gate, up)
    g.update(silu_gate=gate, silu_up=up, silu_hidden=hid, silu_q=hq, silu_scale=hs, silu_sum16=hsm)

    # repack of an E2M3 payload, all three tiers (kernels_dpas.cpp:229-344)
    rng = np.random.Generator(np.random.Philox(key=391))
    M = 32
    codes6 = rng.integers(0, 64, size=(M, K), dtype=np.uint8)
    payload = orc.e2m3_payload_from_codes_fast(codes6)
    # block scales: one per (128 rows, 128 columns), like the model files the reference loads
    bs = (np.float32(0.002) * (1 + rng.integers(0, 7, size=((M + 127) // 128, K // 128)))).astype(np.float32)
    g.update(rp_payload=payload, rp_bs=bs)
    for mode in (0, 1, 2):
        rc, c, sc = orc.w4_repack(payload, bs, K // 128, M, K, mode)
        assert rc == 0
        g[f"rp_codes_m{mode}"] = c
        g[f"rp_scales_m{mode}"] = sc

    # GEMV: two-accumulator order with residual, K32 and K64 (kernels_dpas.cpp:586-675)
    for ksh in (0, 1):
        Mg, Kg = 48, 512
        wc, ws = wl.random_packed_weight(Mg, Kg, seed=7 + ksh, ksh=ksh)
        xv = refgen.shard_check_row(Kg)
        q, s, sm = orc.quantize_act_s8(xv)
        res = refgen.w4_check_row(Mg)
        dots, y = orc.gemv_w4a8(wc, ws, Mg, Kg, ksh, q, s, sm, residual=res, fma=1)
        g.update({f"gv{ksh}_codes": wc, f"gv{ksh}_scales": ws, f"gv{ksh}_x": xv, f"gv{ksh}_res": res,
                  f"gv{ksh}_dots": orc.tile_dots_gemv(wc, Mg, Kg, q), f"gv{ksh}_y": y})

    # batched GEMM with two segments of different split counts (kernels_dpas.cpp:1334-1490)
    Mg, Kg, Tg, offs = 64, 512, 32, [0, 8, 32]
    wc, ws = wl.random_packed_weight(Mg, Kg, seed=11, ksh=1)
    xg = refgen.gemm_check_rows(Tg, Kg)
    aq, as_, asum = orc.quantize_act_chunk(xg)
    _, y = orc.gemm_w4a8(wc, ws, Mg, Kg, 1, aq, as_, asum, Tg, offsets=offs, fma=1)
    g.update(gm_codes=wc, gm_scales=ws, gm_x=xg, gm_offsets=np.array(offs, dtype=np.int32), gm_y=y,
             gm_dots=orc.tile_dots_gemm(wc, Mg, Kg, aq, Tg))

    # per-token activation scales (own extension of the path: one scale per token, one promote
    # per weight-scale group, splits over whole groups): staging and a 16-token GEMM, K64
    aqp, asp, asump = orc.quantize_act_chunk(xg[:16], per_token=True)
    as_tok = asp.reshape(Kg // 32, 16)[0].copy()
    S = orc.choose_pertoken_splits(Mg // 16, 2, Kg // 32, 1)
    _, ypt = orc.gemm_w4a8_pertoken(wc, ws, Mg, Kg, 1, aqp, as_tok, asump, 16, splits=S)
    g.update(pt_aq=aqp, pt_as_tok=as_tok, pt_asum=asump, pt_splits=np.array([S], dtype=np.int32), pt_y=ypt)

    # column shard (kernels_dpas.cpp:463-499): rank 1 of 2 over groups [32, 32]
    rc, sc_c, sc_s = orc.w4_shard_column(wc, ws, Mg, Kg, 1, 1, 2, groups=[32, 32])
    assert rc == 0
    g.update(sh_codes=sc_c, sh_scales=sc_s)
    return g


def main():
    g = cases()
    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT}: {len(g)} arrays, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()
