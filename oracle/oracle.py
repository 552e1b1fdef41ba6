"""numpy front-end to the CPU oracle (oracle/w4a8_oracle.c).

Test infrastructure only: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg. The shipped library never loads it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle_w4a8.so")


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "w4a8_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_e2m3f.restype = C.c_float
        _lib.orc_e2m3f.argtypes = [C.c_uint32]
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_expf.restype = C.c_float
        _lib.orc_expf.argtypes = [C.c_float]
        _lib.orc_fit_int4_asym.restype = C.c_uint16
        _lib.orc_e2m3_code_at.restype = C.c_uint32
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ------------------------------------------------------------------ scalars
def f32_to_f16(x: float) -> int:
    return int(lib().orc_f32_to_f16(C.c_float(x)))


def f16_to_f32(h: int) -> float:
    return float(lib().orc_f16_to_f32(C.c_uint16(h)))


def expf(x: float) -> float:
    return float(lib().orc_expf(C.c_float(x)))


def e2m3f(code: int) -> float:
    return float(lib().orc_e2m3f(C.c_uint32(code)))


def choose_gemv_splits(groups: int) -> int:
    return int(lib().orc_choose_gemv_splits(C.c_int(groups)))


def choose_gemm_splits(rgroups: int, tgroups: int, ktiles: int, forced: int = 0) -> int:
    return int(lib().orc_choose_gemm_splits(C.c_int(rgroups), C.c_int(tgroups),
                                            C.c_int(ktiles), C.c_int(forced)))


def choose_pertoken_splits(rgroups: int, tgroups: int, ktiles: int, ksh: int, forced: int = 0) -> int:
    """Split rule of the per-token decode GEMMs (own rule, not in the reference): the split
    count of an 8-token call, doubled while one split's staged activations (320 bytes per
    k-tile and 8 tokens) exceed 88 KB; splits cut whole weight-scale groups."""
    kgroups = ktiles >> ksh
    s = choose_gemm_splits(rgroups, 1, kgroups, forced=forced)
    if forced in (1, 2, 4, 8, 16):
        return s
    cap = 1
    while cap < 16 and cap * 2 <= kgroups:
        cap *= 2
    while s < cap and (((kgroups + s - 1) // s) << ksh) * tgroups * 320 > 88 * 1024:
        s *= 2
    return s


def fit_int4_asym(wf, reserve_nibble: bool = True):
    wf = _c(wf, np.float32)
    z = C.c_int(0)
    sh = lib().orc_fit_int4_asym(_p(wf), C.c_int(wf.size), C.c_int(int(reserve_nibble)),
                                 C.byref(z))
    return int(sh), int(z.value)


# --------------------------------------------------------- E2M3 payload
def e2m3_payload_from_codes(codes6: np.ndarray) -> np.ndarray:
    """codes6[M][K] (values 0..63) -> dense fragment payload [Mt*Kt*384] bytes."""
    codes6 = _c(codes6, np.uint8)
    M, K = codes6.shape
    Kt = K // 32
    payload = np.zeros((M // 16) * Kt * 384, dtype=np.uint8)
    L = lib()
    for r in range(M):
        for c in range(K):
            L.orc_e2m3_set_code(_p(payload), C.c_int(Kt), C.c_int(r), C.c_int(c),
                                C.c_uint32(int(codes6[r, c])))
    return payload


def e2m3_payload_from_codes_fast(codes6: np.ndarray) -> np.ndarray:
    """Vectorised form of e2m3_payload_from_codes (same closed-form map)."""
    codes6 = _c(codes6, np.uint8).astype(np.uint32)
    M, K = codes6.shape
    Kt = K // 32
    row = np.arange(M)[:, None]
    col = np.arange(K)[None, :]
    mt, kt = row >> 4, col >> 5
    lane = (((row & 15) >> 1) << 2) | ((col & 31) >> 3)
    idx = (((col >> 2) & 1) << 3) | ((row & 1) << 2) | (col & 3)
    bit = 6 * idx
    base = (mt * Kt + kt) * 384 + lane * 12
    nbits = (Mt_ := M // 16) * Kt * 384 * 8
    bitpos = (base * 8 + bit).astype(np.int64)
    bits = np.zeros(nbits, dtype=np.uint8)
    for b in range(6):
        bits[(bitpos + b).ravel()] = ((codes6 >> b) & 1).astype(np.uint8).ravel()
    return np.packbits(bits, bitorder="little")


def e2m3_decode(payload, bs, scale_cols, M, K):
    payload = _c(payload, np.uint8)
    bs = _c(bs, np.float32)
    W = np.empty((M, K), dtype=np.float32)
    lib().orc_e2m3_decode(_p(payload), _p(bs), C.c_int(scale_cols), C.c_int(M), C.c_int(K), _p(W))
    return W


def scale_groups(K: int, mode: int) -> int:
    Kt = K // 32
    return Kt * 2 if mode == 1 else (Kt // 2 if mode == 2 else Kt)


def w4_pack_from_f32(W, mode: int = 0):
    W = _c(W, np.float32)
    M, K = W.shape
    codes = np.zeros(M * K // 2, dtype=np.uint8)
    scales = np.zeros(M * scale_groups(K, mode), dtype=np.uint16)
    rc = lib().orc_w4_pack_from_f32(_p(W), C.c_int(M), C.c_int(K), C.c_int(mode), _p(codes), _p(scales))
    return rc, codes, scales


def w4_repack(payload, bs, scale_cols, M, K, mode: int = 0):
    payload = _c(payload, np.uint8)
    bs = _c(bs, np.float32)
    codes = np.zeros(M * K // 2, dtype=np.uint8)
    scales = np.zeros(M * max(scale_groups(K, mode), 1), dtype=np.uint16)
    rc = lib().orc_w4_repack(_p(payload), _p(bs), C.c_int(scale_cols), C.c_int(M), C.c_int(K),
                             C.c_int(mode), _p(codes), _p(scales))
    return rc, codes, scales


def gemv_e2m3(payload, bs, scale_cols, M, K, x):
    payload, bs, x = _c(payload, np.uint8), _c(bs, np.float32), _c(x, np.float32)
    y = np.empty(M, dtype=np.float32)
    lib().orc_gemv_e2m3(_p(payload), _p(bs), C.c_int(scale_cols), C.c_int(M), C.c_int(K), _p(x), _p(y))
    return y


# ---------------------------------------------------------- quantisers
def quantize_act_s8(x):
    x = _c(x, np.float32)
    K = x.size
    q = np.empty(K, dtype=np.int8)
    s = np.empty(K // 32, dtype=np.float32)
    sm = np.empty(K // 16, dtype=np.int32)
    lib().orc_quantize_act_s8(_p(x), C.c_int(K), _p(q), _p(s), _p(sm))
    return q, s, sm


def silu_mul(gate, up):
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(gate)
    lib().orc_silu_mul(_p(out), _p(gate), _p(up), C.c_int(gate.size))
    return out


def silu_mul_quant(gate, up):
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    K = gate.size
    hidden = np.empty(K, dtype=np.float32)
    q = np.empty(K, dtype=np.int8)
    s = np.empty(K // 32, dtype=np.float32)
    sm = np.empty(K // 16, dtype=np.int32)
    lib().orc_silu_mul_quant(_p(hidden), _p(gate), _p(up), C.c_int(K), _p(q), _p(s), _p(sm))
    return hidden, q, s, sm


def rmsnorm_quant(x, w_bf16, eps):
    x, w = _c(x, np.float32), _c(w_bf16, np.uint16)
    H = x.size
    out = np.empty(H, dtype=np.float32)
    q = np.empty(H, dtype=np.int8)
    s = np.empty(H // 32, dtype=np.float32)
    sm = np.empty(H // 16, dtype=np.int32)
    lib().orc_rmsnorm_quant(_p(out), _p(x), _p(w), C.c_int(H), C.c_float(eps), _p(q), _p(s), _p(sm))
    return out, q, s, sm


def rmsnorm_chunk(x, w_bf16, eps):
    x, w_bf16 = _c(x, np.float32), _c(w_bf16, np.uint16)
    T, H = x.shape
    out = np.empty((T, H), dtype=np.float32)
    lib().orc_rmsnorm_chunk(_p(out), _p(x), _p(w_bf16), C.c_int(H), C.c_int(T), C.c_float(eps))
    return out


def quantize_act_chunk(x, per_token: bool = False):
    x = _c(x, np.float32)
    T, K = x.shape
    Kt = K // 32
    aq = np.empty(Kt * T * 32, dtype=np.int8)
    as_ = np.empty(Kt * T, dtype=np.float32)
    asum = np.empty(Kt * T, dtype=np.int32)
    fn = lib().orc_quantize_act_chunk_pertoken if per_token else lib().orc_quantize_act_chunk
    fn(_p(x), C.c_int(K), C.c_int(T), _p(aq), _p(as_), _p(asum))
    return aq, as_, asum


# ------------------------------------------------------------- dots
def tile_dots_gemv(codes, M, K, q):
    codes, q = _c(codes, np.uint8), _c(q, np.int8)
    d = np.empty((M // 16) * (K // 32) * 16, dtype=np.int32)
    lib().orc_tile_dots_gemv(_p(codes), C.c_int(M), C.c_int(K), _p(q), _p(d))
    return d


def tile_dots_gemm(codes, M, K, aq, T):
    codes, aq = _c(codes, np.uint8), _c(aq, np.int8)
    d = np.empty((K // 32) * T * M, dtype=np.int32)
    lib().orc_tile_dots_gemm(_p(codes), C.c_int(M), C.c_int(K), _p(aq), C.c_int(T), _p(d))
    return d


# ------------------------------------------------------------- GEMV / GEMM
def gemv_w4a8(codes, scales, M, K, ksh, q, as_, sum16, residual=None, fma=1):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    q, as_, sum16 = _c(q, np.int8), _c(as_, np.float32), _c(sum16, np.int32)
    res = None if residual is None else _c(residual, np.float32)
    y = np.empty(M, dtype=np.float32)
    rc = lib().orc_gemv_w4a8(_p(codes), _p(scales), C.c_int(M), C.c_int(K), C.c_int(ksh), _p(q),
                             _p(as_), _p(sum16), _p(res), _p(y), C.c_int(fma))
    return rc, y


def gemv_w4a8_k16(codes, scales, M, K, q, as_, sum16, residual=None, fma=1):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    q, as_, sum16 = _c(q, np.int8), _c(as_, np.float32), _c(sum16, np.int32)
    res = _c(residual, np.float32) if residual is not None else None
    y = np.empty(M, dtype=np.float32)
    rc = lib().orc_gemv_w4a8_k16(_p(codes), _p(scales), C.c_int(M), C.c_int(K), _p(q), _p(as_),
                                 _p(sum16), _p(res) if res is not None else None, _p(y), C.c_int(fma))
    assert rc == 0, rc
    return y


def gemv_w4a8_fanout(weights, K, ksh, q, as_, sum16, fma=1):
    """weights: list of (codes, scales, M)."""
    n = len(weights)
    cs = [_c(w[0], np.uint8) for w in weights]
    ss = [_c(w[1], np.uint16) for w in weights]
    Ms = (C.c_int * n)(*[int(w[2]) for w in weights])
    ys = [np.empty(int(w[2]), dtype=np.float32) for w in weights]
    cp = (C.c_void_p * n)(*[a.ctypes.data for a in cs])
    sp = (C.c_void_p * n)(*[a.ctypes.data for a in ss])
    yp = (C.c_void_p * n)(*[a.ctypes.data for a in ys])
    q, as_, sum16 = _c(q, np.int8), _c(as_, np.float32), _c(sum16, np.int32)
    rc = lib().orc_gemv_w4a8_fanout(cp, sp, Ms, C.c_int(n), C.c_int(K), C.c_int(ksh), _p(q), _p(as_),
                                    _p(sum16), yp, C.c_int(fma))
    return rc, ys


def gemm_w4a8(codes, scales, M, K, ksh, aq, as_, asum, T, offsets=None, forced_splits=0, fma=1):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    aq, as_, asum = _c(aq, np.int8), _c(as_, np.float32), _c(asum, np.int32)
    y = np.empty((T, M), dtype=np.float32)
    if offsets is not None:
        off = (C.c_int * len(offsets))(*offsets)
        nseg = len(offsets) - 1
    else:
        off, nseg = None, 0
    rc = lib().orc_gemm_w4a8(_p(codes), _p(scales), C.c_int(M), C.c_int(K), C.c_int(ksh), _p(aq),
                             _p(as_), _p(asum), _p(y), C.c_int(T), off, C.c_int(nseg),
                             C.c_int(forced_splits), C.c_int(fma))
    return rc, y


def gemm_w4a8_pertoken(codes, scales, M, K, ksh, aq, as_tok, asum, T, splits=1):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    aq, as_tok, asum = _c(aq, np.int8), _c(as_tok, np.float32), _c(asum, np.int32)
    y = np.empty((T, M), dtype=np.float32)
    rc = lib().orc_gemm_w4a8_pertoken(_p(codes), _p(scales), C.c_int(M), C.c_int(K), C.c_int(ksh),
                                      _p(aq), _p(as_tok), _p(asum), _p(y), C.c_int(T),
                                      C.c_int(splits))
    return rc, y


def w8_repack(payload, bs, scale_cols, M, K):
    payload, bs = _c(payload, np.uint8), _c(bs, np.float32)
    codes = np.empty(M * K, dtype=np.uint8)
    scales = np.empty(M * (K // 32), dtype=np.uint16)
    rc = lib().orc_w8_repack(_p(payload), _p(bs), C.c_int(scale_cols), C.c_int(M), C.c_int(K),
                             _p(codes), _p(scales))
    return rc, codes, scales


def gemv_w8a8(codes, scales, M, K, q, as_, residual=None, fma=1):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    q, as_ = _c(q, np.int8), _c(as_, np.float32)
    res = _c(residual, np.float32) if residual is not None else None
    y = np.empty(M, dtype=np.float32)
    rc = lib().orc_gemv_w8a8(_p(codes), _p(scales), C.c_int(M), C.c_int(K), _p(q), _p(as_),
                             _p(res) if res is not None else None, _p(y), C.c_int(fma))
    assert rc == 0, rc
    return y


def gemm_w8a8(codes, scales, M, K, aq, as_, T, fma=1):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    aq, as_ = _c(aq, np.int8), _c(as_, np.float32)
    y = np.empty((T, M), dtype=np.float32)
    rc = lib().orc_gemm_w8a8(_p(codes), _p(scales), C.c_int(M), C.c_int(K), _p(aq), _p(as_), _p(y),
                             C.c_int(T), C.c_int(fma))
    return rc, y


def quantize_act_chunk_s4(x):
    x = _c(x, np.float32)
    T, K = x.shape
    n = K // 64 * T
    aq4 = np.empty(n * 32, dtype=np.uint8)
    as4 = np.empty(n, dtype=np.float32)
    asum4 = np.empty(n, dtype=np.int32)
    lib().orc_quantize_act_chunk_s4(_p(x), C.c_int(K), C.c_int(T), _p(aq4), _p(as4), _p(asum4))
    return aq4, as4, asum4


def gemm_w4a4(codes, scales, M, K, aq4, as4, asum4, T, fma=1):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    aq4, as4, asum4 = _c(aq4, np.uint8), _c(as4, np.float32), _c(asum4, np.int32)
    y = np.empty((T, M), dtype=np.float32)
    rc = lib().orc_gemm_w4a4(_p(codes), _p(scales), C.c_int(M), C.c_int(K), _p(aq4), _p(as4),
                             _p(asum4), _p(y), C.c_int(T), C.c_int(fma))
    return rc, y


def w4_shard_column(codes, scales, M, K, ksh, rank, tp, groups=None, k16=0):
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint16)
    Kt = K // 32
    Mn = M // tp if tp >= 1 else M
    dc = np.zeros(max(Mn, 16) * K // 2, dtype=np.uint8)
    ds = np.zeros(max(Mn, 16) * (Kt >> ksh), dtype=np.uint16)
    if groups:
        g = (C.c_int * len(groups))(*groups)
        ng = len(groups)
    else:
        g, ng = None, 0
    rc = lib().orc_w4_shard_column(_p(codes), _p(scales), C.c_int(M), C.c_int(K), C.c_int(ksh),
                                   C.c_int(k16), C.c_int(rank), C.c_int(tp), g, C.c_int(ng),
                                   _p(dc), _p(ds))
    return rc, dc[: Mn * K // 2], ds[: Mn * (Kt >> ksh)]


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


# ---- weight-format probe (xpu/src/kernels_dpas.cpp:1726-2146), vectorised restatement -------
def _f16rt(s):
    return s.astype(np.float16).astype(np.float32)


def _stored_f16(s):
    """fp16 bits with the low nibble rounded away, as the packed scale stores them."""
    b = s.astype(np.float16).view(np.uint16).astype(np.uint32)
    return (((b + 8) & 0xFFF0).astype(np.uint16)).view(np.float16).astype(np.float32)


def _fit_sym(V, lo_q, hi_q):
    f = np.float32
    hi = np.maximum(V, 0).max(axis=-1)
    neg = np.maximum(-V, 0).max(axis=-1)
    s = np.maximum(hi / f(hi_q), neg / f(-lo_q)).astype(f)
    s[~(s > 0)] = 1.0
    for _ in range(2):
        q = np.clip(np.rint(V / s[..., None]), lo_q, hi_q).astype(f)
        num, den = (V * q).sum(axis=-1, dtype=f), (q * q).sum(axis=-1, dtype=f)
        s = np.where(den > 0, num / np.where(den > 0, den, 1), s).astype(f)
    return _f16rt(s)


def _fit_asym(V, half_q):
    """Asymmetric fit with codes in [-half_q, half_q - 1] (kernels_dpas.cpp:229-256 for 8)."""
    f = np.float32
    lo = np.minimum(V, 0).min(axis=-1)
    hi = np.maximum(V, 0).max(axis=-1)
    s = ((hi - lo) / f(2 * half_q - 1)).astype(f)
    s[~(s > 0)] = 1.0
    for _ in range(3):
        zi = np.clip(np.rint(-lo / s) - half_q, -half_q, half_q - 1).astype(f)
        c = np.clip(np.rint(V / s[..., None] + zi[..., None]), -half_q, half_q - 1).astype(f) - zi[..., None]
        num, den = (V * c).sum(axis=-1, dtype=f), (c * c).sum(axis=-1, dtype=f)
        s = np.where(den > 0, num / np.where(den > 0, den, 1), s).astype(f)
    s = _stored_f16(s)
    zp = np.clip(np.rint(-lo / s) - half_q, -half_q, half_q - 1).astype(f)
    return s, zp


def _asym_hat(V, s, zp, half_q):
    q = np.clip(np.rint(V / s[..., None] + zp[..., None]), -half_q, half_q - 1).astype(np.float32)
    return (s[..., None] * (q - zp[..., None])).astype(np.float32)


def _round_e4m3(v):
    f = np.float32
    v = v.astype(f)
    out = np.zeros_like(v)
    pos = v > 0
    big = pos & (v >= 448)
    sub = pos & (v < 0.015625)
    nor = pos & ~big & ~sub
    out[big] = 448.0
    out[sub] = np.minimum(np.rint(v[sub] * f(512.0)), 7.0) * f(0.001953125)
    x = v[nor]
    e = np.floor(np.log2(x.astype(np.float64))).astype(np.int32)
    p = np.ldexp(f(1.0), e).astype(f)
    q = np.rint((x / p - f(1.0)) * f(8.0)).astype(np.int32)
    roll = q >= 8
    q[roll] = 0
    e[roll] += 1
    p[roll] *= f(2.0)
    top = e >= 8
    p[top] = 256.0
    q[top] = np.minimum(q[top], 6)
    out[nor] = p * (f(1.0) + q.astype(f) * f(0.125))
    return out


def _round_e2m1(v):
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
    best = np.zeros_like(v)
    bd = np.abs(v)
    for gval in grid[1:]:
        d = np.abs(v - gval)
        take = d < bd
        bd = np.where(take, d, bd)
        best = np.where(take, gval, best)
    return best.astype(np.float32)


def w4_grid_probe(W):
    """Cosine, relative L2 error and bits per weight of the eleven formats on W[M][K]
    (the decoded E2M3 source), and the reference's verdict (0: the shipped tier wins)."""
    f = np.float32
    W = _c(W, f)
    M, K = W.shape
    Kt = K // 32
    V = W.reshape(M, Kt, 32)
    glob = np.abs(W.reshape(-1, min(128, M), K) if M % 128 == 0 else W[None]).max(axis=(1, 2)) if M % 128 == 0 else None
    if glob is None:
        nrb = (M + 127) // 128
        glob = np.array([np.abs(W[b * 128:(b + 1) * 128]).max() for b in range(nrb)], dtype=f)
    g_row = glob[np.arange(M) // 128].astype(f)[:, None, None]          # per (row, kt, half)
    hats = {}
    s = _fit_sym(V, -8.0, 7.0)
    hats[0] = s[..., None] * np.clip(np.rint(V / s[..., None]), -8, 7).astype(f)
    s4, zp4 = _fit_asym(V, 8.0)
    hats[1] = _asym_hat(V, s4, zp4, 8.0)
    U = V.reshape(M, Kt, 2, 16)
    s2, zp2 = _fit_asym(U, 8.0)
    hats[2] = _asym_hat(U, s2, zp2, 8.0).reshape(M, Kt, 32)
    mx = np.abs(U).max(axis=-1)
    lo, hi = np.minimum(U, 0).min(axis=-1), np.maximum(U, 0).max(axis=-1)
    has = g_row > 0
    g3 = np.where(has, g_row / f(6.0 * 448.0), f(1.0)).astype(f)
    s3 = (_round_e4m3(mx / (f(6.0) * g3)) * g3).astype(f)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(s3[..., None] > 0, U / np.where(s3 > 0, s3, 1)[..., None], 0).astype(f)
    hats[3] = np.where(s3[..., None] > 0, np.copysign(_round_e2m1(np.abs(r)), U) * s3[..., None], 0).astype(f).reshape(M, Kt, 32)
    s = _f16rt(np.where(np.abs(V).max(axis=-1) > 0, np.abs(V).max(axis=-1) / f(127.0), f(1.0)).astype(f))
    hats[4] = s[..., None] * np.clip(np.rint(V / s[..., None]), -128, 127).astype(f)
    g5 = np.where(has, (f(2.0) * g_row) / f(15.0 * 448.0), f(1.0)).astype(f)
    s5 = (_round_e4m3(((hi - lo) / f(15.0)) / g5) * g5).astype(f)
    s5 = np.where(s5 > 0, s5, np.broadcast_to(g5, s5.shape)).astype(f)
    zp5 = np.clip(np.rint(-lo / s5) - 8.0, -8, 7).astype(f)
    hats[5] = _asym_hat(U, s5, zp5, 8.0).reshape(M, Kt, 32)
    g6 = np.where(has, g_row / f(8.0 * 448.0), f(1.0)).astype(f)
    s6 = (_round_e4m3((mx / f(8.0)) / g6) * g6).astype(f)
    s6 = np.where(s6 > 0, s6, np.broadcast_to(g6, s6.shape)).astype(f)
    hats[6] = (s6[..., None] * np.clip(np.rint(U / s6[..., None]), -8, 7).astype(f)).reshape(M, Kt, 32)
    s = _fit_sym(V, -4.0, 3.0)
    hats[7] = s[..., None] * np.clip(np.rint(V / s[..., None]), -4, 3).astype(f)
    s8, zp8 = _fit_asym(V, 4.0)
    hats[8] = _asym_hat(V, s8, zp8, 4.0)
    err3 = ((V - hats[8]) ** 2).sum(axis=-1, dtype=f)
    err4 = ((V - hats[1]) ** 2).sum(axis=-1, dtype=f)
    use3 = err3 <= f(1.8) * err4
    hats[9] = np.where(use3[..., None], hats[8], hats[1])
    P = W.reshape(M, Kt // 2, 64)
    s10, zp10 = _fit_asym(P, 8.0)
    hats[10] = _asym_hat(P, s10, zp10, 8.0).reshape(M, Kt, 32)
    na = float((V.astype(np.float64) ** 2).sum())
    bits = [4.50, 4.50, 5.00, 4.50, 8.50, 4.75, 4.50, 3.50, 3.50, 0.0, 4.25]
    groups = M * Kt
    count3 = float(use3.sum())
    bits[9] = 0.5 + (3.0 * count3 + 4.0 * (groups - count3)) / groups
    cos, rel = [], []
    for k in range(11):
        h = hats[k].astype(np.float64)
        dot, nb = float((V * h).sum()), float((h * h).sum())
        cos.append(dot / (np.sqrt(na) * np.sqrt(nb)) if na > 0 and nb > 0 else 0.0)
        rel.append(np.sqrt(max(0.0, na - 2 * dot + nb) / na) if na > 0 else 0.0)
    best = 1
    for k in range(11):
        if k != 1 and bits[k] <= bits[1] + 1e-9 and cos[k] > cos[best]:
            best = k
    return np.array(cos), np.array(rel), np.array(bits), (0 if best == 1 else 1)
