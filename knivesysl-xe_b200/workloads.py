"""Seeded synthetic weights and activations of the benchmark shapes, and the host-side
packing into the reference's packed W4 layout (xpu/src/kernels_dpas.cpp:327-342:
tile (g, kt) at ((g*Kt+kt)*256), row n owns 16 bytes, byte b = k 2b (low nibble), 2b+1).

numpy only; used by the benchmark and the tests to build inputs. No model file exists
for this path, so every input is generated.
"""
from __future__ import annotations

import numpy as np


def pack_codes(q: np.ndarray) -> np.ndarray:
    """q[M][K] int (values -8..7) -> packed bytes [Mt][Kt][16][16]."""
    M, K = q.shape
    u = (q.astype(np.int16) & 0xF).astype(np.uint8).reshape(M // 16, 16, K // 32, 32)
    u = u.transpose(0, 2, 1, 3)
    return np.ascontiguousarray(u[..., 0::2] | (u[..., 1::2] << 4)).reshape(-1)


def unpack_codes(codes: np.ndarray, M: int, K: int) -> np.ndarray:
    b = codes.reshape(M // 16, K // 32, 16, 16)
    u = np.empty((M // 16, K // 32, 16, 32), dtype=np.int8)
    u[..., 0::2] = (b & 0xF).astype(np.int8)
    u[..., 1::2] = (b >> 4).astype(np.int8)
    u = np.where(u >= 8, u - 16, u).astype(np.int8)
    return np.ascontiguousarray(u.transpose(0, 2, 1, 3)).reshape(M, K)


def pack_scales(s: np.ndarray) -> np.ndarray:
    """s[M][G] uint16 -> [Mt][G][16]."""
    M, G = s.shape
    return np.ascontiguousarray(s.reshape(M // 16, 16, G).transpose(0, 2, 1)).reshape(-1)


def symmetric_w4(W: np.ndarray, group: int):
    """Symmetric int4 quantisation with one FP16 scale per `group` (32 or 64) K elements:
    scale = fp16(max|w| / 7) with the low nibble rounded away ((bits+8)&0xFFF0), zero point
    0, codes clamp(rint(w / stored_scale), -8, 7). Returns packed (codes, scales)."""
    M, K = W.shape
    G = K // group
    Wg = W.reshape(M, G, group)
    s = (np.abs(Wg).max(axis=2) / np.float32(7.0)).astype(np.float32)
    s[s <= 0] = 1.0
    bits = s.astype(np.float16).view(np.uint16).astype(np.uint32)
    bits = ((bits + 8) & 0xFFF0).astype(np.uint16)
    stored = bits.view(np.float16).astype(np.float32)
    stored_safe = np.where(stored > 0, stored, np.float32(1.0))
    q = np.clip(np.rint(Wg / stored_safe[:, :, None]), -8, 7).astype(np.int8).reshape(M, K)
    return pack_codes(q), pack_scales(bits)


def normal_weights(M: int, K: int, seed: int, std: float = 0.02) -> np.ndarray:
    rng = np.random.Generator(np.random.Philox(key=seed))
    return (rng.standard_normal((M, K), dtype=np.float32) * np.float32(std)).astype(np.float32)


def make_weight_w4(M: int, K: int, seed: int, group: int = 32, chunk_rows: int = 2048):
    """N(0, 0.02) weights -> packed symmetric int4, generated in row chunks."""
    codes, scales = [], []
    rng = np.random.Generator(np.random.Philox(key=seed))
    for r0 in range(0, M, chunk_rows):
        rows = min(chunk_rows, M - r0)
        W = rng.standard_normal((rows, K), dtype=np.float32) * np.float32(0.02)
        c, s = symmetric_w4(W, group)
        codes.append(c)
        scales.append(s)
    return np.concatenate(codes), np.concatenate(scales)


def random_packed_weight(M: int, K: int, seed: int, ksh: int = 0, k16: bool = False):
    """Arbitrary codes, positive normal FP16 scales with every zero point -8..7 and some
    zero scales: the pattern of the reference's fan-out probe (xpu/probe/fanout_bench.cpp:
    66-77), driven by its LCG."""
    n_codes = M * K // 2
    n_scales = M * (K // 16) if k16 else M * ((K // 32) >> ksh)
    state = np.uint32(391 + seed)
    # vectorised LCG: x_{n} = a^n x0 + c (a^n - 1)/(a - 1) is awkward in uint32, so use numpy's
    # generator for bulk values and keep the scale pattern itself exact
    rng = np.random.Generator(np.random.Philox(key=int(state)))
    codes = rng.integers(0, 256, size=n_codes, dtype=np.uint8)
    mant = rng.integers(0, 64, size=n_scales, dtype=np.uint16)
    idx = np.arange(n_scales)
    mag = np.where(idx % 37 == 0, 0, 0x2400 + mant * 16).astype(np.uint16)
    scales = (mag | (idx & 15).astype(np.uint16)).astype(np.uint16)
    return codes, scales


def activations_normal(T: int, K: int, seed: int, outlier_frac: float = 0.0,
                       outlier_gain: float = 20.0) -> np.ndarray:
    rng = np.random.Generator(np.random.Philox(key=seed))
    x = rng.standard_normal((T, K), dtype=np.float32)
    if outlier_frac > 0:
        n = max(1, int(round(K * outlier_frac)))
        ch = rng.choice(K, size=n, replace=False)
        x[:, ch] *= np.float32(outlier_gain)
    return x


def weight_bytes(M: int, K: int, group: int) -> int:
    """Algorithmic weight bytes of one pass: codes + FP16 scales (xpu/tools/bench_gemm.py:54)."""
    return M * K // 2 + M * (K // group) * 2
