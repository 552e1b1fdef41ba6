"""Closed-form inputs the reference's own checks and probes use, restated in numpy."""
import numpy as np


def gemm_check_rows(T, K, prefix=None, salt=0):
    """xpu/src/kernels_dpas.cpp:2225-2234, 2280-2286."""
    prefix = T if prefix is None else prefix
    k = np.arange(K, dtype=np.int64)[None, :]
    t = np.arange(T, dtype=np.int64)[:, None]
    s = np.where(t >= prefix, salt, 0).astype(np.int64)
    mag = np.exp2(((k * 7 + t * 3 + (s & 7)) % 13 - 6).astype(np.float32)).astype(np.float32)
    h = ((k * 2654435761 + t) & 0xFFFFFFFF) ^ s
    sgn = np.where((h >> 31) & 1, -1.0, 1.0).astype(np.float32)
    x = sgn * mag
    x[:, (np.arange(K) % 97) == 0] = 0.0
    return np.ascontiguousarray(x, dtype=np.float32)


def w4_check_row(K):
    """xpu/src/kernels_dpas.cpp:2705-2710."""
    return gemm_check_rows(1, K)[0]


def shard_check_row(K):
    """xpu/src/kernels_dpas.cpp:2517-2518."""
    j = np.arange(K, dtype=np.uint64)
    v = ((j * 1103515245 + 12345) & 0xFFFFFFFF) % 97
    return (np.float32(0.05) * v.astype(np.float32) - np.float32(2.0)).astype(np.float32)


def lcg_floats(n, seed=391):
    """Probe LCG (xpu/probe/chunk_quant_bench.cpp:55-59): returns values and final seed."""
    out = np.empty(n, dtype=np.float32)
    s = seed
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(((s >> 8) - 8388608)) / np.float32(1048576.0)
    return out, s


def chunk_quant_probe_input(K, T, exceptional):
    """xpu/probe/chunk_quant_bench.cpp:52-100: LCG values with zero / denormal / half-way /
    FLT_MAX blocks, and (exceptional) NaN and infinity walks."""
    n = K * T
    x, _ = lcg_floats(n)
    fmax = np.finfo(np.float32).max
    den = np.float32(1e-45)
    for block in range(n // 64):
        p = x[block * 64:(block + 1) * 64]
        m = block % 16
        if m == 0:
            p[:] = 0.0
            p[0] = -0.0
        elif m == 1:
            j = np.arange(64)
            p[:] = np.where(j & 1, -1.0, 1.0).astype(np.float32) * np.float32(1.0e-20) * (j + 1).astype(np.float32)
        elif m == 2:
            p[:] = (np.arange(64) - 32).astype(np.float32) + np.float32(0.5)
            p[0] = p[32] = 127.0
        elif m == 3:
            p[:] = den
            p[0] = -den
        elif m == 4:
            p[0] = fmax
            p[32] = -fmax
        if exceptional:
            p[block % 64] = np.nan
            if block % 67 == 0:
                p[:] = np.nan
            elif block % 67 == 1:
                p[(block + 17) % 64] = np.inf
            elif block % 67 == 2:
                p[(block + 31) % 64] = -np.inf
    return x.reshape(T, K)
