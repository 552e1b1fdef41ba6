"""The allocation-free GEMV entry point against the ordinary one, through the C-ABI.

Why it exists: some users of this library pre-allocate all device memory (or hand the whole
GPU to their own pool) and cannot let a projection call reach cudaMalloc, which the ordinary
GEMV does when it grows its activation scratch. qwn_x_gemv_w4a8_static stages the activation
in an array built into the library instead. This file is collected last on purpose, and the
test also has to pass when it is the only thing run in a fresh process.
"""
import numpy as np
import pytest

import refgen

pytestmark = pytest.mark.gpu


def test_static_gemv_matches_regular_gemv_twice_in_a_row(lib, pkg, wl):
    M, K = 1088, 5120
    codes, scales = wl.make_weight_w4(M, K, seed=3, group=64)
    w = pkg.PackedWeight(codes, scales, M, K, k64=True)
    xs = [refgen.shard_check_row(K), wl.activations_normal(1, K, seed=8, outlier_frac=0.01)[0]]
    y_ref, y_new = pkg.DevBuf(M * 4), pkg.DevBuf(M * 4)
    for x in xs:                       # second call reuses the array the first one left dirty
        dx = pkg.DevBuf.from_numpy(x)
        y_ref.fill(0xA5)
        y_new.fill(0x5A)
        assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y_ref.ptr) == 0
        assert lib.qwn_x_gemv_w4a8_static(w.ref, dx.ptr, y_new.ptr) == 0
        lib.tq_sync()
        # same tolerance as the other GPU tests: bit-for-bit
        assert y_new.to_numpy(np.float32).tobytes() == y_ref.to_numpy(np.float32).tobytes()
    assert lib.tq_last_error() == 0


def test_static_gemv_rejects_oversized_k(lib, pkg, wl):
    kmax = lib.qwn_static_max_k()
    assert kmax == 32768
    c, s = wl.random_packed_weight(16, 128, seed=1)
    big = pkg.PackedWeight(c, s, 16, kmax + 32)      # never launched: rejected on the host
    y, x = pkg.DevBuf(64), pkg.DevBuf(16)
    assert lib.qwn_x_gemv_w4a8_static(big.ref, x.ptr, y.ptr) == -30
    assert lib.qwn_x_gemv_w4a8_static(None, x.ptr, y.ptr) == -1
