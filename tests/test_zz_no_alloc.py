"""The allocation-free GEMV entry point against the ordinary one, through the C-ABI.

Why it exists: some users of this library pre-allocate all device memory (or hand the whole
GPU to their own pool) and cannot let a projection call reach cudaMalloc, which the ordinary
GEMV does when it grows its activation scratch. qwn_x_gemv_w4a8_static stages the activation
in an array built into the library instead. This file is collected last on purpose, and the
test also has to pass when it is the only thing run in a fresh process.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

import refgen

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

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


def test_static_gemv_allocates_nothing_where_the_regular_one_must(lib, pkg, wl):
    """K = 32768 is larger than any row staged before in this process, so the regular GEMV has
    to grow its scratch (tq_dev_alloc is called), while the static entry point, called first,
    leaves both the library's allocation counter and the driver's free-memory figure alone."""
    M, K = 64, lib.qwn_static_max_k()
    c, s = wl.random_packed_weight(M, K, seed=9)
    w = pkg.PackedWeight(c, s, M, K)
    x = wl.activations_normal(1, K, seed=10)[0]
    dx = pkg.DevBuf.from_numpy(x)
    y_new, y_ref = pkg.DevBuf(M * 4), pkg.DevBuf(M * 4)
    lib.tq_sync()
    before = lib.tq_dev_alloc_count()
    for _ in range(2):
        assert lib.qwn_x_gemv_w4a8_static(w.ref, dx.ptr, y_new.ptr) == 0
    lib.tq_sync()
    assert lib.tq_dev_alloc_count() == before
    assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y_ref.ptr) == 0
    lib.tq_sync()
    assert lib.tq_dev_alloc_count() > before         # the ordinary path had to allocate
    assert y_new.to_numpy(np.float32).tobytes() == y_ref.to_numpy(np.float32).tobytes()
    assert lib.tq_last_error() == 0


_COLD = r"""
import importlib, sys
import numpy as np
sys.path.insert(0, {root!r})
sys.path.insert(0, {root!r} + "/tests")
pkg = importlib.import_module("knivesysl-xe_b200")
wl = importlib.import_module("knivesysl-xe_b200.workloads")
lib = pkg.load()
assert lib.tq_set_device(0) == 0
M, K = 320, 1024
c, s = wl.make_weight_w4(M, K, seed=4, group=32)
w = pkg.PackedWeight(c, s, M, K)
x = wl.activations_normal(1, K, seed=6)[0]
dx = pkg.DevBuf.from_numpy(x)
y0, y1 = pkg.DevBuf(M * 4), pkg.DevBuf(M * 4)
n = lib.tq_dev_alloc_count()
assert lib.qwn_x_gemv_w4a8_static(w.ref, dx.ptr, y0.ptr) == 0   # first projection call at all
lib.tq_sync()
assert lib.tq_dev_alloc_count() == n
assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y1.ptr) == 0
lib.tq_sync()
assert y0.to_numpy(np.float32).tobytes() == y1.to_numpy(np.float32).tobytes()
assert lib.tq_last_error() == 0
print("cold ok")
"""


def test_static_gemv_as_the_first_call_of_a_fresh_process(lib):
    """The address of the built-in array is looked up on the first call; here that call is
    the first projection call the process ever makes (no kernel of the library has run)."""
    out = subprocess.run([sys.executable, "-c", _COLD.format(root=ROOT)], capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0 and "cold ok" in out.stdout, out.stdout + out.stderr
