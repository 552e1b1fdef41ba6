"""Per-projection timers: off by default, and with profiling on every GEMV / GEMM entry point is
timed by a pair of events on the stream and reported per (rows, K, tokens, tier)."""
import ctypes as C

import numpy as np
import pytest


@pytest.mark.gpu
def test_projection_timers(lib, pkg, wl):
    M, K, T = 1088, 1024, 8
    codes, scales = wl.make_weight_w4(M, K, seed=1, group=64)
    w = pkg.PackedWeight(codes, scales, M, K, k64=True)
    codes2, scales2 = wl.make_weight_w4(256, K, seed=2, group=32)
    w2 = pkg.PackedWeight(codes2, scales2, 256, K)
    x = wl.activations_normal(T, K, seed=2)
    dx = pkg.DevBuf.from_numpy(x)
    y, y2 = pkg.DevBuf(T * M * 4), pkg.DevBuf(256 * 4)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    rows = (C.c_double * (6 * 8))()

    def work():
        for _ in range(3):
            assert lib.qwn_x_gemv_w4a8(w.ref, dx.ptr, y.ptr) == 0
        assert lib.qwn_x_gemv_w4a8(w2.ref, dx.ptr, y2.ptr) == 0
        lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
        for _ in range(2):
            assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, y.ptr, T, None, 0) == 0

    was = lib.tq_profile_enable(0)
    try:
        work()
        assert lib.tq_profile_report(rows, 8) == 0              # off: nothing recorded
        lib.tq_profile_enable(1)
        work()
        nrec = lib.tq_profile_report(rows, 8)
        got = {(int(rows[6 * i]), int(rows[6 * i + 1]), int(rows[6 * i + 2]), int(rows[6 * i + 3])):
               (int(rows[6 * i + 4]), rows[6 * i + 5]) for i in range(nrec)}
        assert set(got) == {(M, K, 1, 64), (256, K, 1, 4), (M, K, T, 64)}
        assert got[(M, K, 1, 64)][0] == 3 and got[(256, K, 1, 4)][0] == 1 and got[(M, K, T, 64)][0] == 2
        assert all(0.5 < us < 5e4 for _, us in got.values())     # microseconds of device time
        assert lib.tq_profile_report(rows, 8) == 0              # the report clears the record
        # calls captured into a CUDA graph are not timed (their events would belong to the graph)
        assert lib.tq_graph_capture_begin() == 0
        assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, y.ptr, T, None, 0) == 0
        g = lib.tq_graph_capture_end()
        assert g
        lib.tq_graph_launch(g)
        assert lib.tq_profile_report(rows, 8) == 0
        lib.tq_graph_destroy(g)
    finally:
        lib.tq_profile_enable(was)
    assert lib.tq_last_error() == 0
