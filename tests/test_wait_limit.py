"""A bounded device-side wait that runs out: the kernel returns, the host reads the status.

The fused all-gather waits, inside a kernel, for a step flag that every other rank stores
into this rank's flag array. Here the "other rank" is a second set of plain buffers on the
same GPU that nobody ever publishes to, so the wait can only end by its wall-clock limit
(shortened to 50 ms). Nothing faults, traps or spins forever: the kernel records status 31,
returns normally, and the context stays usable.
"""
import ctypes as C

import numpy as np
import pytest

import refgen

pytestmark = pytest.mark.gpu


def test_gather_flag_wait_gives_up_and_reports(lib, pkg, wl):
    K, T, M = 512, 8, 1088
    w = pkg.PackedWeight(*wl.random_packed_weight(M, K, seed=5, ksh=1), M, K, k64=True)
    x = refgen.gemm_check_rows(T, K)
    dx = pkg.DevBuf.from_numpy(x)
    n = K // 32 * T
    aq, as_, asum = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4)
    lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    y = pkg.DevBuf(T * M * 4)
    warr = pkg.weight_array([w])
    assert lib.qwn_x_gemm_w4a8_fanout(warr, pkg.ptr_array([y]), 1, aq.ptr, as_.ptr, asum.ptr, T,
                                      None, 0) == 0
    lib.tq_sync()
    want = y.to_numpy(np.float32)
    assert lib.tq_last_error() == 0

    block = T * M
    mine, peer = pkg.DevBuf(2 * 2 * block * 4), pkg.DevBuf(2 * 2 * block * 4)
    fmine, fpeer = pkg.DevBuf(8), pkg.DevBuf(8)
    lib.tq_dev_zero(fpeer.ptr, 8)
    bufs = (C.c_void_p * 2)(mine.ptr, peer.ptr)
    flags = (C.c_void_p * 2)(fmine.ptr, fpeer.ptr)
    assert lib.tq_comm_gather_setup(bufs, flags, 2, 0) == 0      # world of 2; rank 1 never runs
    lib.tq_set_wait_limit_ms(50)
    try:
        off = C.c_size_t(0)
        assert lib.qwn_x_gemm_w4a8_fanout_gathered(warr, 1, aq.ptr, as_.ptr, asum.ptr, T,
                                                   C.byref(off)) == 0
        lib.tq_sync()                                  # returns: the wait gave up after 50 ms
        assert lib.tq_last_error() == 10031
        # this rank's own slice did arrive in both buffers, and its own flag was published
        got = mine.to_numpy(np.float32)[off.value: off.value + block]
        assert got.tobytes() == want.tobytes()
        got_peer = peer.to_numpy(np.float32)[off.value: off.value + block]
        assert got_peer.tobytes() == want.tobytes()
        assert fmine.to_numpy(np.int32)[0] == 1 and fpeer.to_numpy(np.int32)[0] == 1
        assert fmine.to_numpy(np.int32)[1] == 0        # rank 1's word: never written
    finally:
        lib.tq_set_wait_limit_ms(2000)
        lib.tq_clear_error()
    assert lib.tq_last_error() == 0
    # the context is intact: an ordinary call gives the same bits as before
    y.fill(0xA5)
    assert lib.qwn_x_gemm_w4a8_fanout(warr, pkg.ptr_array([y]), 1, aq.ptr, as_.ptr, asum.ptr, T,
                                      None, 0) == 0
    lib.tq_sync()
    assert y.to_numpy(np.float32).tobytes() == want.tobytes()
    assert lib.tq_last_error() == 0
    # leave a world of one behind for whatever uses the gather next
    one_b, one_f = (C.c_void_p * 1)(mine.ptr), (C.c_void_p * 1)(fmine.ptr)
    assert lib.tq_comm_gather_setup(one_b, one_f, 1, 0) == 0
