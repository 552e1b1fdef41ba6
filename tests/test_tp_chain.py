"""The tensor-parallel decode chain on one GPU: column shards computed one after the other
through the scatter API fill the same activation matrix the unsharded call produces, bit for
bit (a shard keeps the split count of the whole weight), and the exchange points work in a
world of one (the rank waits for its own flag), eagerly and when replayed from a CUDA graph."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("per_token", [True, False])
@pytest.mark.parametrize("M,K,T,tp", [(5120, 1024, 8, 4), (2048, 2112, 8, 2), (1024, 512, 16, 8)])
def test_column_shards_scatter_to_the_unsharded_result(lib, pkg, orc, wl, M, K, T, tp, per_token):
    codes, scales = wl.random_packed_weight(M, K, seed=M + K + tp)
    w = pkg.PackedWeight(codes, scales, M, K)
    x = wl.activations_normal(T, K, seed=3, outlier_frac=0.01)
    dx = pkg.DevBuf.from_numpy(x)
    n = K // 32 * T
    aq, as_, asum, at = pkg.DevBuf(n * 32), pkg.DevBuf(n * 4), pkg.DevBuf(n * 4), pkg.DevBuf(T * 4)
    if per_token:
        lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
    else:
        lib.qwn_x_quantize_act_chunk(dx.ptr, K, T, aq.ptr, as_.ptr, asum.ptr)
    full = pkg.DevBuf(T * M * 4)
    if per_token:
        assert lib.qwn_x_gemm_w4a8_pertoken(w.ref, aq.ptr, at.ptr, asum.ptr, full.ptr, T, 0) == 0
    else:
        assert lib.qwn_x_gemm_w4a8(w.ref, aq.ptr, as_.ptr, asum.ptr, full.ptr, T, None, 0) == 0
    lib.tq_sync()
    want = full.to_numpy(np.float32)
    # a world of one whose symmetric matrix is wider than the projection: ld = M + 64
    ld = M + 64
    mat, flags = pkg.DevBuf(T * ld * 4), pkg.DevBuf(4)
    mat.fill(0xA5)
    one = C.c_void_p * 1
    assert lib.tq_comm_gather_setup(one(mat.ptr), one(flags.ptr), 1, 0) == 0
    assert lib.tq_comm_sym_register(5, one(mat.ptr)) == 0
    for r in range(tp):
        sh = pkg.TqWeight()
        assert lib.qwn_x_w4_shard(C.byref(sh), w.ref, r, tp, 0, None, 0) == 0
        warr = (C.POINTER(pkg.TqWeight) * 1)(C.pointer(sh))
        rc = lib.qwn_x_gemm_w4a8_fanout_tp(warr, 1, aq.ptr, None if per_token else as_.ptr,
                                           at.ptr if per_token else None, asum.ptr, T, (C.c_int * 1)(M),
                                           None, 5, (C.c_size_t * 1)(32 + r * (M // tp)), ld)
        assert rc == 0, rc
        lib.tq_sync()
        lib.qwn_x_w4_shard_free(C.byref(sh))
    got = mat.to_numpy(np.float32).reshape(T, ld)
    assert got[:, 32:32 + M].tobytes() == want.reshape(T, M).tobytes()
    # the columns beside the projection were not touched
    assert np.all(got[:, :32].view(np.uint32) == 0xA5A5A5A5)
    assert np.all(got[:, 32 + M:].view(np.uint32) == 0xA5A5A5A5)
    assert lib.tq_last_error() == 0


def test_exchange_points_in_a_world_of_one_and_graph_replay(lib, pkg, wl):
    """norm -> staging(sync) -> scatter GEMM -> silu*mul scatter -> staging(sync), issued
    eagerly twice and replayed from a CUDA graph three times: every pass gives the same bytes
    and the step base advances by the pass's exchange points."""
    T, H, N = 8, 1024, 2048
    w1 = pkg.PackedWeight(*wl.random_packed_weight(2 * N, H, seed=1), 2 * N, H)     # gate|up as one
    x = wl.activations_normal(T, H, seed=2)
    dx = pkg.DevBuf.from_numpy(x)
    y1, hbuf, flags = pkg.DevBuf(T * 2 * N * 4), pkg.DevBuf(T * N * 4), pkg.DevBuf(4)
    one = C.c_void_p * 1
    assert lib.tq_comm_gather_setup(one(y1.ptr), one(flags.ptr), 1, 0) == 0
    assert lib.tq_comm_sym_register(0, one(y1.ptr)) == 0
    assert lib.tq_comm_sym_register(1, one(hbuf.ptr)) == 0
    nb = 2 * N // 32 * T
    aq, as_, asum, at = pkg.DevBuf(nb * 32), pkg.DevBuf(nb * 4), pkg.DevBuf(nb * 4), pkg.DevBuf(T * 4)
    warr = (C.POINTER(pkg.TqWeight) * 1)(C.pointer(w1.rec))

    def issue():
        lib.qwn_x_quantize_act_chunk_pertoken(dx.ptr, H, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
        assert lib.qwn_x_gemm_w4a8_fanout_tp(warr, 1, aq.ptr, None, at.ptr, asum.ptr, T, None, None, 0,
                                             (C.c_size_t * 1)(0), 2 * N) == 0
        # the next reader of y1 carries the exchange point
        lib.qwn_x_quantize_act_chunk_pertoken_sync(y1.ptr, 2 * N, T, aq.ptr, as_.ptr, asum.ptr, at.ptr)
        assert lib.tq_comm_exchange_sync() == 0
        assert lib.tq_comm_exchange_advance() == 0

    issue()
    lib.tq_sync()
    first = (y1.to_numpy(np.uint32).copy(), aq.to_numpy(np.uint8).copy())
    assert flags.to_numpy(np.int32)[0] == 2
    issue()
    lib.tq_sync()
    assert flags.to_numpy(np.int32)[0] == 4
    assert lib.tq_graph_capture_begin() == 0
    issue()
    g = lib.tq_graph_capture_end()
    assert g
    for rep in range(3):
        y1.fill(0)
        lib.tq_graph_launch(g)
        lib.tq_sync()
        assert np.array_equal(y1.to_numpy(np.uint32), first[0])
        assert np.array_equal(aq.to_numpy(np.uint8), first[1])
        assert flags.to_numpy(np.int32)[0] == 6 + 2 * rep
    lib.tq_graph_destroy(g)
    assert lib.tq_last_error() == 0
