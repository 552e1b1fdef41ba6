"""ctypes binding of libforward_qwen_xpu.so (B200 build) — the same kind of binding the
reference's Python tools use over its flat C ABI (xpu/tools/bench_gemm.py:35-47).

There is no CPU fallback: importing works without a GPU (symbols can be inspected), but
any compute call needs the CUDA library and a device, and `load()` raises if the shared
object has not been built.

The directory name contains a hyphen; import it with
    importlib.import_module("knivesysl-xe_b200")
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libforward_qwen_xpu.so")

_lib = None


class TqWeight(C.Structure):
    """tq_qmma_weight_t (include/tq_w4a8.h; field order of xpu/src/tq_common.hpp:49-76)."""
    _fields_ = [
        ("M", C.c_int), ("K", C.c_int), ("Mt", C.c_int), ("Kt", C.c_int),
        ("inv_scale", C.c_float),
        ("d_A", C.c_void_p), ("d_block_scale_inv", C.c_void_p),
        ("block_scaled", C.c_int), ("row_major", C.c_int), ("word_major", C.c_int),
        ("e2m3", C.c_int), ("e2m1", C.c_int), ("e2m3_byte", C.c_int),
        ("scale_rows", C.c_int), ("scale_cols", C.c_int),
        ("d_s4", C.c_void_p), ("d_s4_scale", C.c_void_p),
        ("s4_ready", C.c_int), ("s4_k16", C.c_int), ("s4_k64", C.c_int),
        ("d_s8", C.c_void_p), ("d_s8_scale", C.c_void_p), ("s8_ready", C.c_int),
    ]


_WP = C.POINTER(TqWeight)
_vp, _i, _sz, _f, _d = C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_double

# name -> (restype, argtypes); every symbol include/tq_w4a8.h declares in its C section
SIGNATURES = {
    "tq_set_device": (_i, [_i]), "tq_device": (_i, []), "tq_stream": (_vp, []),
    "tq_dev_alloc": (_vp, [_sz, C.c_char_p]), "tq_dev_free": (None, [_vp]),
    "tq_h2d": (None, [_vp, _vp, _sz]), "tq_d2h": (None, [_vp, _vp, _sz]),
    "tq_dev_zero": (None, [_vp, _sz]), "tq_dev_fill": (None, [_vp, _i, _sz]),
    "tq_sync": (None, []), "tq_last_error": (_i, []),
    "tq_set_wait_limit_ms": (None, [_i]), "tq_clear_error": (None, []),
    "tq_dev_alloc_count": (C.c_ulonglong, []),
    "tq_host_alloc_pinned": (_vp, [_sz]), "tq_host_free_pinned": (None, [_vp]),
    "tq_h2d_async": (None, [_vp, _vp, _sz]), "tq_d2h_async": (None, [_vp, _vp, _sz]),
    "tq_d2h_overlapped": (C.c_int, [_vp, _vp, _sz]),
    "tq_h2d_overlapped": (C.c_int, [_vp, _vp, _sz]), "tq_stream_wait_copy": (None, [C.c_int]),
    "tq_d2d_async": (None, [_vp, _vp, _sz]),
    "tq_event_create": (_vp, []), "tq_event_destroy": (None, [_vp]),
    "tq_event_record": (None, [_vp]), "tq_event_elapsed_ms": (_f, [_vp, _vp]),
    "tq_graph_capture_begin": (_i, []), "tq_graph_capture_end": (_vp, []),
    "tq_graph_launch": (None, [_vp]), "tq_graph_destroy": (None, [_vp]),
    "qwn_x_w4_repack_weight": (_i, [_WP]), "qwn_x_w4_repack_weight_mode": (_i, [_WP, _i]),
    "qwn_x_quantize_act_s8": (None, [_vp, _i, _vp, _vp, _vp]),
    "qwn_x_prepare_gemv_act_s8": (None, [_vp, _i]),
    "qwn_x_silu_mul_quant": (None, [_vp, _vp, _vp, _i]),
    "qwn_x_rmsnorm_quant": (None, [_vp, _vp, _vp, _i, _f]),
    "qwn_x_prepare_gemv_act_s8_pertoken": (None, [_vp, _i]),
    "qwn_x_silu_mul_quant_pertoken": (None, [_vp, _vp, _vp, _i]),
    "qwn_x_gemv_w4a8": (_i, [_WP, _vp, _vp]),
    "qwn_x_gemv_w4a8_add": (_i, [_WP, _vp, _vp, _vp]),
    "qwn_x_gemv_w4a8_prepared": (_i, [_WP, _vp, _vp]),
    "qwn_x_gemv_w4a8_fused": (_i, [_WP, _vp, _vp, _vp]),
    "qwn_x_gemv_w4a8_fanout": (_i, [C.POINTER(_WP), C.POINTER(_vp), _i]),
    "qwn_x_w8_repack_weight": (_i, [_WP]),
    "qwn_x_gemv_w8a8": (_i, [_WP, _vp, _vp]), "qwn_x_gemv_w8a8_add": (_i, [_WP, _vp, _vp, _vp]),
    "qwn_x_gemv_w8a8_prepared": (_i, [_WP, _vp, _vp]),
    "qwn_x_gemm_w8a8": (_i, [_WP, _vp, _vp, _vp, _i]),
    "qwn_x_gemv_qmma": (_i, [_WP, _vp, _vp]),
    "qwn_x_gemv_qmma_add": (_i, [_WP, _vp, _vp, _vp]),
    "qwn_x_gemv_qmma_prepared": (_i, [_WP, _vp, _vp, _vp]),
    "qwn_x_silu_mul": (None, [_vp, _vp, _vp, _i]),
    "qwn_x_add_inplace": (None, [_vp, _vp, _i]),
    "qwn_x_quantize_act_chunk": (None, [_vp, _i, _i, _vp, _vp, _vp]),
    "qwn_x_gemm_w4a8": (_i, [_WP, _vp, _vp, _vp, _vp, _i, C.POINTER(_i), _i]),
    "qwn_x_w4_shard": (_i, [_WP, _WP, _i, _i, _i, C.POINTER(_i), _i]),
    "qwn_x_w4_shard_free": (None, [_WP]),
    "tq_profile_enable": (_i, [_i]), "tq_profile_report": (_i, [_vp, _i]),
    "qwn_choose_gemv_splits": (_i, [_i]), "qwn_choose_gemm_splits": (_i, [_i, _i, _i]),
    "qwn_choose_pertoken_splits": (_i, [_i, _i, _i, _i]),
    "qwn_x_gemm_w4a8_fanout": (_i, [C.POINTER(_WP), C.POINTER(_vp), _i, _vp, _vp, _vp, _i,
                                    C.POINTER(_i), _i]),
    "qwn_x_quantize_act_chunk_pertoken": (None, [_vp, _i, _i, _vp, _vp, _vp, _vp]),
    "qwn_x_gemm_w4a8_pertoken": (_i, [_WP, _vp, _vp, _vp, _vp, _i, _i]),
    "qwn_x_gemm_w4a8_fanout_pertoken": (_i, [C.POINTER(_WP), C.POINTER(_vp), _i, _vp, _vp, _vp, _i]),
    "qwn_x_quantize_act_chunk_s4": (None, [_vp, _i, _i, _vp, _vp, _vp]),
    "qwn_x_rmsnorm_chunk": (None, [_vp, _vp, _vp, _i, _i, C.c_float]),
    "qwn_x_gemm_w4a4": (_i, [_WP, _vp, _vp, _vp, _vp, _i]),
    "qwn_dbg_tile_dots_gemv": (_i, [_WP, _vp]),
    "qwn_dbg_tile_dots_gemm": (_i, [_WP, _vp, _i, _vp]),
    "qwn_dbg_prepared_act": (_i, [_i, _vp, _vp, _vp]),
    "qwn_gemv_bench": (_d, [_WP, _i]), "qwn_gemm_bench": (_d, [_WP, _i, _i]),
    "qwn_gemm_check": (_i, [_WP, _i, C.POINTER(_d), C.POINTER(_d)]),
    "qwn_specwave_check": (_i, [_WP]), "qwn_shard_check": (_i, [_WP, _i]),
    "qwn_shard_check_all": (_i, [C.POINTER(_WP), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), _i]),
    "qwn_w4_check": (_i, [_WP, _i, C.POINTER(_d), C.POINTER(_d)]),
    "qwn_tqf_read_qmma": (_i, [_vp, _sz, _i, _i, C.c_uint32, _WP, C.POINTER(_sz)]),
    "qwn_tqf_free_qmma": (None, [_WP]),
    "tq_selector_has": (_i, [C.c_char_p, C.c_char_p]), "tq_repack_tier_for": (_i, [C.c_char_p]),
    "qwn_repack_by_policy": (_i, [_WP, C.c_char_p]),
    "qwn_x_gemv_w4a8_static": (_i, [_WP, _vp, _vp]), "qwn_static_max_k": (_i, []),
    "qwn_tc_int8_peak": (_d, [_i]), "qwn_tc_int8_probe": (_d, [_i, _i, _i, _vp]),
    "tq_comm_unique_id": (_i, [_vp]), "tq_comm_init": (_i, [_vp, _i, _i]),
    "tq_comm_allgather": (_i, [_vp, _vp, _sz]),
    "tq_comm_allreduce_sum": (_i, [_vp, _vp, _sz]),
    "tq_comm_ipc_export": (_i, [_vp, _vp]), "tq_comm_ipc_open": (_vp, [_vp]),
    "tq_comm_ipc_close": (None, [_vp]),
    "tq_comm_gather_setup": (_i, [C.POINTER(_vp), C.POINTER(_vp), _i, _i]),
    "tq_comm_gather_wait": (_i, []),
    "qwn_x_gemm_w4a8_fanout_gathered": (_i, [C.POINTER(_WP), _i, _vp, _vp, _vp, _i,
                                         C.POINTER(_sz)]),
    "qwn_x_gemm_w4a8_fanout_fused": (_i, [C.POINTER(_WP), C.POINTER(_vp), _i, _vp, _i, _i]),
    "qwn_x_gemm_w4a8_fanout_gathered_fused": (_i, [C.POINTER(_WP), _i, _vp, _i, _i, C.POINTER(_sz)]),
    "tq_comm_sym_register": (_i, [_i, C.POINTER(_vp)]), "tq_comm_exchange_advance": (_i, []),
    "tq_comm_exchange_rewind": (_i, []), "tq_comm_exchange_sync": (_i, []),
    "qwn_x_gemm_w4a8_fanout_tp": (_i, [C.POINTER(_WP), _i, _vp, _vp, _vp, _vp, _i, C.POINTER(_i),
                                   C.POINTER(_vp), _i, C.POINTER(_sz), _sz]),
    "qwn_x_quantize_act_chunk_sync": (None, [_vp, _i, _i, _vp, _vp, _vp]),
    "qwn_x_quantize_act_chunk_pertoken_sync": (None, [_vp, _i, _i, _vp, _vp, _vp, _vp]),
    "qwn_x_rmsnorm_chunk_sync": (None, [_vp, _vp, _vp, _i, _i, C.c_float]),
    "qwn_w4_grid_probe": (_i, [_vp, _vp, _vp, _vp]),
    "qwn_x_rmsnorm_quant_chunk_pertoken": (None, [_vp, _vp, _vp, _i, _i, C.c_float, _vp, _vp, _vp, _vp, _i]),
    "qwn_x_silu_mul_quant_chunk_pertoken": (None, [_vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp]),
    "qwn_x_silu_mul_scatter": (_i, [_vp, _vp, _i, _i, _i, _sz, _sz]),
    "tq_comm_rank": (_i, []), "tq_comm_world": (_i, []), "tq_comm_destroy": (None, []),
}


def load() -> C.CDLL:
    """Load the CUDA library; raises if it is missing (there is no other path)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python knivesysl-xe_b200/build.py`; "
            "this package has no CPU or eager fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError = a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class DevBuf:
    """A device allocation owned through tq_dev_alloc/tq_dev_free."""

    def __init__(self, nbytes: int, what: str = "py"):
        self.lib = load()
        self.nbytes = int(nbytes)
        self.ptr = self.lib.tq_dev_alloc(self.nbytes, what.encode())

    @classmethod
    def from_numpy(cls, a: np.ndarray, what: str = "py") -> "DevBuf":
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes, what)
        b.lib.tq_h2d(b.ptr, a.ctypes.data, a.nbytes)
        return b

    def to_numpy(self, dtype, count: int | None = None) -> np.ndarray:
        dt = np.dtype(dtype)
        n = self.nbytes // dt.itemsize if count is None else count
        out = np.empty(n, dtype=dt)
        self.lib.tq_d2h(out.ctypes.data, self.ptr, out.nbytes)
        return out

    def fill(self, byte: int) -> None:
        self.lib.tq_dev_fill(self.ptr, byte, self.nbytes)

    def free(self) -> None:
        if self.ptr:
            self.lib.tq_dev_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PackedWeight:
    """A packed W4 record on the device, built from host codes + scales."""

    def __init__(self, codes: np.ndarray, scales: np.ndarray, M: int, K: int, k64: bool = False,
                 k16: bool = False):
        self.codes = DevBuf.from_numpy(np.ascontiguousarray(codes, dtype=np.uint8), "w4.codes")
        self.scales = DevBuf.from_numpy(np.ascontiguousarray(scales, dtype=np.uint16), "w4.scales")
        self.rec = TqWeight()
        self.rec.M, self.rec.K, self.rec.Mt, self.rec.Kt = M, K, M // 16, K // 32
        self.rec.d_s4, self.rec.d_s4_scale = self.codes.ptr, self.scales.ptr
        self.rec.s4_ready, self.rec.s4_k64, self.rec.s4_k16 = 1, int(k64), int(k16)

    @property
    def ref(self):
        return C.byref(self.rec)

    @property
    def weight_bytes(self) -> int:
        return self.codes.nbytes + self.scales.nbytes


def weight_array(ws):
    arr = (_WP * len(ws))(*[C.pointer(w.rec) for w in ws])
    return arr


def ptr_array(bufs):
    return (_vp * len(bufs))(*[b.ptr for b in bufs])
