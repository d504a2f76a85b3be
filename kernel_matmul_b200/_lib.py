"""ctypes binding of ``libkm_b200.so`` (declarations in ``include/km_b200.h``).

There is no fallback: if the library is missing, importing this module raises, and every op
of the package raises with it.
"""
from __future__ import annotations

import ctypes
import os

KM_MAX_BATCH_DIMS = 4
KM_MAX_PARAMS = 4
KM_OK = 0

KERNEL_TYPES = {"rbf": 0, "spectral": 1, "locally_periodic": 2}

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkm_b200.so")


class KmBatch(ctypes.Structure):
    _fields_ = [("ndim", ctypes.c_int32), ("size", ctypes.c_int64 * KM_MAX_BATCH_DIMS)]


class KmView(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("batch_stride", ctypes.c_int64 * KM_MAX_BATCH_DIMS),
        ("stride", ctypes.c_int64 * 2),
    ]


class KmError(RuntimeError):
    """An entry point of libkm_b200 returned a non-zero status."""


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python kernel_matmul_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
    bp, wp = ctypes.POINTER(KmBatch), ctypes.POINTER(KmView)
    lib.km_last_error.restype = ctypes.c_char_p
    lib.km_last_error.argtypes = []
    lib.km_version.restype = ctypes.c_char_p
    lib.km_version.argtypes = []
    lib.km_num_params.restype = ctypes.c_int
    lib.km_num_params.argtypes = [ctypes.c_int]
    lib.km_matmul_f32.restype = ctypes.c_int
    lib.km_matmul_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, vp]
    lib.km_matmul_rows_f32.restype = ctypes.c_int
    lib.km_matmul_rows_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, i64, i64, i32, vp]
    lib.km_sum_phases_workspace_bytes.restype = sz
    lib.km_sum_phases_workspace_bytes.argtypes = [bp, i64, i64]
    lib.km_sum_phases_prepare_f32.restype = ctypes.c_int
    lib.km_sum_phases_prepare_f32.argtypes = [bp, i64, i64, wp, wp, wp, i64, i64, i64, i64, vp, sz, vp]
    lib.km_matmul_rows_phases_f32.restype = ctypes.c_int
    lib.km_matmul_rows_phases_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, i64, i64, vp, sz, vp]
    lib.km_matmul_tc_workspace_bytes.restype = sz
    lib.km_matmul_tc_workspace_bytes.argtypes = [bp, i64, i64, wp]
    lib.km_matmul_tc_f32.restype = ctypes.c_int
    lib.km_matmul_tc_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, vp, sz, vp]
    lib.km_matmul_tc_rows_f32.restype = ctypes.c_int
    lib.km_matmul_tc_rows_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, i64, i64, vp, sz, vp]
    lib.km_workspace_status.restype = ctypes.c_int
    lib.km_workspace_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    lib.km_grad_workspace_bytes.restype = sz
    lib.km_grad_workspace_bytes.argtypes = [ctypes.c_int, bp, i64]
    lib.km_bilinear_derivative_f32.restype = ctypes.c_int
    lib.km_bilinear_derivative_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, wp, vp, sz, vp]
    lib.km_matmul_bwd_f32.restype = ctypes.c_int
    lib.km_matmul_bwd_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, wp, vp, sz, vp]
    lib.km_grad_tc_workspace_bytes.restype = sz
    lib.km_grad_tc_workspace_bytes.argtypes = [bp, i64, i64, i64, wp]
    lib.km_bilinear_derivative_tc_f32.restype = ctypes.c_int
    lib.km_bilinear_derivative_tc_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, wp, vp, sz, vp]
    lib.km_matmul_bwd_tc_f32.restype = ctypes.c_int
    lib.km_matmul_bwd_tc_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, wp, vp, sz, vp]
    lib.km_bilinear_derivative_static_f32.restype = ctypes.c_int
    lib.km_bilinear_derivative_static_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, wp, wp, wp, vp]
    lib.km_dense_f32.restype = ctypes.c_int
    lib.km_dense_f32.argtypes = [ctypes.c_int, bp, i64, i64, wp, wp, wp, wp, wp, wp, vp]
    lib.km_dense_bwd_f32.restype = ctypes.c_int
    lib.km_dense_bwd_f32.argtypes = [ctypes.c_int, bp, i64, i64, wp, wp, wp, wp, wp, wp, wp, vp, sz, vp]
    pp = ctypes.POINTER(ctypes.c_void_p)
    lib.km_index_f32.restype = ctypes.c_int
    lib.km_index_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, pp, vp, vp, vp, vp]
    lib.km_index_bwd_workspace_bytes.restype = sz
    lib.km_index_bwd_workspace_bytes.argtypes = [ctypes.c_int, bp]
    lib.km_index_bwd_f32.restype = ctypes.c_int
    lib.km_index_bwd_f32.argtypes = [ctypes.c_int, bp, i64, i64, i64, wp, wp, wp, wp, wp, pp, vp, vp, vp, wp, vp, sz, vp]
    lib.km_make_ranges_f32.restype = ctypes.c_int
    lib.km_make_ranges_f32.argtypes = [i64, i64, i64, vp, vp, ctypes.c_float, i32, i32, vp, vp, vp, vp]
    lib.km_make_ranges_symmetric_f32.restype = ctypes.c_int
    lib.km_make_ranges_symmetric_f32.argtypes = [i64, i64, vp, ctypes.c_float, i32, vp, vp, vp, vp]
    lib.km_make_ranges_symmetric_cutoffs_f32.restype = ctypes.c_int
    lib.km_make_ranges_symmetric_cutoffs_f32.argtypes = [i64, i64, vp, i64, vp, i32, vp, vp, vp, vp]
    lib.km_transpose_ranges_i32.restype = ctypes.c_int
    lib.km_transpose_ranges_i32.argtypes = [i64, i64, vp, vp, i64, i64, i32, vp, vp, vp]
    lib.km_count_entries.restype = ctypes.c_int
    lib.km_count_entries.argtypes = [bp, i64, i64, wp, wp, vp, vp]
    lib.km_probe_fp32_peak.restype = ctypes.c_int
    lib.km_probe_fp32_peak.argtypes = [i64, vp, ctypes.POINTER(ctypes.c_double), vp]
    lib.km_probe_sfu_peak.restype = ctypes.c_int
    lib.km_probe_sfu_peak.argtypes = [i64, vp, ctypes.POINTER(ctypes.c_double), vp]
    f32 = ctypes.c_float
    lib.km_cg_block_dots_f32.restype = ctypes.c_int
    lib.km_cg_block_dots_f32.argtypes = [i64, vp, vp, i64, i64, vp, vp]
    lib.km_cg_q_dots_f32.restype = ctypes.c_int
    lib.km_cg_q_dots_f32.argtypes = [i64, vp, vp, f32, i64, i64, vp, vp, i64, vp, i64, vp]
    lib.km_cg_segment_sums_f32.restype = ctypes.c_int
    lib.km_cg_segment_sums_f32.argtypes = [i64, vp, i64, i64, vp, vp]
    lib.km_cg_init_scalars_f32.restype = ctypes.c_int
    lib.km_cg_init_scalars_f32.argtypes = [i64, vp, i64, i32, i32, vp, vp, vp]
    lib.km_cg_update_xr_f32.restype = ctypes.c_int
    lib.km_cg_update_xr_f32.argtypes = [i64, vp, vp, vp, vp, vp, i64, vp, i64, i64, i64, i64, i64, vp, i64, i32, i32, vp, vp, vp, vp]
    lib.km_cg_update_p_f32.restype = ctypes.c_int
    lib.km_cg_update_p_f32.argtypes = [i64, vp, vp, i64, i64, vp, i64, i32, i32, vp, vp, vp, vp, vp, vp]
    lib.km_selftest_bounded_wait.restype = ctypes.c_int
    lib.km_selftest_bounded_wait.argtypes = [i64, vp, vp]
    lib.km_selftest_set_wait_polls.restype = ctypes.c_int
    lib.km_selftest_set_wait_polls.argtypes = [i64]
    return lib


lib = _load()

EXPORTED = [
    "km_last_error", "km_version", "km_num_params", "km_matmul_f32", "km_matmul_rows_f32", "km_matmul_tc_workspace_bytes", "km_matmul_tc_f32", "km_matmul_tc_rows_f32",
    "km_workspace_status", "km_grad_workspace_bytes", "km_grad_tc_workspace_bytes", "km_bilinear_derivative_tc_f32",
    "km_matmul_bwd_tc_f32",
    "km_bilinear_derivative_f32", "km_bilinear_derivative_static_f32", "km_matmul_bwd_f32", "km_dense_f32", "km_dense_bwd_f32",
    "km_index_f32", "km_index_bwd_workspace_bytes", "km_index_bwd_f32", "km_make_ranges_f32",
    "km_make_ranges_symmetric_f32", "km_make_ranges_symmetric_cutoffs_f32", "km_transpose_ranges_i32", "km_count_entries",
    "km_probe_fp32_peak", "km_probe_sfu_peak", "km_selftest_bounded_wait", "km_selftest_set_wait_polls",
    "km_cg_block_dots_f32", "km_cg_q_dots_f32", "km_cg_segment_sums_f32", "km_cg_init_scalars_f32", "km_cg_update_xr_f32",
    "km_cg_update_p_f32", "km_sum_phases_workspace_bytes", "km_sum_phases_prepare_f32", "km_matmul_rows_phases_f32",
]


def check(status: int) -> None:
    if status != KM_OK:
        raise KmError(f"[km status {status}] {lib.km_last_error().decode()}")
