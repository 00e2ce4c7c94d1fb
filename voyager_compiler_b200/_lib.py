"""ctypes binding of ``libvoyager_b200.so`` (the C ABI in ``include/voyager_b200.h``).

There is no fallback: if the shared library is missing or was built for another ABI version,
importing this module raises.  Build it with ``python voyager_compiler_b200/build.py``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvoyager_b200.so")
ABI_VERSION = 2

VQ_F32, VQ_BF16 = 0, 1
TABLE_NONE, TABLE_LUT16, TABLE_INT, TABLE_RUNS = 0, 1, 2, 3
SCALE_SCALAR, SCALE_ROWBLOCK, SCALE_STRIDED = 0, 1, 2


class VqTable(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("n_runs", C.c_int32),
        ("lut16", C.c_void_p), ("lut8", C.c_void_p),
        ("lo", C.c_float), ("hi", C.c_float),
        ("run_keys", C.c_void_p), ("run_vals", C.c_void_p), ("run_codes", C.c_void_p),
        ("nan_val", C.c_uint16), ("pinf_val", C.c_uint16), ("ninf_val", C.c_uint16),
        ("nan_code", C.c_uint8), ("pinf_code", C.c_uint8), ("ninf_code", C.c_uint8),
        ("nan_uniform", C.c_uint8), ("flat_tiny", C.c_uint8), ("reserved", C.c_uint8 * 5),
        ("levels2", C.c_void_p),
    ]


class VqChannelItem(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("channels", C.c_int64), ("length", C.c_int64), ("scale_in", C.c_void_p),
        ("amax_out", C.c_void_p), ("scale_out", C.c_void_p), ("values", C.c_void_p), ("codes", C.c_void_p),
        ("dequant", C.c_void_p),
    ]


class VqScaleLayout(C.Structure):
    _fields_ = [
        ("mode", C.c_int32), ("ndim", C.c_int32),
        ("rows", C.c_int64), ("K", C.c_int64), ("block", C.c_int64),
        ("size", C.c_int64 * 6), ("div", C.c_int64 * 6), ("stride", C.c_int64 * 6),
    ]


class VqExpTables(C.Structure):
    _fields_ = [("bump_at", C.c_void_p), ("scale_of", C.c_void_p)]


class VqMxExtras(C.Structure):
    _fields_ = [
        ("scale_f32", C.c_void_p), ("exp_e8", C.c_void_p), ("codes", C.c_void_p),
        ("code_bits", C.c_int32), ("dequant", C.c_void_p),
    ]


class VqMxItem(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("out_scale", C.c_void_p), ("out_codes", C.c_void_p), ("scale_f32", C.c_void_p),
        ("exp_e8", C.c_void_p), ("codes", C.c_void_p), ("dequant", C.c_void_p), ("n", C.c_int64),
    ]


class VoyagerB200Error(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python voyager_compiler_b200/build.py`). There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    lib.vq_version.restype = C.c_int
    if lib.vq_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {lib.vq_version()}, expected {ABI_VERSION}; rebuild it")
    lib.vq_last_error.restype = C.c_char_p
    lib.vq_launch_count.restype = C.c_uint64
    vp, i64, ci, dbl = C.c_void_p, C.c_int64, C.c_int, C.c_double
    T, L, E, X = C.POINTER(VqTable), C.POINTER(VqScaleLayout), C.POINTER(VqExpTables), C.POINTER(VqMxExtras)
    sigs = {
        "vq_selftest_fastdiv": [C.c_uint32, C.c_uint32],
        "vq_lut_map": [vp, ci, i64, T, vp, vp],
        "vq_quantize": [vp, ci, i64, vp, vp, L, T, vp, vp, ci, vp],
        "vq_dequantize": [vp, ci, i64, vp, vp, L, T, T, vp, vp],
        "vq_fake_quantize": [vp, ci, i64, vp, L, T, vp, vp],
        "vq_amax": [vp, ci, i64, i64, i64, vp, vp],
        "vq_filter_outlier": [vp, ci, i64, i64, i64, dbl, i64, C.c_int32, vp, vp, vp, vp, vp, C.c_size_t, vp],
        "vq_spmm_csr": [vp, vp, vp, vp, ci, i64, i64, i64, i64, i64, i64, vp, vp, vp],
        "vq_observer_update": [vp, vp, vp, ci, i64, dbl, ci, vp, vp],
        "vq_observer_step": [vp, ci, i64, i64, i64, vp, vp, vp, ci, dbl, ci, vp, vp],
        "vq_exp_histogram": [vp, ci, i64, E, vp, vp, C.c_size_t, vp],
        "vq_group_affine_fake_quantize": [vp, ci, i64, i64, i64, dbl, dbl, vp, vp, vp, vp, vp],
        "vq_outlier_split": [vp, ci, i64, vp, vp, vp, vp],
        "vq_outlier_merge": [vp, vp, ci, i64, vp, vp, vp],
        "vq_mx_scale": [vp, ci, i64, i64, i64, i64, dbl, ci, E, T, vp, vp],
        "vq_quantize_mx": [vp, ci, i64, i64, i64, i64, dbl, ci, E, T, T, vp, vp, X, vp],
        "vq_row_codebook": [vp, ci, i64, i64, vp, ci, ci, vp, vp, vp, C.c_size_t, vp],
        "vq_row_quantile": [vp, ci, i64, i64, ci, vp, vp],
        "vq_lcq_accumulate": [vp, ci, i64, i64, C.c_double, vp, i64, vp, ci, vp, vp, vp, vp],
        "vq_codebook_qmap": [vp, ci, vp, vp],
        "vq_gptq_block": [vp, i64, i64, i64, ci, vp, i64, vp, ci, C.c_double, vp, vp, vp, i64, vp, vp, vp],
        "vq_conv_patches": [vp, ci, i64, i64, i64, i64, i64, i64, i64, i64, ci, ci, ci, ci, ci, ci, ci, ci,
                            vp, i64, i64, i64, i64, i64, vp, i64, vp],
        "vq_conv2d_bf16": [vp, i64, i64, i64, i64, i64, i64, i64, vp, i64, i64, i64, i64, vp, i64, ci, ci, ci, ci, ci, ci, ci,
                           ci, ci, vp, vp, vp, vp],
        "vq_dequantize_packed": [vp, ci, vp, ci, vp, vp, i64, i64, vp, ci, vp],
        "vq_gemm_bf16_tn": [vp, vp, vp, vp, i64, i64, i64, vp, vp],
        "vq_slice_csr": [vp, vp, vp, ci, i64, i64, ci, i64, i64, i64, vp, vp, vp, vp, C.c_size_t, vp],
        "vq_gemm_bf16_tn_batched": [vp, vp, vp, i64, i64, i64, i64, ci, ci, vp, vp],
        "vq_gemm_f32_tn_batched": [vp, vp, vp, vp, i64, i64, i64, i64, ci, ci, vp, vp],
        "vq_dequantize_transpose": [vp, vp, i64, i64, i64, i64, i64, vp, vp],
        "vq_gemm_bf16_tn_scatter": [vp, vp, vp, C.POINTER(C.c_void_p), ci, i64, i64, i64, i64, i64, vp, vp],
        "vq_linear_mx": [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, vp],
        "vq_linear_mx_packed": [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, vp],
        "vq_quantize_mx_multi": [C.POINTER(VqMxItem), ci, ci, i64, dbl, ci, E, T, T, ci, vp, C.c_size_t, vp],
        "vq_channel_quantize_multi": [C.POINTER(VqChannelItem), ci, ci, dbl, T, vp, C.c_size_t, vp],
        "vq_quantize_mx_multi_static": [C.POINTER(VqMxItem), ci, ci, i64, dbl, ci, E, T, T, ci, vp],
        "vq_mx_plan_create": [C.POINTER(VqMxItem), ci, ci, i64, dbl, ci, E, T, T, ci, vp, C.c_size_t, vp,
                              C.POINTER(C.c_void_p)],
        "vq_mx_plan_run": [vp, vp],
        "vq_channel_plan_create": [C.POINTER(VqChannelItem), ci, ci, dbl, T, vp, C.c_size_t, vp, C.POINTER(C.c_void_p)],
        "vq_channel_plan_run": [vp, vp],
        "vq_channel_status": [],
    }
    lib.vq_channel_plan_destroy.argtypes = [vp]
    lib.vq_channel_plan_destroy.restype = None
    lib.vq_mx_plan_destroy.argtypes = [vp]
    lib.vq_mx_plan_destroy.restype = None
    lib.vq_quantize_mx_multi_static_max_items.argtypes = []
    lib.vq_quantize_mx_multi_static_max_items.restype = C.c_int
    lib.vq_quantize_mx_multi_workspace.argtypes = [ci]
    lib.vq_quantize_mx_multi_workspace.restype = C.c_size_t
    lib.vq_channel_quantize_multi_workspace.argtypes = [C.POINTER(VqChannelItem), ci]
    lib.vq_channel_quantize_multi_workspace.restype = C.c_size_t
    lib.vq_filter_outlier_workspace.argtypes = [i64, i64]
    lib.vq_filter_outlier_workspace.restype = C.c_size_t
    lib.vq_slice_csr_workspace.argtypes = [i64]
    lib.vq_slice_csr_workspace.restype = C.c_size_t
    lib.vq_conv2d_weight_columns.argtypes = [i64, ci, ci]
    lib.vq_conv2d_weight_columns.restype = i64
    lib.vq_row_codebook_workspace.argtypes = [i64, ci]
    lib.vq_row_codebook_workspace.restype = C.c_size_t
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int
    return lib


lib = _load()


def check(rc: int, what: str = "") -> None:
    """Raise on a non-zero status: AssertionError-free, always a VoyagerB200Error subclass of
    RuntimeError; unsupported argument combinations raise NotImplementedError."""
    if rc == 0:
        return
    msg = lib.vq_last_error().decode(errors="replace")
    if rc == -2:
        raise NotImplementedError(f"{what}: {msg}" if what else msg)
    if rc == -1:
        raise ValueError(f"{what}: {msg}" if what else msg)
    raise VoyagerB200Error(f"{what}: {msg} (status {rc})" if what else f"{msg} (status {rc})")


def launch_count() -> int:
    return int(lib.vq_launch_count())
