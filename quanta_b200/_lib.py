"""ctypes loader for libqb200.so (the C ABI declared in include/qb200.h).

The library is the product: there is no Python or CPU fallback.  If the shared
object is missing it is built in place with nvcc; if that is impossible the
import fails loudly.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

u64, u32, i32, vp, cp = ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_char_p
P = ctypes.POINTER

OK, ERR_RANK, ERR_GRANULARITY, ERR_GRID, ERR_FORMAT, ERR_NOT_SUPPORTED, ERR_SCALE, ERR_LENGTH, \
    ERR_INVALID_PARAM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT = range(12)

PER_TENSOR, PER_CHANNEL, GROUP, BLOCK = 0, 1, 2, 3
IN_OUT, OUT_IN = 0, 1
F32, BF16, F16 = 0, 1, 2
TP_COLUMN, TP_ROW = 0, 1


class StItem(ctypes.Structure):
    _fields_ = [
        ("name", cp), ("quantized", i32), ("dtype", cp), ("ndim", u32), ("shape", P(u64)),
        ("data_offset", u64), ("data_len", u64), ("bits", u32), ("gr", u64), ("gc", u64),
        ("scales_offset", u64), ("scales_len", u64), ("gran_kind", i32), ("gran_axis", u64),
        ("gran_size", u64), ("gran_size2", u64),
    ]


# name -> (restype, argtypes); mirrors include/qb200.h one to one
SIGNATURES = {
    "qb200_version": (cp, []),
    "qb200_last_error": (ctypes.c_size_t, [ctypes.c_char_p, ctypes.c_size_t]),
    "qb200_device_count": (i32, []),
    "qb200_tile": (i32, [i32, u64, u64, u64, u64, u64, P(u64), P(u64)]),
    "qb200_granularity_from_grid": (i32, [u64, u64, u64, u64, i32, P(i32), P(u64), P(u64), P(u64)]),
    "qb200_codes_bytes": (i32, [u64, u64, u32, P(u64)]),
    "qb200_scales_count": (i32, [u64, u64, u64, u64, P(u64), P(u64)]),
    "qb200_check_parts": (i32, [u64, u64, u64, u64, u64, u64, u32, u64, u64]),
    "qb200_quantize": (i32, [vp, i32, u64, u64, u32, u64, u64, vp, vp, vp]),
    "qb200_dequantize": (i32, [vp, vp, u64, u64, u32, u64, u64, vp, vp]),
    "qb200_qlinear_create": (i32, [vp, vp, u64, u64, u32, u64, u64, i32, vp, u64, P(vp)]),
    "qb200_qlinear_destroy": (None, [vp]),
    "qb200_qlinear_in_dim": (u64, [vp]),
    "qb200_qlinear_out_dim": (u64, [vp]),
    "qb200_qlinear_forward": (i32, [vp, vp, i32, u64, vp, i32, vp]),
    "qb200_qlinear_forward_static": (i32, [vp, vp, i32, u64, vp, i32, vp]),
    "qb200_qlinear_forward_many": (i32, [P(vp), u32, P(vp), i32, u64, P(vp), i32, vp]),
    "qb200_qlinear_forward_many_host": (i32, [P(vp), u32, P(vp), i32, u64, P(vp), i32]),
    "qb200_add_rmsnorm": (i32, [vp, vp, u32, vp, u64, u64, ctypes.c_float, vp, vp]),
    "qb200_rope_append": (i32, [vp, vp, vp, vp, vp, u32, u32, u32, vp, vp, vp, u32, u32, vp]),
    "qb200_sdpa_decode_scratch_floats": (u64, [u32, u32, u32]),
    "qb200_sdpa_decode": (i32, [vp, vp, vp, u32, u32, u32, u32, u32, ctypes.c_float, vp, vp, vp]),
    "qb200_swiglu_sliced": (i32, [vp, vp, u64, u64, P(u32), u32, u32, vp, vp]),
    "qb200_sum_arrays": (i32, [vp, u32, u64, vp, vp]),
    "qb200_peer_alloc": (i32, [u64, P(vp), ctypes.c_char_p]),
    "qb200_peer_open": (i32, [ctypes.c_char_p, P(vp)]),
    "qb200_peer_close": (i32, [vp]),
    "qb200_peer_free": (i32, [vp]),
    "qb200_qlinear_forward_many_gather": (i32, [P(vp), u32, P(vp), i32, u64, P(vp), i32, P(vp), P(vp), u32, u32, vp]),
    "qb200_peer_signal_wait": (i32, [P(vp), u32, u32, vp, vp]),
    "qb200_qlinear_forward_many_push": (i32, [P(vp), u32, P(vp), i32, u64, P(vp), P(vp), u32, u32, vp, u64, vp]),
    "qb200_add_rmsnorm_pushed": (i32, [vp, vp, u32, vp, vp, u64, u64, ctypes.c_float, vp, vp, vp]),
    "qb200_gather_pushed": (i32, [vp, u32, u64, u32, u64, vp, vp, u64, vp, vp]),
    "qb200_peer_set_spin_limit": (i32, [u32]),
    "qb200_qlinear_check": (i32, [vp, vp]),
    "qb200_shard_rows": (i32, [u64, u64, u32, u32, P(u64), P(u64)]),
    "qb200_shard_cols": (i32, [u64, u64, u32, u32, u32, P(u64), P(u64)]),
    "qb200_tp_unique_id": (i32, [ctypes.c_char_p]),
    "qb200_tp_create": (i32, [u32, u32, ctypes.c_char_p, P(vp)]),
    "qb200_tp_destroy": (None, [vp]),
    "qb200_tp_rank": (u32, [vp]),
    "qb200_tp_world": (u32, [vp]),
    "qb200_qlinear_forward_tp": (i32, [vp, vp, i32, u64, u64, vp, i32, u64, vp, i32, vp]),
    "qb200_tp_status": (i32, [vp, vp, vp]),
    "qb200_gemm_quant": (i32, [i32, u32, u32, u32, ctypes.c_float, ctypes.c_float, ctypes.c_float, vp, vp, ctypes.c_float, vp, vp]),
    "qb200_gemm_quant4": (i32, [i32, u32, u32, u32, ctypes.c_float, ctypes.c_float, ctypes.c_float, vp, vp, ctypes.c_float, vp, vp]),
    "qb200_gemv_quant": (i32, [i32, u32, u32, ctypes.c_float, ctypes.c_float, ctypes.c_float, vp, vp, ctypes.c_float, vp, vp]),
    "qb200_gemv_quant4": (i32, [i32, u32, u32, ctypes.c_float, ctypes.c_float, ctypes.c_float, vp, vp, ctypes.c_float, vp, vp]),
    "qb200_gemm_quant_check": (i32, [vp]),
    "qb200_qlinear_forward_host": (i32, [vp, vp, i32, u64, vp, i32]),
    "qb200_qlinear_last_kernel": (cp, [vp]),
    "qb200_st_validate": (i32, [vp, u64, i32, P(vp)]),
    "qb200_st_free": (None, [vp]),
    "qb200_st_num_items": (u64, [vp]),
    "qb200_st_item_at": (i32, [vp, u64, P(StItem)]),
    "qb200_st_num_metadata": (u64, [vp]),
    "qb200_st_metadata_at": (i32, [vp, u64, P(cp), P(cp)]),
    "qb200_st_plain_to_f32": (i32, [vp, u64, vp, u64]),
    "qb200_st_writer_create": (i32, [P(vp)]),
    "qb200_st_writer_free": (None, [vp]),
    "qb200_st_writer_set_has_metadata": (i32, [vp, i32]),
    "qb200_st_writer_add_metadata": (i32, [vp, cp, cp]),
    "qb200_st_writer_add_f32": (i32, [vp, cp, P(u64), u32, vp]),
    "qb200_st_writer_add_quantized": (i32, [vp, cp, u32, u64, u64, u64, u64, vp, vp]),
    "qb200_st_writer_finish": (i32, [vp, P(vp), P(u64)]),
    "qb200_st_parse_quant_meta": (i32, [cp, cp, P(u32), P(u64), P(u64), P(u64), P(u64)]),
}

_lib = None


def lib_path() -> str:
    return _build.LIB


def load() -> ctypes.CDLL:
    """Loads (building first if stale or absent) the native library.  Raises on failure."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if not os.path.exists(path) or os.environ.get("QB200_REBUILD"):
        _build.build(force=bool(os.environ.get("QB200_REBUILD")))
    try:
        L = ctypes.CDLL(path)
    except OSError as e:  # pragma: no cover - loud failure is the contract
        raise ImportError(f"quanta_b200: the native library {path} could not be loaded ({e}); "
                          "there is no fallback implementation") from e
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def last_error() -> str:
    L = load()
    n = L.qb200_last_error(None, 0)
    buf = ctypes.create_string_buffer(n + 1)
    L.qb200_last_error(buf, n + 1)
    return buf.value.decode("utf-8", "replace")
