"""CPU oracle for the quantized-inference path (TEST INFRASTRUCTURE ONLY).

ctypes bindings over ``oracle/libquant_oracle.so`` (built from
``quant_oracle.c`` by ``oracle/Makefile``) with numpy arrays in and out, plus
``safetensors_oracle`` — a pure-Python restatement of the reference's
quantized-safetensors writer / validator.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package; the product library never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libquant_oracle.so")

OK, ERR_RANK, ERR_GRANULARITY, ERR_LENGTH = 0, 1, 2, 7

PER_TENSOR, PER_CHANNEL, GROUP, BLOCK = 0, 1, 2, 3


def build(force: bool = False) -> str:
    """Compile the C oracle in place (gcc, seconds)."""
    src = os.path.join(_HERE, "quant_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libquant_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        u64, u32, i32, vp = ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32, ctypes.c_void_p
        L.qo_bf16_to_f32.restype = ctypes.c_float
        L.qo_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.qo_f32_to_bf16.restype = ctypes.c_uint16
        L.qo_f32_to_bf16.argtypes = [ctypes.c_float]
        L.qo_f16_to_f32.restype = ctypes.c_float
        L.qo_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.qo_quant_range.restype = None
        L.qo_quant_range.argtypes = [u32, ctypes.POINTER(i32), ctypes.POINTER(i32)]
        L.qo_quantize_sym.restype = i32
        L.qo_quantize_sym.argtypes = [ctypes.c_float, ctypes.c_float, u32]
        L.qo_dequantize_sym.restype = ctypes.c_float
        L.qo_dequantize_sym.argtypes = [i32, ctypes.c_float]
        L.qo_int4_unpack.restype = i32
        L.qo_int4_unpack.argtypes = [u32, u32]
        L.qo_int4_pack.restype = u32
        L.qo_int4_pack.argtypes = [u32, u32, i32]
        L.qo_tile.restype = ctypes.c_int
        L.qo_tile.argtypes = [ctypes.c_int, u64, u64, u64, u64, u64, ctypes.POINTER(u64), ctypes.POINTER(u64)]
        L.qo_quantize_host.restype = ctypes.c_int
        L.qo_quantize_host.argtypes = [vp, u64, u64, u64, u32, u64, u64, vp, vp]
        L.qo_dequantize_host.restype = ctypes.c_int
        L.qo_dequantize_host.argtypes = [vp, u64, vp, u64, u64, u64, u32, u64, u64, vp]
        L.qo_linear_forward_f32.restype = ctypes.c_int
        L.qo_linear_forward_f32.argtypes = [vp, vp, vp, u64, u64, u64, ctypes.c_int, ctypes.c_int, vp]
        L.qo_linear_forward_f64.restype = ctypes.c_int
        L.qo_linear_forward_f64.argtypes = [vp, vp, vp, u64, u64, u64, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp]
        L.qo_qlinear_apply.restype = ctypes.c_int
        L.qo_qlinear_apply.argtypes = [vp, vp, u64, u64, u32, u64, u64, ctypes.c_int, vp, u64, vp, ctypes.c_int, vp, vp]
        L.qo_max_threads.restype = ctypes.c_int
        _lib = L
    return _lib


class OracleError(Exception):
    def __init__(self, code: int, what: str):
        super().__init__(what)
        self.code = code


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def div_ceil(a: int, b: int) -> int:
    return -(-a // b)


# -- scalar arithmetic (quanta-ir/src/dtype.rs) -----------------------------

def quant_range(bits: int):
    lo, hi = ctypes.c_int32(), ctypes.c_int32()
    lib().qo_quant_range(bits, ctypes.byref(lo), ctypes.byref(hi))
    return lo.value, hi.value


def quantize_sym(x: float, scale: float, bits: int) -> int:
    return lib().qo_quantize_sym(np.float32(x), np.float32(scale), bits)


def dequantize_sym(q: int, scale: float) -> np.float32:
    return np.float32(lib().qo_dequantize_sym(q, np.float32(scale)))


def int4_unpack(word: int, i: int) -> int:
    return lib().qo_int4_unpack(word & 0xFFFFFFFF, i)


def int4_pack(word: int, i: int, q: int) -> int:
    return lib().qo_int4_pack(word & 0xFFFFFFFF, i, q)


def f32_to_bf16(a) -> np.ndarray:
    """Vectorised dtype.rs:14-21 (round-to-nearest-even, NaN quieted) -> uint16 bits."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32)
    nan = np.isnan(a)
    bias = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    out = ((bits + bias) >> np.uint32(16)).astype(np.uint16)
    out[nan] = ((bits[nan] >> np.uint32(16)).astype(np.uint16)) | np.uint16(0x0040)
    return out


def bf16_to_f32(b) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


# -- Granularity::tile (quanta-array/src/quant.rs:109-144) ------------------

def tile(kind: int, rows: int, cols: int, axis: int = 0, size: int = 0, size2: int = 0):
    gr, gc = ctypes.c_uint64(), ctypes.c_uint64()
    rc = lib().qo_tile(kind, axis, size, size2, rows, cols, ctypes.byref(gr), ctypes.byref(gc))
    if rc != OK:
        raise OracleError(rc, "invalid quantization granularity")
    return gr.value, gc.value


# -- quantize_host / dequantize_host ---------------------------------------

def quantize_host(w, rows: int, cols: int, bits: int, gr: int, gc: int):
    """Returns (codes, scales): codes int8 [rows, cols] or uint32 [rows, ceil(cols/8)]."""
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    if rows == 0 or cols == 0:
        raise OracleError(ERR_RANK, "rank")
    if w.size != rows * cols:
        raise OracleError(ERR_LENGTH, f"expected {rows * cols}, got {w.size}")
    if gr <= 0 or gc <= 0 or gr > rows or gc > cols:
        raise OracleError(ERR_GRANULARITY, "granularity")
    tr, tc = div_ceil(rows, gr), div_ceil(cols, gc)
    scales = np.empty((tr, tc), dtype=np.float32)
    if bits == 8:
        codes = np.empty((rows, cols), dtype=np.int8)
    else:
        codes = np.empty((rows, div_ceil(cols, 8)), dtype=np.uint32)
    rc = lib().qo_quantize_host(_ptr(w), w.size, rows, cols, bits, gr, gc, _ptr(codes), _ptr(scales))
    if rc != OK:
        raise OracleError(rc, "quantize_host")
    return codes, scales


def dequantize_host(codes, scales, rows: int, cols: int, bits: int, gr: int, gc: int):
    codes = np.ascontiguousarray(codes)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    out = np.empty((max(rows, 0), max(cols, 0)), dtype=np.float32)
    rc = lib().qo_dequantize_host(_ptr(codes), codes.size, _ptr(scales), scales.size, rows, cols,
                                  bits, gr, gc, _ptr(out))
    if rc != OK:
        raise OracleError(rc, "dequantize_host")
    return out


# -- QuantizedLinear forward ------------------------------------------------

IN_OUT, OUT_IN = 0, 1


def linear_forward(x, wd, bias=None, layout: int = IN_OUT, threads: int = 1):
    """y = x @ wd (+ b) (layout IN_OUT) or x @ wd^T (OUT_IN); sequential-k f32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    wd = np.ascontiguousarray(wd, dtype=np.float32)
    m, k = x.shape
    in_dim, out_dim = (wd.shape if layout == IN_OUT else wd.shape[::-1])
    assert k == in_dim
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    y = np.empty((m, out_dim), dtype=np.float32)
    lib().qo_linear_forward_f32(_ptr(x), _ptr(wd), _ptr(bias), m, in_dim, out_dim, layout, threads, _ptr(y))
    return y


def linear_forward_f64(x, wd, bias=None, layout: int = IN_OUT, stage_w: bool = False, threads: int = 1):
    x = np.ascontiguousarray(x, dtype=np.float32)
    wd = np.ascontiguousarray(wd, dtype=np.float32)
    m, k = x.shape
    in_dim, out_dim = (wd.shape if layout == IN_OUT else wd.shape[::-1])
    assert k == in_dim
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    y = np.empty((m, out_dim), dtype=np.float64)
    lib().qo_linear_forward_f64(_ptr(x), _ptr(wd), _ptr(bias), m, in_dim, out_dim, layout,
                                int(stage_w), threads, _ptr(y))
    return y


def qlinear_apply(codes, scales, rows, cols, bits, gr, gc, layout, x, bias=None, threads: int = 1,
                  scratch=None):
    """dequantize + GEMM + bias, the whole QuantizedLinear::apply on the host."""
    codes = np.ascontiguousarray(codes)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    out_dim = cols if layout == IN_OUT else rows
    if scratch is None:
        scratch = np.empty(rows * cols, dtype=np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    y = np.empty((m, out_dim), dtype=np.float32)
    lib().qo_qlinear_apply(_ptr(codes), _ptr(scales), rows, cols, bits, gr, gc, layout, _ptr(x), m,
                           _ptr(bias), threads, _ptr(scratch), _ptr(y))
    return y


def max_threads() -> int:
    """Host threads the timed baselines use: every core this process may run on (launchers such as
    torchrun pin OMP_NUM_THREADS to 1; the thread count is passed to the library explicitly)."""
    if lib().qo_max_threads() <= 0:
        return 1
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)
