"""Host-side mirror of ``quanta_blas``'s quantized entries (crates/sci/quanta-blas/src/mixed_quant.rs:22-147):
``gemm_quant`` / ``gemv_quant`` over int8 codes (one per int32 word) and ``gemm_quant4`` / ``gemv_quant4`` over
int4 codes packed eight per word, integer codes for BOTH operands with per-tensor symmetric scales, C in f32.
The tensors are the reference's ``Field``s: flat device buffers; the ``Gpu`` argument is the tensors' device."""
from __future__ import annotations

import ctypes
from enum import Enum

import torch

from . import _lib as L
from .quant import QuantError, _require_cuda, _stream, check


class GemmQuantType(Enum):
    """mixed_quant.rs:22-31."""
    Q8Symmetric = 0
    Q4Symmetric = 1


def _field(t: torch.Tensor, dtype: torch.dtype, length: int, who: str, what: str) -> ctypes.c_void_p:
    _require_cuda(t, f"{who}: {what}")
    if t.dtype != dtype or not t.is_contiguous():
        raise QuantError(L.ERR_INVALID_PARAM, f"{who}: {what} must be a contiguous {dtype} buffer")
    if t.numel() != length:
        raise QuantError(L.ERR_LENGTH, f"{who}: {what} holds {t.numel()} words, the shape needs {length}")
    return ctypes.c_void_p(t.data_ptr())


def _dims(who: str, *dims: int):
    for d in dims:
        if d < 0 or d > 0xFFFFFFFF:
            raise QuantError(L.ERR_INVALID_PARAM, f"{who}: dimension {d} is not a u32")


def gemm_quant(qty: GemmQuantType, m: int, n: int, k: int, alpha: float, a_scale: float, b_scale: float,
               a: torch.Tensor, b: torch.Tensor, beta: float, c: torch.Tensor) -> None:
    """``C <- alpha * (a_scale * A) * (b_scale * B) + beta * C`` (mixed_quant.rs:47-81): A ``m x k`` and B ``k x n``
    row-major int8 codes in int32 words, C ``m x n`` f32, read and overwritten.  Asynchronous on the current stream."""
    who = "gemm_quant"
    _dims(who, m, n, k)
    ap, bp = _field(a, torch.int32, m * k, who, "A"), _field(b, torch.int32, k * n, who, "B")
    cp = _field(c, torch.float32, m * n, who, "C")
    check(L.load().qb200_gemm_quant(qty.value, m, n, k, alpha, a_scale, b_scale, ap, bp, beta, cp, _stream(c)))


def gemm_quant4(qty: GemmQuantType, m: int, n: int, k: int, alpha: float, a_scale: float, b_scale: float,
                a: torch.Tensor, b: torch.Tensor, beta: float, c: torch.Tensor) -> None:
    """The int4 twin (mixed_quant.rs:104-127): A and B are ``ceil(m*k/8)`` / ``ceil(k*n/8)`` packed words (int32
    tensors holding the u32 bit patterns; element i in nibble ``i % 8`` of word ``i // 8``)."""
    who = "gemm_quant4"
    _dims(who, m, n, k)
    ap, bp = _field(a, torch.int32, -(-(m * k) // 8), who, "A"), _field(b, torch.int32, -(-(k * n) // 8), who, "B")
    cp = _field(c, torch.float32, m * n, who, "C")
    check(L.load().qb200_gemm_quant4(qty.value, m, n, k, alpha, a_scale, b_scale, ap, bp, beta, cp, _stream(c)))


def gemv_quant(qty: GemmQuantType, m: int, n: int, alpha: float, a_scale: float, x_scale: float, a: torch.Tensor,
               x: torch.Tensor, beta: float, y: torch.Tensor) -> None:
    """``y <- alpha * (a_scale * A) * (x_scale * x) + beta * y``, A ``m x n`` (mixed_quant.rs:83-100)."""
    who = "gemv_quant"
    _dims(who, m, n)
    ap, xp = _field(a, torch.int32, m * n, who, "A"), _field(x, torch.int32, n, who, "x")
    yp = _field(y, torch.float32, m, who, "y")
    check(L.load().qb200_gemv_quant(qty.value, m, n, alpha, a_scale, x_scale, ap, xp, beta, yp, _stream(y)))


def gemv_quant4(qty: GemmQuantType, m: int, n: int, alpha: float, a_scale: float, x_scale: float, a: torch.Tensor,
                x: torch.Tensor, beta: float, y: torch.Tensor) -> None:
    """mixed_quant.rs:129-147."""
    who = "gemv_quant4"
    _dims(who, m, n)
    ap, xp = _field(a, torch.int32, -(-(m * n) // 8), who, "A"), _field(x, torch.int32, -(-n // 8), who, "x")
    yp = _field(y, torch.float32, m, who, "y")
    check(L.load().qb200_gemv_quant4(qty.value, m, n, alpha, a_scale, x_scale, ap, xp, beta, yp, _stream(y)))


def check_stream(t: torch.Tensor) -> None:
    """Waits for the current stream of ``t``'s device and raises what the kernels recorded on it: an int8 code
    outside [-128, 127] (InvalidParam) or a bounded wait that ran out (Timeout)."""
    check(L.load().qb200_gemm_quant_check(_stream(t)))
