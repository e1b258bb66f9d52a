"""Array-level mirror of ``quanta::sci::quant`` over the qb200 C ABI.

Same names and argument meaning as the reference's
``crates/sci/quanta-array/src/quant.rs``: ``QuantDtype``, ``Granularity``,
``QuantizedMatrix`` (``quantize`` / ``from_parts`` / ``dequantize`` /
accessors) and ``QuantError``.  torch tensors stand in for the reference's
device ``Array``: they own the HBM buffers and supply the CUDA stream; every
computation is a kernel of libqb200.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from enum import Enum

import torch

from . import _lib as L


class QuantError(Exception):
    """Mirror of ``ArrayError`` for this path.  ``kind`` names the reference arm:
    Rank / Granularity / Grid / Format / NotSupported / Scale (QuantError, quant.rs:210-233),
    LengthMismatch (ArrayError), InvalidParam (QuantaError::invalid_param), Cuda, Nccl, Timeout."""

    KINDS = {L.ERR_RANK: "Rank", L.ERR_GRANULARITY: "Granularity", L.ERR_GRID: "Grid", L.ERR_FORMAT: "Format",
             L.ERR_NOT_SUPPORTED: "NotSupported", L.ERR_SCALE: "Scale", L.ERR_LENGTH: "LengthMismatch",
             L.ERR_INVALID_PARAM: "InvalidParam", L.ERR_CUDA: "Cuda", L.ERR_NCCL: "Nccl", L.ERR_TIMEOUT: "Timeout"}

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code
        self.kind = self.KINDS.get(code, "Unknown")


def check(status: int) -> None:
    if status != L.OK:
        raise QuantError(status, L.last_error())


class QuantDtype(Enum):
    """quant.rs:59-87."""
    Int8 = 8
    Int4 = 4

    def bits(self) -> int:
        return self.value


@dataclass(frozen=True)
class Granularity:
    """quant.rs:94-144.  Build with PerTensor() / PerChannel(axis) / Group(axis, size) /
    Block(rows, cols) (the additive 2-D block arm)."""
    kind: int
    axis: int = 0
    size: int = 0
    size2: int = 0

    def tile(self, rows: int, cols: int):
        gr, gc = L.u64(), L.u64()
        check(L.load().qb200_tile(self.kind, self.axis, self.size, self.size2, rows, cols,
                                  ctypes.byref(gr), ctypes.byref(gc)))
        return gr.value, gc.value

    def __repr__(self):
        if self.kind == L.PER_TENSOR:
            return "PerTensor"
        if self.kind == L.PER_CHANNEL:
            return f"PerChannel {{ axis: {self.axis} }}"
        if self.kind == L.GROUP:
            return f"Group {{ axis: {self.axis}, size: {self.size} }}"
        return f"Block {{ rows: {self.size}, cols: {self.size2} }}"


def PerTensor() -> Granularity:
    return Granularity(L.PER_TENSOR)


def PerChannel(axis: int) -> Granularity:
    return Granularity(L.PER_CHANNEL, axis=axis)


def Group(axis: int, size: int) -> Granularity:
    return Granularity(L.GROUP, axis=axis, size=size)


def Block(rows: int, cols: int) -> Granularity:
    return Granularity(L.BLOCK, size=rows, size2=cols)


def granularity_from_grid(rows, cols, gr, gc, allow_block=False) -> Granularity:
    kind, axis, size, size2 = L.i32(), L.u64(), L.u64(), L.u64()
    check(L.load().qb200_granularity_from_grid(rows, cols, gr, gc, int(allow_block), ctypes.byref(kind),
                                               ctypes.byref(axis), ctypes.byref(size), ctypes.byref(size2)))
    return Granularity(kind.value, axis.value, size.value, size2.value)


_SRC = {torch.float32: L.F32, torch.bfloat16: L.BF16, torch.float16: L.F16}


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise QuantError(L.ERR_CUDA, f"{what} must live on a CUDA device (this library has no CPU path)")


class QuantizedMatrix:
    """quant.rs:452-637 — integer codes + the f32 scale grid, both resident in HBM.

    codes: torch.int8 ``[R, C]`` or torch.int32 ``[R, ceil(C/8)]`` (the packed u32 words,
    low nibble first); scales: torch.float32 ``[ceil(R/gr), ceil(C/gc)]``."""

    def __init__(self, codes, scales, rows, cols, gr, gc, dtype: QuantDtype, granularity: Granularity):
        self._codes, self._scales = codes, scales
        self._rows, self._cols, self._gr, self._gc = rows, cols, gr, gc
        self._dtype, self._granularity = dtype, granularity

    @staticmethod
    def quantize(a: torch.Tensor, dtype: QuantDtype, granularity: Granularity) -> "QuantizedMatrix":
        """quant.rs:480-513: max-abs per-tile scales + round-ties-even codes — one device pass."""
        if a.dim() != 2 or a.shape[0] == 0 or a.shape[1] == 0:
            raise QuantError(L.ERR_RANK, "quantized leaves must be rank-2 with nonzero extents, got shape "
                             f"{list(a.shape)} (reshape rank-2 views before quantizing)")
        rows, cols = a.shape
        gr, gc = granularity.tile(rows, cols)
        _require_cuda(a, "the weight array")
        if a.dtype not in _SRC:
            raise QuantError(L.ERR_INVALID_PARAM, f"quantize: source dtype {a.dtype} is not f32 / bf16 / f16")
        a = a.contiguous()
        tr, tc = -(-rows // gr), -(-cols // gc)
        scales = torch.empty((tr, tc), dtype=torch.float32, device=a.device)
        if dtype is QuantDtype.Int8:
            codes = torch.empty((rows, cols), dtype=torch.int8, device=a.device)
        else:
            codes = torch.empty((rows, -(-cols // 8)), dtype=torch.int32, device=a.device)
        with torch.cuda.device(a.device):
            check(L.load().qb200_quantize(a.data_ptr(), _SRC[a.dtype], rows, cols, dtype.bits(), gr, gc,
                                          codes.data_ptr(), scales.data_ptr(), _stream(a)))
        return QuantizedMatrix(codes, scales, rows, cols, gr, gc, dtype, granularity)

    @staticmethod
    def from_parts(codes: torch.Tensor, shape, scales: torch.Tensor, granularity: Granularity) -> "QuantizedMatrix":
        """quant.rs:521-568 — assemble from already-resident parts with total validation."""
        rows, cols = shape
        if codes.dtype == torch.int8:
            dtype = QuantDtype.Int8
        elif codes.dtype in (torch.int32, torch.uint32):
            dtype = QuantDtype.Int4
        else:
            raise QuantError(L.ERR_INVALID_PARAM, f"codes dtype {codes.dtype} is neither int8 nor packed u32")
        if rows == 0 or cols == 0:
            check(L.load().qb200_codes_bytes(rows, cols, dtype.bits(), ctypes.byref(L.u64())))
        gr, gc = granularity.tile(rows, cols)
        cs = list(codes.shape) + [0, 0]
        ss = list(scales.shape) + [0, 0]
        if codes.dim() != 2 or scales.dim() != 2:
            cs, ss = [0, 0], [0, 0]
        check(L.load().qb200_check_parts(cs[0], cs[1], ss[0], ss[1], rows, cols, dtype.bits(), gr, gc))
        if scales.dtype != torch.float32:
            raise QuantError(L.ERR_GRID, "quantized matrix parts disagree: scales must be f32")
        return QuantizedMatrix(codes.contiguous(), scales.contiguous(), rows, cols, gr, gc, dtype, granularity)

    def shape(self):
        return [self._rows, self._cols]

    def dtype(self) -> QuantDtype:
        return self._dtype

    def granularity(self) -> Granularity:
        return self._granularity

    def tile(self):
        return (self._gr, self._gc)

    def codes(self) -> torch.Tensor:
        return self._codes

    def scales(self) -> torch.Tensor:
        return self._scales

    def dequantize(self) -> torch.Tensor:
        """quant.rs:605-637 — one device dispatch back to f32 ``[R, C]``, bit-exact ``s * f32(q)``."""
        _require_cuda(self._codes, "the codes")
        out = torch.empty((self._rows, self._cols), dtype=torch.float32, device=self._codes.device)
        with torch.cuda.device(out.device):
            check(L.load().qb200_dequantize(self._codes.data_ptr(), self._scales.data_ptr(), self._rows, self._cols,
                                            self._dtype.bits(), self._gr, self._gc, out.data_ptr(), _stream(out)))
        return out

    def __repr__(self):
        return (f"QuantizedMatrix {{ shape: {self.shape()}, dtype: {self._dtype.name}, "
                f"granularity: {self._granularity!r}, tile: {self.tile()}, .. }}")
