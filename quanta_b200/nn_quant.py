"""Layer / checkpoint mirror of ``quanta::nn::quant`` over the qb200 C ABI.

Same names and argument meaning as the reference's
``crates/ml/quanta-nn/src/quant.rs``: ``QuantLeaf``, ``quantize_named``,
``save_named``, ``load_named`` (Mode B), ``load_named_f32`` / ``load`` (Mode A),
``LoadedQuant``, ``FORMAT_VERSION`` and ``QuantizedLinear`` (``new`` /
``dequantized`` / ``apply`` plus the tape-free ``forward``).  Checkpoint I/O is
bytes-level, like the reference.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple, Union

import numpy as np
import torch

from . import _lib as L
from .quant import (Granularity, QuantDtype, QuantError, QuantizedMatrix, _require_cuda, _stream, check,
                    granularity_from_grid)

FORMAT_VERSION = "1"

Leaf = Union[torch.Tensor, QuantizedMatrix]


@dataclass
class QuantLeaf:
    """quant.rs:152-155 — one named checkpoint leaf: plain f32, or a quantized matrix."""
    value: Leaf

    @staticmethod
    def F32(a: torch.Tensor) -> "QuantLeaf":
        return QuantLeaf(a)

    @staticmethod
    def Quantized(m: QuantizedMatrix) -> "QuantLeaf":
        return QuantLeaf(m)

    @property
    def is_quantized(self) -> bool:
        return isinstance(self.value, QuantizedMatrix)


def quantize_named(leaves: List[Tuple[str, torch.Tensor]],
                   policy: Callable[[str, torch.Tensor], Optional[Tuple[QuantDtype, Granularity]]]):
    """quant.rs:161-182 — quantize named leaves under a caller-owned policy."""
    out = []
    for name, arr in leaves:
        choice = policy(name, arr)
        if choice is None:
            out.append((name, QuantLeaf.F32(arr)))
        else:
            out.append((name, QuantLeaf.Quantized(QuantizedMatrix.quantize(arr, choice[0], choice[1]))))
    return out


def save_named(entries: List[Tuple[str, QuantLeaf]], metadata: Optional[Dict[str, str]] = None) -> bytes:
    """quant.rs:279-390 — leaves in the given order + optional user metadata -> file bytes."""
    lib = L.load()
    w = L.vp()
    check(lib.qb200_st_writer_create(ctypes.byref(w)))
    try:
        if metadata is not None:
            check(lib.qb200_st_writer_set_has_metadata(w, 1))
            for k, v in metadata.items():
                check(lib.qb200_st_writer_add_metadata(w, k.encode("utf-8"), v.encode("utf-8")))
        keep = []
        for name, leaf in entries:
            v = leaf.value if isinstance(leaf, QuantLeaf) else leaf
            if isinstance(v, QuantizedMatrix):
                codes = np.ascontiguousarray(v.codes().detach().cpu().numpy())
                scales = np.ascontiguousarray(v.scales().detach().cpu().numpy(), dtype=np.float32)
                keep += [codes, scales]
                rows, cols = v.shape()
                gr, gc = v.tile()
                check(lib.qb200_st_writer_add_quantized(w, name.encode("utf-8"), v.dtype().bits(), rows, cols, gr, gc,
                                                        codes.ctypes.data, scales.ctypes.data))
            else:
                host = np.ascontiguousarray(v.detach().to(torch.float32).cpu().numpy())
                keep.append(host)
                shape = (L.u64 * max(host.ndim, 1))(*host.shape)
                check(lib.qb200_st_writer_add_f32(w, name.encode("utf-8"), shape, host.ndim, host.ctypes.data))
        out, n = L.vp(), L.u64()
        check(lib.qb200_st_writer_finish(w, ctypes.byref(out), ctypes.byref(n)))
        return ctypes.string_at(out.value, n.value)
    finally:
        lib.qb200_st_writer_free(w)


@dataclass
class LoadedQuant:
    """quant.rs:666-669."""
    leaves: List[Tuple[str, QuantLeaf]]
    metadata: Dict[str, str] = field(default_factory=dict)


@dataclass
class LoadedSafetensors:
    """safetensors.rs:34-37."""
    tensors: List[Tuple[str, torch.Tensor]]
    metadata: Dict[str, str] = field(default_factory=dict)


class _Validated:
    """Validated view over file bytes (total validation happens before anything uploads)."""

    def __init__(self, data: bytes, allow_block: bool):
        self.lib = L.load()
        self.buf = np.frombuffer(data, dtype=np.uint8)
        self.h = L.vp()
        check(self.lib.qb200_st_validate(self.buf.ctypes.data, self.buf.size, int(allow_block), ctypes.byref(self.h)))

    def close(self):
        if self.h:
            self.lib.qb200_st_free(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def items(self):
        for i in range(self.lib.qb200_st_num_items(self.h)):
            it = L.StItem()
            check(self.lib.qb200_st_item_at(self.h, i, ctypes.byref(it)))
            yield i, it

    def metadata(self) -> Dict[str, str]:
        out = {}
        for i in range(self.lib.qb200_st_num_metadata(self.h)):
            k, v = L.cp(), L.cp()
            check(self.lib.qb200_st_metadata_at(self.h, i, ctypes.byref(k), ctypes.byref(v)))
            out[k.value.decode("utf-8")] = v.value.decode("utf-8")
        return out

    def plain_f32(self, i, it) -> np.ndarray:
        shape = [it.shape[d] for d in range(it.ndim)]
        n = max(int(np.prod(shape, dtype=np.uint64)) if shape else 1, 1)
        host = np.empty(n, dtype=np.float32)
        check(self.lib.qb200_st_plain_to_f32(self.h, i, host.ctypes.data, n))
        return host.reshape(shape) if int(np.prod(shape, dtype=np.uint64) if shape else 1) == n else host

    def matrix(self, it, device) -> QuantizedMatrix:
        rows, cols = it.shape[0], it.shape[1]
        raw = self.buf[it.data_offset:it.data_offset + it.data_len]
        if it.bits == 8:
            codes = torch.from_numpy(raw.view(np.int8).reshape(rows, cols).copy())
        else:
            codes = torch.from_numpy(raw.view("<u4").astype(np.uint32).view(np.int32).reshape(rows, -(-cols // 8)).copy())
        sraw = self.buf[it.scales_offset:it.scales_offset + it.scales_len]
        scales = torch.from_numpy(sraw.view("<f4").reshape(-(-rows // it.gr), -(-cols // it.gc)).copy())
        gran = Granularity(it.gran_kind, it.gran_axis, it.gran_size, it.gran_size2)
        return QuantizedMatrix.from_parts(codes.to(device), [rows, cols], scales.to(device), gran)


def load_named(device, data: bytes, allow_block: bool = False) -> LoadedQuant:
    """quant.rs:676-729 — **Mode B**: quantized leaves arrive resident as QuantizedMatrix
    (codes at storage width), plain leaves as f32 tensors."""
    with _Validated(data, allow_block) as v:
        leaves = []
        for i, it in v.items():
            name = it.name.decode("utf-8")
            if it.quantized:
                leaves.append((name, QuantLeaf.Quantized(v.matrix(it, device))))
            else:
                leaves.append((name, QuantLeaf.F32(torch.from_numpy(v.plain_f32(i, it)).to(device))))
        return LoadedQuant(leaves, v.metadata())


def load_named_f32(device, data: bytes, allow_block: bool = False) -> LoadedSafetensors:
    """quant.rs:735-775 — **Mode A**: every quantized leaf is dequantized before use and
    arrives as f32 ``[rows, cols]`` under its own name.  The reference dequantizes on the host
    and uploads; here the codes upload and the device kernel dequantizes (the same exact
    ``scale * q``, bit-identical)."""
    with _Validated(data, allow_block) as v:
        tensors = []
        for i, it in v.items():
            name = it.name.decode("utf-8")
            if it.quantized:
                tensors.append((name, v.matrix(it, device).dequantize()))
            else:
                tensors.append((name, torch.from_numpy(v.plain_f32(i, it)).to(device)))
        return LoadedSafetensors(tensors, v.metadata())


def load(device, witness: Dict[str, torch.Tensor], data: bytes) -> Dict[str, torch.Tensor]:
    """quant.rs:783-809 — the Mode A tree form: rebuild a tree of ``witness``'s shape,
    matching by NAME; a missing, extra or wrong-shape tensor is a loud error naming the path."""
    loaded = load_named_f32(device, data)
    by_name = dict(loaded.tensors)
    out = {}
    for name, want in witness.items():
        if name not in by_name:
            raise QuantError(L.ERR_INVALID_PARAM, f'quantized-safetensors load: missing tensor "{name}"')
        got = by_name.pop(name)
        if list(got.shape) != list(want.shape):
            raise QuantError(L.ERR_INVALID_PARAM, f'quantized-safetensors load: "{name}": shape {list(got.shape)} '
                                                  f"in file, tree wants {list(want.shape)}")
        out[name] = got
    if by_name:
        extra = next(iter(by_name))
        raise QuantError(L.ERR_INVALID_PARAM, f'quantized-safetensors load: tensor "{extra}" has no home in the tree')
    return out


_ACT = {torch.float32: L.F32, torch.bfloat16: L.BF16}
_NP_ACT = {np.dtype(np.float32): L.F32, np.dtype(np.uint16): L.BF16}


class QuantizedLinear:
    """quant.rs:830-919 — a frozen quantized dense layer ``[M, in] -> [M, out]``.

    ``layout`` IN_OUT stores the weight ``[in, out]`` like the reference's Linear
    (y = x @ deq(w)); OUT_IN stores it ``[out, in]`` (y = x @ deq(w)^T)."""

    IN_OUT, OUT_IN = L.IN_OUT, L.OUT_IN

    def __init__(self):
        raise TypeError("use QuantizedLinear.new(...) or QuantizedLinear.dequantized(...)")

    @classmethod
    def _make(cls):
        self = object.__new__(cls)
        self._h = None
        self._w = None
        self._held = None
        self._b = None
        return self

    @staticmethod
    def _check_bias(b, out_dim):
        if b is not None and list(b.shape) != [out_dim]:
            raise QuantError(L.ERR_INVALID_PARAM, f"QuantizedLinear: bias shape {list(b.shape)}, weight [in, {out_dim}] "
                                                  f"wants [{out_dim}]")

    @classmethod
    def new(cls, w: QuantizedMatrix, b: Optional[torch.Tensor] = None, layout: int = L.IN_OUT) -> "QuantizedLinear":
        """**Mode B** (quant.rs:853-862): codes stay resident; every forward is one fused kernel."""
        self = cls._make()
        rows, cols = w.shape()
        self._layout = layout
        self._in, self._out = (rows, cols) if layout == L.IN_OUT else (cols, rows)
        cls._check_bias(b, self._out)
        _require_cuda(w.codes(), "the codes")
        self._w = w
        self._b = None if b is None else b.to(torch.float32).contiguous()
        gr, gc = w.tile()
        h = L.vp()
        with torch.cuda.device(w.codes().device):
            check(L.load().qb200_qlinear_create(
                w.codes().data_ptr(), w.scales().data_ptr(), rows, cols, w.dtype().bits(), gr, gc, layout,
                None if self._b is None else self._b.data_ptr(), 0 if self._b is None else self._b.numel(),
                ctypes.byref(h)))
        self._h = h
        return self

    @classmethod
    def dequantized(cls, w: QuantizedMatrix, b: Optional[torch.Tensor] = None, layout: int = L.IN_OUT):
        """**Mode A** (quant.rs:866-876): dequantize once here and hold the f32 weight; each
        forward then costs what a plain f32 Linear costs (a library GEMM)."""
        self = cls._make()
        rows, cols = w.shape()
        self._layout = layout
        self._in, self._out = (rows, cols) if layout == L.IN_OUT else (cols, rows)
        cls._check_bias(b, self._out)
        self._held = w.dequantize()
        self._b = None if b is None else b.to(torch.float32).contiguous()
        return self

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                L.load().qb200_qlinear_destroy(h)
            except Exception:
                pass

    # Layer bookkeeping (quant.rs:879-890)
    def in_dim(self) -> int:
        return self._in

    def out_dim(self, _in: Optional[int] = None) -> int:
        return self._out

    def init(self, *_a, **_k) -> tuple:
        return ()

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The tape-free spelling of ``Layer::apply`` (quant.rs:903-918): y = x @ deq(w) (+ b).  ``out``: a
        contiguous ``[m, out]`` tensor of the output dtype to write into (Mode B)."""
        if x.dim() != 2 or x.shape[1] != self._in:
            raise QuantError(L.ERR_INVALID_PARAM, f"QuantizedLinear: input shape {list(x.shape)}, layer wants [m, {self._in}]")
        if self._held is not None:
            w = self._held if self._layout == L.IN_OUT else self._held.t()
            y = x.to(torch.float32) @ w
            if self._b is not None:
                y = y + self._b.reshape(1, self._out)
            return y if out_dtype is None else y.to(out_dtype)
        _require_cuda(x, "the input")
        if x.dtype not in _ACT:
            raise QuantError(L.ERR_INVALID_PARAM, f"QuantizedLinear: activations are f32 or bf16, got {x.dtype}")
        out_dtype = out_dtype or x.dtype
        x = x.contiguous()
        if out is not None:
            if out.shape != (x.shape[0], self._out) or out.dtype != out_dtype or not out.is_contiguous():
                raise QuantError(L.ERR_INVALID_PARAM, "QuantizedLinear: out must be a contiguous [m, out] tensor of the output dtype")
            y = out
        else:
            y = torch.empty((x.shape[0], self._out), dtype=out_dtype, device=x.device)
        with torch.cuda.device(x.device):
            check(L.load().qb200_qlinear_forward(self._h, x.data_ptr(), _ACT[x.dtype], x.shape[0], y.data_ptr(),
                                                 _ACT[out_dtype], _stream(x)))
        return y

    @staticmethod
    def forward_many(layers: List["QuantizedLinear"], xs: List[torch.Tensor], out_dtype: Optional[torch.dtype] = None,
                     outs: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
        """``[layer.forward(x) for layer, x in zip(layers, xs)]`` in one call: layers that share the input
        width and take the decode path run as one persistent launch (fused QKV / gate+up projections)."""
        if len(layers) != len(xs):
            raise QuantError(L.ERR_INVALID_PARAM, "forward_many: one input per layer")
        if not layers:
            return []
        m, dt = xs[0].shape[0], xs[0].dtype
        out_dtype = out_dtype or dt
        for ql, x in zip(layers, xs):
            if ql._h is None:
                raise QuantError(L.ERR_INVALID_PARAM, "forward_many needs Mode B layers")
            if x.dim() != 2 or x.shape[1] != ql._in or x.shape[0] != m or x.dtype != dt or dt not in _ACT:
                raise QuantError(L.ERR_INVALID_PARAM, "forward_many: inputs must be [m, in] of one f32 / bf16 dtype")
            _require_cuda(x, "the input")
        xs = [x.contiguous() for x in xs]
        if outs is None:
            outs = [torch.empty((m, ql._out), dtype=out_dtype, device=xs[0].device) for ql in layers]
        n = len(layers)
        hs = (L.vp * n)(*[ql._h for ql in layers])
        xp = (L.vp * n)(*[x.data_ptr() for x in xs])
        yp = (L.vp * n)(*[y.data_ptr() for y in outs])
        with torch.cuda.device(xs[0].device):
            check(L.load().qb200_qlinear_forward_many(hs, n, xp, _ACT[dt], m, yp, _ACT[out_dtype], _stream(xs[0])))
        return outs

    def apply(self, _tape, _params, x: torch.Tensor) -> torch.Tensor:
        """``Layer::apply(tape, &(), x)`` — the params slot is the empty tree, the tape is unused."""
        return self.forward(x)

    def forward_host(self, x: np.ndarray, y: Optional[np.ndarray] = None, bf16_out: bool = False) -> np.ndarray:
        """Host buffers in, host buffers out (H2D copy, kernel, D2H copy, synchronise).
        x: float32 ``[m, in]`` or uint16 bf16 bits ``[m, in]``."""
        if self._h is None:
            raise QuantError(L.ERR_INVALID_PARAM, "forward_host needs a Mode B layer")
        m = x.shape[0]
        xd = _NP_ACT[x.dtype]
        if y is None:
            y = np.empty((m, self._out), dtype=np.uint16 if bf16_out else np.float32)
        with torch.cuda.device(self._w.codes().device):
            check(L.load().qb200_qlinear_forward_host(self._h, x.ctypes.data, xd, m, y.ctypes.data, _NP_ACT[y.dtype]))
        return y

    def last_kernel(self) -> str:
        return L.load().qb200_qlinear_last_kernel(self._h).decode() if self._h else "f32_held"
