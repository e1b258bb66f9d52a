"""Decode-step support ops and a Llama-shaped decoder stack over QuantizedLinear layers.

The reference composes these ops from `quanta-nn` (`norm.rs`, `rope.rs`, `kernel.rs`,
`activation.rs`, `attention.rs`); here each is one CUDA kernel behind the C ABI, and the
stack strings them together around the grouped decode launches (fused QKV, fused gate + up,
a down projection run as column slices of at most 4096 inputs).  Residual stream in f32,
inputs of the linears and the KV cache in bf16.
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional

import numpy as np
import torch

from . import _lib as L
from .nn_quant import QuantizedLinear
from .quant import Group, QuantDtype, QuantError, QuantizedMatrix, check as _check


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], gamma: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None):
    """h += delta (in place, when delta is given; a ``[parts, n, c]`` delta is summed over parts first);
    returns bf16(rmsnorm(h) * gamma)."""
    n, c = h.shape
    out = torch.empty(n, c, dtype=torch.bfloat16, device=h.device) if out is None else out
    parts = 0 if delta is None else (delta.shape[0] if delta.dim() == 3 else 1)
    _check(L.load().qb200_add_rmsnorm(h.data_ptr(), 0 if delta is None else delta.data_ptr(), parts, gamma.data_ptr(), n, c, eps,
                                      out.data_ptr(), _stream(h.device)))
    return out


def rope_rows(pos: int, d: int, base: float = 10000.0):
    """cos / sin rows of one position, computed in float64 and cast to float32 (numpy arrays)."""
    half = d // 2
    theta = float(pos) * np.power(float(base), -2.0 * np.arange(half, dtype=np.float64) / float(d))
    c, s = np.cos(theta), np.sin(theta)
    return np.concatenate([c, c]).astype(np.float32), np.concatenate([s, s]).astype(np.float32)


def rope_append(q, k, v, cos_row, sin_row, heads: int, q_out, kcache, vcache, pos: int):
    b = q.shape[0]
    hd = q.shape[1] // heads
    _check(L.load().qb200_rope_append(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos_row.data_ptr(), sin_row.data_ptr(), b, heads, hd,
                                      q_out.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), kcache.shape[1], pos, _stream(q.device)))


def sdpa_decode(q, kcache, vcache, kv_len: int, scale: float, scratch, out):
    b, ctx_max, heads, hd = kcache.shape
    _check(L.load().qb200_sdpa_decode(q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), b, heads, hd, ctx_max, kv_len, scale,
                                      scratch.data_ptr(), out.data_ptr(), _stream(q.device)))
    return out


def sdpa_scratch(b: int, heads: int, kv_len: int, device) -> torch.Tensor:
    return torch.empty(int(L.load().qb200_sdpa_decode_scratch_floats(b, heads, kv_len)), dtype=torch.float32, device=device)


def swiglu_sliced(gate, up, widths: List[int], out, pad_to: int = 0):
    """silu(gate) * up as bf16 in column slices: block s is ``[n, widths[s]]`` (``[n, pad_to]`` with pad_to > 0; the
    padding columns are not written)."""
    n, h = gate.shape
    w = (ctypes.c_uint32 * len(widths))(*widths)
    _check(L.load().qb200_swiglu_sliced(gate.data_ptr(), up.data_ptr(), n, h, w, len(widths), pad_to, out.data_ptr(),
                                        _stream(gate.device)))
    return out


def sum_arrays(parts: torch.Tensor, out: torch.Tensor):
    _check(L.load().qb200_sum_arrays(parts.data_ptr(), parts.shape[0], out.numel(), out.data_ptr(), _stream(out.device)))
    return out


def _slices(width: int, limit: int = 4096, group: int = 128) -> List[int]:
    """Column slices of a linear's input: as few as cover `width` with at most `limit` columns each,
    every one a multiple of the scale group."""
    n = -(-width // limit)
    groups = width // group
    base, extra = divmod(groups, n)
    return [(base + (1 if i < extra else 0)) * group for i in range(n)]


class DecoderStack:
    """`n_layers` Llama-shaped blocks with int4 (grid 1x128) linears, random-initialised, plus the final
    norm and the vocabulary projection.  `step()` runs one decode step for `batch` sequences at cache
    position `pos` and returns the logits."""

    def __init__(self, n_layers: int, d: int, heads: int, ffn: int, vocab: int, batch: int, ctx_max: int, device,
                 seed: int = 4, eps: float = 1e-5, rope_base: float = 10000.0):
        if d % heads or (d // heads) != 128:
            raise QuantError(L.ERR_NOT_SUPPORTED, "DecoderStack: head dim 128 only")
        self.n_layers, self.d, self.heads, self.ffn, self.vocab, self.batch, self.ctx_max = n_layers, d, heads, ffn, vocab, batch, ctx_max
        self.eps, self.rope_base, self.device = eps, rope_base, device
        gen = torch.Generator(device=device).manual_seed(seed)

        def qlin(n_out, n_in, pad_to=0):
            w = torch.randn(n_out, n_in, device=device, generator=gen) * 0.02
            if pad_to > n_in:  # zero weights for the padding columns of a slice (their codes and scales are zero)
                w = torch.cat([w, torch.zeros(n_out, pad_to - n_in, device=device)], 1)
            return QuantizedLinear.new(QuantizedMatrix.quantize(w, QuantDtype.Int4, Group(1, 128)), None, L.OUT_IN)

        # the down projection runs as column slices of its input, all padded to one width so that the slices are
        # ONE grouped launch: W_down = [W_0 | W_1 | ...], y = sum_s x_s @ W_s^T
        self.down_widths = _slices(ffn)
        self.down_pad = -(-max(self.down_widths) // 512) * 512  # rows of scales that are whole 16-byte units
        self.layers = []
        for _ in range(n_layers):
            blk = {"qkv": [qlin(d, d) for _ in range(3)], "o": qlin(d, d), "gate_up": [qlin(ffn, d) for _ in range(2)],
                   "down": [qlin(d, w, self.down_pad) for w in self.down_widths],
                   "g1": torch.ones(d, device=device), "g2": torch.ones(d, device=device)}
            self.layers.append(blk)
        self.g_final = torch.ones(d, device=device)
        self.lm_head = qlin(vocab, d)
        self.weight_bytes = sum(self._bytes(q) for blk in self.layers for key in ("qkv", "gate_up", "down") for q in blk[key])
        self.weight_bytes += sum(self._bytes(blk["o"]) for blk in self.layers) + self._bytes(self.lm_head)
        hd = d // heads
        self.kcache = torch.randn(n_layers, batch, ctx_max, heads, hd, device=device, generator=gen).to(torch.bfloat16)
        self.vcache = torch.randn(n_layers, batch, ctx_max, heads, hd, device=device, generator=gen).to(torch.bfloat16)
        f32 = dict(dtype=torch.float32, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)
        self.h = torch.zeros(batch, d, **f32)
        self.xn = torch.empty(batch, d, **bf)
        self.qkv = torch.empty(3, batch, d, **f32)
        self.qb = torch.empty(batch, d, **bf)
        self.att = torch.empty(batch, d, **bf)
        self.o = torch.empty(batch, d, **f32)
        self.gu = torch.empty(2, batch, ffn, **f32)
        self.act = torch.zeros(len(self.down_widths), batch, self.down_pad, **bf)  # [slice][batch][padded width]
        self.down_parts = torch.empty(len(self.down_widths), batch, d, **f32)
        self.logits = torch.empty(batch, vocab, **f32)
        self.scratch = sdpa_scratch(batch, heads, ctx_max, device)
        self.cos = torch.empty(hd, **f32)
        self.sin = torch.empty(hd, **f32)
        self._act_views = [self.act[i] for i in range(len(self.down_widths))]

    @staticmethod
    def _bytes(ql: QuantizedLinear) -> int:
        return ql.out_dim() * ql.in_dim() // 2 + ql.out_dim() * (ql.in_dim() // 128) * 4

    def kv_bytes(self, kv_len: int) -> int:
        return 2 * self.n_layers * self.batch * kv_len * self.d * 2

    def set_position(self, pos: int):
        c, s = rope_rows(pos, self.d // self.heads, self.rope_base)
        self.cos.copy_(torch.from_numpy(c))
        self.sin.copy_(torch.from_numpy(s))
        self.pos = pos

    def step(self, h0: torch.Tensor) -> torch.Tensor:
        """One decode step from the embedded tokens h0 [batch, d] (f32) at the position given to set_position."""
        f32 = torch.float32
        self.h.copy_(h0)
        pos, kv_len, scale = self.pos, self.pos + 1, 1.0 / math.sqrt(self.d // self.heads)
        delta = None
        for li, blk in enumerate(self.layers):
            add_rmsnorm(self.h, delta, blk["g1"], self.eps, self.xn)
            QuantizedLinear.forward_many(blk["qkv"], [self.xn] * 3, out_dtype=f32, outs=[self.qkv[0], self.qkv[1], self.qkv[2]])
            rope_append(self.qkv[0], self.qkv[1], self.qkv[2], self.cos, self.sin, self.heads, self.qb, self.kcache[li], self.vcache[li], pos)
            sdpa_decode(self.qb, self.kcache[li], self.vcache[li], kv_len, scale, self.scratch, self.att)
            blk["o"].forward(self.att, out_dtype=f32, out=self.o)
            add_rmsnorm(self.h, self.o, blk["g2"], self.eps, self.xn)
            QuantizedLinear.forward_many(blk["gate_up"], [self.xn] * 2, out_dtype=f32, outs=[self.gu[0], self.gu[1]])
            swiglu_sliced(self.gu[0], self.gu[1], self.down_widths, self.act, self.down_pad)
            QuantizedLinear.forward_many(blk["down"], self._act_views, out_dtype=f32, outs=[p for p in self.down_parts])
            delta = self.down_parts  # summed by the next add_rmsnorm
        add_rmsnorm(self.h, delta, self.g_final, self.eps, self.xn)
        self.lm_head.forward(self.xn, out_dtype=f32, out=self.logits)
        return self.logits
