"""Decode-step support ops and a Llama-shaped decoder stack over QuantizedLinear layers.

The reference composes these ops from `quanta-nn` (`norm.rs`, `rope.rs`, `kernel.rs`,
`activation.rs`, `attention.rs`); here each is one CUDA kernel behind the C ABI, and the
stack strings them together around the grouped decode launches (fused QKV, fused gate + up,
a down projection run as column slices of at most 4096 inputs).  Residual stream in f32,
inputs of the linears and the KV cache in bf16.

With a process group the stack is tensor-parallel over the node's GPUs (the reference has no multi-GPU
code, ``crates/ml/quanta-nn/PARITY.md:76-79``; the head split is its column blocks of width ``hd``,
``crates/ml/quanta-nn/src/attention.rs``): whole heads per rank, two exchanges per block, each fused
into the decode kernel that produces the data (peer stores + arrival barrier, ``tp.PeerArena``).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

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


def _split_groups(groups: int, n: int) -> List[int]:
    """`groups` scale groups of 128 columns cut into n runs as even as possible; widths in columns."""
    base, extra = divmod(groups, n)
    return [(base + (1 if i < extra else 0)) * 128 for i in range(n)]


def shard_units(units: int, world: int, rank: int) -> Tuple[int, int]:
    """Units [lo, hi) of `units` equal pieces (heads, scale groups, vocabulary rows) that rank owns: the first
    ``units % world`` ranks own one more than the others."""
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


@dataclass(frozen=True)
class StackPlan:
    """How one rank of `world` cuts a Llama-shaped block, and where each rank's outputs lie in the exchange
    buffers (identical on every rank, so a peer's copy of a slot is at the same offset of its arena).

    Whole heads per rank: Q, K, V are column-sharded (rows [q_lo, q_hi) of the `[out, in]` weights), so RoPE,
    the KV cache and attention are local to the rank's heads.  The output projection is row-parallel over the
    same features (columns [q_lo, q_hi) of W_o): every rank produces a partial `[batch, d]` and pushes it into
    slot `rank` of every rank's buffer "o"; the next add + RMSNorm sums the slots.  Gate and up are column-sharded
    over whole scale groups of the FFN width, SwiGLU is local, and the down projection is row-parallel over the
    same columns, cut into `down_slices` runs of at most 4096 inputs padded to one width: buffer "d" holds
    `[world, down_slices, batch, d]` partial outputs.  The vocabulary projection is column-sharded and its
    logits are gathered from buffer "v" `[world, batch, v_max]`.  Buffer elements are 8 bytes: the exchanges are
    pushed (every value travels with the number of its exchange and the consumers poll for it; no barrier), and
    consecutive exchanges alternate between "o" and "d", which is what makes reusing a buffer safe."""
    world: int
    rank: int
    d: int
    heads: int
    ffn: int
    vocab: int
    batch: int
    q_lo: int
    q_hi: int
    f_lo: int
    f_hi: int
    v_lo: int
    v_hi: int
    v_max: int
    down_widths: Tuple[int, ...]
    down_pad: int
    down_slices: int

    @staticmethod
    def make(world: int, rank: int, d: int, heads: int, ffn: int, vocab: int, batch: int) -> "StackPlan":
        if world < 1 or not 0 <= rank < world:
            raise QuantError(L.ERR_INVALID_PARAM, f"DecoderStack: rank {rank} outside a world of {world}")
        if heads % world:
            raise QuantError(L.ERR_INVALID_PARAM, f"DecoderStack: {heads} heads do not divide over {world} ranks")
        if ffn % 128 or ffn // 128 < world:
            raise QuantError(L.ERR_INVALID_PARAM, "DecoderStack: the FFN width must be whole scale groups (128), at least one per rank")
        if vocab < world:
            raise QuantError(L.ERR_INVALID_PARAM, "DecoderStack: fewer vocabulary rows than ranks")
        hd = d // heads
        h_lo, h_hi = shard_units(heads, world, rank)
        g_lo, g_hi = shard_units(ffn // 128, world, rank)
        v_lo, v_hi = shard_units(vocab, world, rank)
        # every rank cuts its FFN columns into the same number of runs, padded to the widest run of any rank
        g_max = shard_units(ffn // 128, world, 0)[1]
        n_slices = -(-g_max * 128 // 4096)
        pad = -(-max(_split_groups(g_max, n_slices)) // 512) * 512  # rows of scales that are whole 16-byte units
        v0 = shard_units(vocab, world, 0)
        return StackPlan(world, rank, d, heads, ffn, vocab, batch, h_lo * hd, h_hi * hd, g_lo * 128, g_hi * 128, v_lo, v_hi,
                         v0[1] - v0[0], tuple(_split_groups(g_hi - g_lo, n_slices)), pad, n_slices)

    ELEM = 8  # bytes of a pushed element: the f32 bits and the number of the exchange that wrote them

    def arena_sizes(self) -> Dict[str, int]:
        return {"o": self.world * self.batch * self.d * self.ELEM,
                "d": self.world * self.down_slices * self.batch * self.d * self.ELEM,
                "v": self.world * self.batch * self.v_max * self.ELEM}

    def o_offset(self, rank: int) -> int:
        return rank * self.batch * self.d * self.ELEM

    def d_offset(self, rank: int, s: int) -> int:
        return (rank * self.down_slices + s) * self.batch * self.d * self.ELEM

    def v_offset(self, rank: int) -> int:
        return rank * self.batch * self.v_max * self.ELEM


def _rows_of(m: QuantizedMatrix, lo: int, hi: int) -> QuantizedMatrix:
    """Rows [lo, hi) of an `[out, in]` int4 1x128 matrix (a column shard of the layer): copies of the slices."""
    _, cols = m.shape()
    return QuantizedMatrix(m.codes()[lo:hi].contiguous(), m.scales()[lo:hi].contiguous(), hi - lo, cols, 1, 128, m.dtype(), m.granularity())


def _cols_of(m: QuantizedMatrix, lo: int, hi: int, pad_to: int = 0) -> QuantizedMatrix:
    """Columns [lo, hi) (whole scale groups) of an `[out, in]` int4 1x128 matrix (a row-parallel shard), padded with
    zero codes and zero scales to `pad_to` columns."""
    rows, _ = m.shape()
    width = max(hi - lo, pad_to)
    codes = torch.zeros(rows, width // 8, dtype=m.codes().dtype, device=m.codes().device)
    scales = torch.zeros(rows, width // 128, dtype=torch.float32, device=m.codes().device)
    codes[:, : (hi - lo) // 8] = m.codes()[:, lo // 8: hi // 8]
    scales[:, : (hi - lo) // 128] = m.scales()[:, lo // 128: hi // 128]
    return QuantizedMatrix(codes, scales, rows, width, 1, 128, m.dtype(), m.granularity())


class DecoderStack:
    """`n_layers` Llama-shaped blocks with int4 (grid 1x128) linears, random-initialised, plus the final
    norm and the vocabulary projection.  `step()` runs one decode step for `batch` sequences at cache
    position `pos` and returns the logits.

    With `group` (a torch.distributed process group of the node's GPUs, one process each) the stack is
    tensor-parallel as `StackPlan` describes; every rank draws the same full weights from `seed`, quantizes
    them and keeps its shard, so the sharded stack holds exactly the codes and scales of the single-GPU one
    and differs from it only in the order of the f32 sums across ranks."""

    def __init__(self, n_layers: int, d: int, heads: int, ffn: int, vocab: int, batch: int, ctx_max: int, device,
                 seed: int = 4, eps: float = 1e-5, rope_base: float = 10000.0, group=None):
        if d % heads or (d // heads) != 128:
            raise QuantError(L.ERR_NOT_SUPPORTED, "DecoderStack: head dim 128 only")
        self.n_layers, self.d, self.heads, self.ffn, self.vocab, self.batch, self.ctx_max = n_layers, d, heads, ffn, vocab, batch, ctx_max
        self.eps, self.rope_base, self.device = eps, rope_base, device
        self.group = group
        self.exchange = True  # False: step() leaves every exchange out (for timing what the exchanges cost)
        world = rank = 0
        if group is not None:
            import torch.distributed as dist
            world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.world, self.rank = max(world, 1), rank
        self.plan = p = StackPlan.make(self.world, rank, d, heads, ffn, vocab, batch)
        self.arena = None
        if self.world > 1:
            from .tp import PeerArena
            self.arena = PeerArena(p.arena_sizes(), group)
        gen = torch.Generator(device=device).manual_seed(seed)

        def full(n_out, n_in):  # the same full matrix on every rank
            w = torch.randn(n_out, n_in, device=device, generator=gen) * 0.02
            return QuantizedMatrix.quantize(w, QuantDtype.Int4, Group(1, 128))

        def lin(qm):
            return QuantizedLinear.new(qm, None, L.OUT_IN)

        self.heads_local = (p.q_hi - p.q_lo) // 128
        self.d_local = p.q_hi - p.q_lo
        self.f_local = p.f_hi - p.f_lo
        self.down_widths, self.down_pad = list(p.down_widths), p.down_pad
        self.layers = []
        for _ in range(n_layers):
            qkv = [lin(_rows_of(full(d, d), p.q_lo, p.q_hi)) for _ in range(3)]
            o = lin(_cols_of(full(d, d), p.q_lo, p.q_hi))
            gate_up = [lin(_rows_of(full(ffn, d), p.f_lo, p.f_hi)) for _ in range(2)]
            wd, down, c0 = full(d, ffn), [], p.f_lo
            for w in self.down_widths:
                down.append(lin(_cols_of(wd, c0, c0 + w, self.down_pad)))
                c0 += w
            del wd
            self.layers.append({"qkv": qkv, "o": o, "gate_up": gate_up, "down": down,
                                "g1": torch.ones(d, device=device), "g2": torch.ones(d, device=device)})
        self.g_final = torch.ones(d, device=device)
        self.lm_head = lin(_rows_of(full(vocab, d), p.v_lo, p.v_hi))
        self.weight_bytes = sum(self._bytes(q) for blk in self.layers for key in ("qkv", "gate_up", "down") for q in blk[key])
        self.weight_bytes += sum(self._bytes(blk["o"]) for blk in self.layers) + self._bytes(self.lm_head)
        hd, hl, dl = d // heads, self.heads_local, self.d_local
        # random cache contents: every rank draws the full cache of a block and keeps its heads
        self.kcache = torch.empty(n_layers, batch, ctx_max, hl, hd, dtype=torch.bfloat16, device=device)
        self.vcache = torch.empty(n_layers, batch, ctx_max, hl, hd, dtype=torch.bfloat16, device=device)
        h_lo = p.q_lo // hd
        for cache in (self.kcache, self.vcache):
            for li in range(n_layers):
                cache[li].copy_(torch.randn(batch, ctx_max, heads, hd, device=device, generator=gen)[:, :, h_lo: h_lo + hl])
        f32 = dict(dtype=torch.float32, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)
        ns = p.down_slices
        self.h = torch.zeros(batch, d, **f32)
        self.xn = torch.empty(batch, d, **bf)
        self.qkv = torch.empty(3, batch, dl, **f32)
        self.qb = torch.empty(batch, dl, **bf)
        self.att = torch.empty(batch, dl, **bf)
        self.gu = torch.empty(2, batch, self.f_local, **f32)
        self.act = torch.zeros(ns, batch, self.down_pad, **bf)  # [slice][batch][padded width]
        self.scratch = sdpa_scratch(batch, hl, ctx_max, device)
        self.cos = torch.empty(hd, **f32)
        self.sin = torch.empty(hd, **f32)
        self._act_views = [self.act[i] for i in range(ns)]
        self.logits = torch.empty(batch, vocab, **f32)
        if self.arena is None:
            self.o = torch.empty(1, batch, d, **f32)
            self.down_parts = torch.empty(ns, batch, d, **f32)
        else:
            a = self.arena
            self._o_own = [a.address("o", p.o_offset(rank))]
            self._d_own = [a.address("d", p.d_offset(rank, s)) for s in range(ns)]
            self._v_own = [a.address("v", p.v_offset(rank))]
            # what the exchanges are timed against: the same launches storing plain f32 locally
            self._o_local = torch.empty(1, batch, d, **f32)
            self._d_local = torch.empty(ns, batch, d, **f32)
            self._v_local = torch.empty(batch, p.v_hi - p.v_lo, **f32)

    @staticmethod
    def _bytes(ql: QuantizedLinear) -> int:
        return ql.out_dim() * ql.in_dim() // 2 + ql.out_dim() * (ql.in_dim() // 128) * 4

    def kv_bytes(self, kv_len: int) -> int:
        """Bytes of this rank's KV rows read by one step."""
        return 2 * self.n_layers * self.batch * kv_len * self.d_local * 2

    def exchange_bytes(self) -> int:
        """Bytes this rank stores into EACH peer per step (partial outputs of the output and down projections,
        its slice of the logits; 8 bytes per value)."""
        p = self.plan
        return (self.n_layers * (1 + p.down_slices) * self.batch * self.d + self.batch * (p.v_hi - p.v_lo)) * p.ELEM

    def set_position(self, pos: int):
        c, s = rope_rows(pos, self.d // self.heads, self.rope_base)
        self.cos.copy_(torch.from_numpy(c))
        self.sin.copy_(torch.from_numpy(s))
        self.pos = pos

    def step(self, h0: torch.Tensor) -> torch.Tensor:
        """One decode step from the embedded tokens h0 [batch, d] (f32, the same on every rank) at the position
        given to set_position; returns the logits [batch, vocab] (on every rank)."""
        if self.arena is not None and not self.exchange:
            return self._step_without_exchanges(h0)
        f32 = torch.float32
        self.h.copy_(h0)
        pos, kv_len, scale = self.pos, self.pos + 1, 1.0 / math.sqrt(self.d // self.heads)
        a, B, W, ns = self.arena, self.batch, self.world, self.plan.down_slices
        first = True
        for li, blk in enumerate(self.layers):
            if a is None or first:
                add_rmsnorm(self.h, None if first else self.down_parts, blk["g1"], self.eps, self.xn)
            else:  # the down projection's partial outputs of every rank and slice, pushed into buffer "d"
                a.add_rmsnorm_pushed(self.h, "d", W * ns, blk["g1"], self.eps, self.xn)
            first = False
            QuantizedLinear.forward_many(blk["qkv"], [self.xn] * 3, out_dtype=f32, outs=[self.qkv[0], self.qkv[1], self.qkv[2]])
            rope_append(self.qkv[0], self.qkv[1], self.qkv[2], self.cos, self.sin, self.heads_local, self.qb, self.kcache[li], self.vcache[li], pos)
            sdpa_decode(self.qb, self.kcache[li], self.vcache[li], kv_len, scale, self.scratch, self.att)
            if a is None:
                blk["o"].forward(self.att, out_dtype=f32, out=self.o[0])
                add_rmsnorm(self.h, self.o, blk["g2"], self.eps, self.xn)
            else:  # partial outputs over this rank's heads -> slot `rank` of every rank's buffer "o"
                a.push_pushed([blk["o"]], [self.att], self._o_own, B)
                a.add_rmsnorm_pushed(self.h, "o", W, blk["g2"], self.eps, self.xn)
            QuantizedLinear.forward_many(blk["gate_up"], [self.xn] * 2, out_dtype=f32, outs=[self.gu[0], self.gu[1]])
            swiglu_sliced(self.gu[0], self.gu[1], self.down_widths, self.act, self.down_pad)
            if a is None:
                QuantizedLinear.forward_many(blk["down"], self._act_views, out_dtype=f32, outs=[p for p in self.down_parts])
            else:
                a.push_pushed(blk["down"], self._act_views, self._d_own, B)
        if a is None:
            add_rmsnorm(self.h, self.down_parts if self.layers else None, self.g_final, self.eps, self.xn)
            self.lm_head.forward(self.xn, out_dtype=f32, out=self.logits)
            return self.logits
        if self.layers:
            a.add_rmsnorm_pushed(self.h, "d", W * ns, self.g_final, self.eps, self.xn)
        else:
            add_rmsnorm(self.h, None, self.g_final, self.eps, self.xn)
        # the logits: a block with no layers would push twice in a row into nothing in between; the vocabulary
        # buffer is a third one, so the alternation of "o" and "d" is not disturbed
        a.push_pushed([self.lm_head], [self.xn], self._v_own, B)
        a.gather_pushed("v", W, B * self.plan.v_max, B, self.vocab, self.logits)
        return self.logits

    def _step_without_exchanges(self, h0: torch.Tensor) -> torch.Tensor:
        """The sharded step with every exchange left out: each rank keeps its own partial outputs (plain f32, local)
        and nothing waits.  Its logits mean nothing; its time is what the exchanges are measured against."""
        f32 = torch.float32
        self.h.copy_(h0)
        pos, kv_len, scale = self.pos, self.pos + 1, 1.0 / math.sqrt(self.d // self.heads)
        delta = None
        for li, blk in enumerate(self.layers):
            add_rmsnorm(self.h, delta, blk["g1"], self.eps, self.xn)
            QuantizedLinear.forward_many(blk["qkv"], [self.xn] * 3, out_dtype=f32, outs=[self.qkv[0], self.qkv[1], self.qkv[2]])
            rope_append(self.qkv[0], self.qkv[1], self.qkv[2], self.cos, self.sin, self.heads_local, self.qb, self.kcache[li], self.vcache[li], pos)
            sdpa_decode(self.qb, self.kcache[li], self.vcache[li], kv_len, scale, self.scratch, self.att)
            QuantizedLinear.forward_many([blk["o"]], [self.att], out_dtype=f32, outs=[self._o_local[0]])
            add_rmsnorm(self.h, self._o_local, blk["g2"], self.eps, self.xn)
            QuantizedLinear.forward_many(blk["gate_up"], [self.xn] * 2, out_dtype=f32, outs=[self.gu[0], self.gu[1]])
            swiglu_sliced(self.gu[0], self.gu[1], self.down_widths, self.act, self.down_pad)
            QuantizedLinear.forward_many(blk["down"], self._act_views, out_dtype=f32, outs=[p for p in self._d_local])
            delta = self._d_local
        add_rmsnorm(self.h, delta, self.g_final, self.eps, self.xn)
        QuantizedLinear.forward_many([self.lm_head], [self.xn], out_dtype=f32, outs=[self._v_local])
        return self.logits

    def close(self):
        if self.arena is not None:
            self.arena.close()
            self.arena = None
