"""Column-sharded tensor parallelism for QuantizedLinear (one process per GPU).

The reference has no distributed code (``crates/ml/quanta-nn/PARITY.md:76-79``); this module is
the sharding the BASELINE configuration asks for.  Output features are independent, so rank p owns a
contiguous block of rows of the ``[out, in]`` codes and scales — a slice, no data movement — and
the shard outputs are all-gathered along the feature axis (``torch.distributed``: NCCL over
NVLink on GPUs, gloo on CPU for the host-side tests).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib as L
from .nn_quant import QuantizedLinear
from .quant import QuantError, QuantizedMatrix


def shard_range(out_dim: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Rows [lo, hi) of rank's shard: equal blocks rounded up to ``multiple`` (the scale tile height,
    so no tile straddles a boundary); trailing ranks may get a short or empty block."""
    if world < 1 or not 0 <= rank < world:
        raise QuantError(L.ERR_INVALID_PARAM, f"shard_range: rank {rank} outside world of {world}")
    if multiple < 1:
        raise QuantError(L.ERR_INVALID_PARAM, "shard_range: multiple must be positive")
    per = -(-out_dim // world)
    per = -(-per // multiple) * multiple
    lo = min(out_dim, rank * per)
    return lo, min(out_dim, lo + per)


def shard_matrix(m: QuantizedMatrix, world: int, rank: int) -> QuantizedMatrix:
    """Rank's row block of an ``[out, in]`` matrix: views into the codes and the scale grid."""
    rows, cols = m.shape()
    gr, gc = m.tile()
    lo, hi = shard_range(rows, world, rank, gr)
    if hi <= lo:
        raise QuantError(L.ERR_INVALID_PARAM, f"shard_matrix: rank {rank} of {world} owns no rows of a {rows}-row matrix")
    codes = m.codes()[lo:hi].contiguous()
    scales = m.scales()[lo // gr: -(-hi // gr)].contiguous()
    return QuantizedMatrix(codes, scales, hi - lo, cols, min(gr, hi - lo), gc, m.dtype(), m.granularity())


def gather_columns(y_local: torch.Tensor, out_dim: int, group=None, multiple: int = 1) -> torch.Tensor:
    """All-gather of the shard outputs along the feature axis.  ``y_local`` is ``[m, n_local]``;
    returns ``[m, out_dim]`` on every rank.  Shards are padded to the widest one for the collective."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    m = y_local.shape[0]
    ranges = [shard_range(out_dim, world, r, multiple) for r in range(world)]
    widths = [hi - lo for lo, hi in ranges]
    return _gather(y_local, m, widths, group)


def _gather(y_local, m, widths, group):
    world, wmax = len(widths), max(widths)
    send = y_local
    if y_local.shape[1] != wmax:
        send = torch.zeros((m, wmax), dtype=y_local.dtype, device=y_local.device)
        send[:, : y_local.shape[1]] = y_local
    flat = torch.empty((world * m, wmax), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    out = flat.view(world, m, wmax)
    return torch.cat([out[r, :, : widths[r]] for r in range(world)], dim=1)


class TensorParallelLinear:
    """A QuantizedLinear whose output features are sharded over the ranks of a process group."""

    def __init__(self, local: Optional[QuantizedLinear], out_dim: int, widths: List[int], group=None):
        self.local, self._out, self._widths, self.group = local, out_dim, widths, group

    @classmethod
    def new(cls, w: QuantizedMatrix, b: Optional[torch.Tensor] = None, group=None) -> "TensorParallelLinear":
        """Shards an ``[out, in]`` matrix (and its bias) by rows of the scale grid over the group."""
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        rows, _ = w.shape()
        gr, _ = w.tile()
        ranges = [shard_range(rows, world, r, gr) for r in range(world)]
        lo, hi = ranges[rank]
        local = None
        if hi > lo:
            local = QuantizedLinear.new(shard_matrix(w, world, rank), None if b is None else b[lo:hi].contiguous(), L.OUT_IN)
        return cls(local, rows, [h - l for l, h in ranges], group)

    def out_dim(self) -> int:
        return self._out

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        rank = dist.get_rank(self.group)
        if self.local is not None:
            y = self.local.forward(x, out_dtype=out_dtype)
        else:
            y = torch.empty((x.shape[0], 0), dtype=out_dtype, device=x.device)
        assert y.shape[1] == self._widths[rank]
        if dist.get_world_size(self.group) == 1:
            return y
        return _gather(y, x.shape[0], self._widths, self.group)
