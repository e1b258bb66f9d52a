"""Column-sharded tensor parallelism for QuantizedLinear (one process per GPU).

The reference has no distributed code (``crates/ml/quanta-nn/PARITY.md:76-79``); this module is
the sharding of large layers over the GPUs of one node.  Output features are independent, so rank p owns a
contiguous block of rows of the ``[out, in]`` codes and scales — a slice, no data movement — and
the shard outputs are all-gathered along the feature axis (``torch.distributed``: NCCL over
NVLink on GPUs, gloo on CPU for the host-side tests).
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib as L
from .nn_quant import QuantizedLinear
from .quant import QuantError, QuantizedMatrix, check as _check


def shard_range(out_dim: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Rows [lo, hi) of rank's shard (qb200_shard_rows): equal blocks rounded up to ``multiple`` (the scale tile height,
    so no tile straddles a boundary); trailing ranks may get a short or empty block."""
    if world < 1 or not 0 <= rank < world:
        raise QuantError(L.ERR_INVALID_PARAM, f"shard_range: rank {rank} outside world of {world}")
    if multiple < 1:
        raise QuantError(L.ERR_INVALID_PARAM, "shard_range: multiple must be positive")
    lo, hi = L.u64(), L.u64()
    _check(L.load().qb200_shard_rows(out_dim, multiple, world, rank, ctypes.byref(lo), ctypes.byref(hi)))
    return lo.value, hi.value


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


class TpComm:
    """The library's own communicator (qb200_tp_create: NCCL opened at run time), one per rank with its device current.
    Rank 0's unique id travels to the other ranks through the torch process group that launched them."""

    def __init__(self, group=None):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        lib = L.load()
        ident = ctypes.create_string_buffer(128)
        dev = torch.device("cuda", torch.cuda.current_device())
        err = None
        if self.rank == 0 and self.world > 1:
            try:
                _check(lib.qb200_tp_unique_id(ident))
            except QuantError as e:
                err = e
        if self.world > 1:
            t = torch.frombuffer(bytearray(ident.raw), dtype=torch.uint8).to(dev)
            dist.broadcast(t, 0, group=group)
            ident = ctypes.create_string_buffer(t.cpu().numpy().tobytes(), 128)
        h = L.vp()
        if err is None:
            try:
                _check(lib.qb200_tp_create(self.rank, self.world, ident if self.world > 1 else None, ctypes.byref(h)))
            except QuantError as e:
                err = e
        ok = torch.tensor([0.0 if err is not None else 1.0], device=dev)
        if self.world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() == 0:
            if h.value:
                lib.qb200_tp_destroy(h)
            raise QuantError(L.ERR_NCCL, "TpComm: a rank could not create its communicator" + (f" ({err})" if err is not None else ""))
        self._h = h

    def forward(self, shard: Optional[QuantizedLinear], mode: int, full_dim: int, granule: int, x: torch.Tensor, out: torch.Tensor):
        """qb200_qlinear_forward_tp: the shard's forward plus the gather (TP_COLUMN) or the sum (TP_ROW) of the outputs."""
        act = {torch.float32: L.F32, torch.bfloat16: L.BF16}
        x = x.contiguous()
        _check(L.load().qb200_qlinear_forward_tp(self._h, shard._h if shard is not None else None, mode, full_dim, granule, x.data_ptr(),
                                                  act[x.dtype], x.shape[0], out.data_ptr(), act[out.dtype],
                                                  torch.cuda.current_stream(x.device).cuda_stream))
        return out

    def close(self):
        if self._h is not None:
            torch.cuda.synchronize()
            L.load().qb200_tp_destroy(self._h)
            self._h = None


class TensorParallelLinear:
    """A QuantizedLinear whose output features are sharded over the ranks of a process group.  On GPUs with a
    ``TpComm`` the forward is the library's qb200_qlinear_forward_tp (shard forward + NCCL all-gather behind the C
    ABI); without one the gather goes through torch.distributed (gloo on CPU ranks, for the host-side tests)."""

    def __init__(self, local: Optional[QuantizedLinear], out_dim: int, widths: List[int], group=None, comm: Optional[TpComm] = None,
                 granule: int = 1):
        self.local, self._out, self._widths, self.group, self.comm, self.granule = local, out_dim, widths, group, comm, granule

    @classmethod
    def new(cls, w: QuantizedMatrix, b: Optional[torch.Tensor] = None, group=None, comm: Optional[TpComm] = None) -> "TensorParallelLinear":
        """Shards an ``[out, in]`` matrix (and its bias) by rows of the scale grid over the group."""
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        rows, _ = w.shape()
        gr, _ = w.tile()
        ranges = [shard_range(rows, world, r, gr) for r in range(world)]
        lo, hi = ranges[rank]
        local = None
        if hi > lo:
            local = QuantizedLinear.new(shard_matrix(w, world, rank), None if b is None else b[lo:hi].contiguous(), L.OUT_IN)
        return cls(local, rows, [h - l for l, h in ranges], group, comm, gr)

    def out_dim(self) -> int:
        return self._out

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        rank = dist.get_rank(self.group)
        if self.comm is not None:
            out = torch.empty((x.shape[0], self._out), dtype=out_dtype, device=x.device)
            return self.comm.forward(self.local, L.TP_COLUMN, self._out, self.granule, x, out)
        if self.local is not None:
            y = self.local.forward(x, out_dtype=out_dtype)
        else:
            y = torch.empty((x.shape[0], 0), dtype=out_dtype, device=x.device)
        assert y.shape[1] == self._widths[rank]
        if dist.get_world_size(self.group) == 1:
            return y
        return _gather(y, x.shape[0], self._widths, self.group)


def shard_columns(m: QuantizedMatrix, world: int, rank: int):
    """Rank's block of input features (columns) of an ``[out, in]`` matrix, for the row-parallel pairing: returns
    ``(shard or None, lo, hi)``.  Boundaries are multiples of the scale tile's width (and of the eight codes of a
    packed int4 word), so no tile and no word straddles them; the shard's codes and scales are copies."""
    rows, cols = m.shape()
    gr, gc = m.tile()
    a, b = L.u64(), L.u64()
    _check(L.load().qb200_shard_cols(cols, gc, m.dtype().bits(), world, rank, ctypes.byref(a), ctypes.byref(b)))
    lo, hi = a.value, b.value
    if hi <= lo:
        return None, lo, hi
    if m.dtype().bits() == 8:
        codes = m.codes()[:, lo:hi].contiguous()
    else:
        codes = m.codes()[:, lo // 8: -(-hi // 8)].contiguous()
    scales = m.scales()[:, lo // gc: -(-hi // gc)].contiguous()
    return QuantizedMatrix(codes, scales, rows, hi - lo, gr, min(gc, hi - lo), m.dtype(), m.granularity()), lo, hi


class RowParallelLinear:
    """A QuantizedLinear whose INPUT features are sharded over the ranks: every rank multiplies its slice of the
    activations by its block of columns and the partial outputs are summed (all-reduce).  Paired after a
    column-sharded layer it consumes that layer's local output as is, so a block of two linears needs one
    collective instead of two.  The sum's order differs from the unsharded layer's: equal to 1e-4, not bit for bit."""

    def __init__(self, local: Optional[QuantizedLinear], bias: Optional[torch.Tensor], out_dim: int, lo: int, hi: int, group=None,
                 comm: Optional[TpComm] = None):
        self.local, self.bias, self._out, self.lo, self.hi, self.group, self.comm = local, bias, out_dim, lo, hi, group, comm

    @classmethod
    def new(cls, w: QuantizedMatrix, b: Optional[torch.Tensor] = None, group=None, comm: Optional[TpComm] = None) -> "RowParallelLinear":
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        shard, lo, hi = shard_columns(w, world, rank)
        local = None if shard is None else QuantizedLinear.new(shard, None, L.OUT_IN)
        return cls(local, None if b is None else b.to(torch.float32), w.shape()[0], lo, hi, group, comm)

    def out_dim(self) -> int:
        return self._out

    def forward(self, x: torch.Tensor, sliced: bool = False) -> torch.Tensor:
        """``x`` is the full ``[m, in]`` activation (this rank's columns are cut out) or, with ``sliced``, already
        this rank's ``[m, hi - lo]`` block.  Returns the f32 ``[m, out]`` on every rank."""
        if self.comm is not None:  # the shard's forward and the sum behind the C ABI (qb200_qlinear_forward_tp)
            xs = x if sliced else x[:, self.lo: self.hi].contiguous()
            y = torch.empty((x.shape[0], self._out), dtype=torch.float32, device=x.device)
            self.comm.forward(self.local, L.TP_ROW, self._out, 1, xs, y)
            if self.bias is not None:
                y = y + self.bias.to(y.device).reshape(1, self._out)
            return y
        if self.local is not None:
            xs = x if sliced else x[:, self.lo: self.hi].contiguous()
            y = self.local.forward(xs, out_dtype=torch.float32)
        else:
            y = torch.zeros((x.shape[0], self._out), dtype=torch.float32, device=x.device)
        if dist.get_world_size(self.group) > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias is not None:
            y = y + self.bias.to(y.device).reshape(1, self._out)
        return y


class _RawCuda:
    """A raw device allocation seen through the CUDA array interface (torch.as_tensor aliases it)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


class PeerArena:
    """One device allocation per rank, shared with the node's other ranks through CUDA IPC, cut into named
    buffers of the same layout on every rank, plus the barrier state (16 u64) of the arrival barrier.

    ``push`` runs the grouped decode kernel with peer stores: every output element is written to the same
    offset of EVERY rank's arena (plain stores over NVLink, no collective), and the launch's last CTA runs the
    arrival barrier, so when the launch ends all ranks' outputs are here.  What a rank writes and where is the
    caller's layout: giving every rank its own slot of a buffer makes the exchange an all-gather (column
    shards) or, with the consumer summing the slots, an all-reduce of partial outputs (row-parallel layers).

    A buffer that one exchange fills may be written again only after every rank has finished reading it.  The
    barrier of the NEXT exchange proves exactly that (a rank signals it after its own reads, in stream order),
    so two exchanges in a row must use different buffers, and a buffer is free again once another exchange
    has completed in between."""

    def __init__(self, sizes, group=None):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise QuantError(L.ERR_NOT_SUPPORTED, "PeerArena: at most 8 ranks (one NVSwitch node)")
        self.offsets, off = {}, 0
        for name, nbytes in sizes.items():
            self.offsets[name] = off
            off += -(-int(nbytes) // 256) * 256
        self.data_bytes = max(off, 256)
        lib = L.load()
        self.device = torch.device("cuda", torch.cuda.current_device())
        # The ranks walk through the same collectives whatever happens locally, and agree at the end on
        # whether every one of them mapped every buffer; then all raise or none does.
        own, handle, err = L.vp(), ctypes.create_string_buffer(64), None
        try:
            _check(lib.qb200_peer_alloc(self.data_bytes + 128, ctypes.byref(own), handle))
        except QuantError as e:
            err = e
        mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).to(self.device)
        every = torch.empty(self.world * 64, dtype=torch.uint8, device=self.device)
        dist.all_gather_into_tensor(every, mine, group=group)
        every = every.cpu().numpy().tobytes()
        self._own = own.value
        self.bases: List[int] = []
        for p in range(self.world):
            if p == self.rank:
                self.bases.append(self._own)
                continue
            ptr = L.vp()
            if err is None:
                try:
                    _check(lib.qb200_peer_open(every[64 * p: 64 * p + 64], ctypes.byref(ptr)))
                except QuantError as e:
                    err = e
            self.bases.append(ptr.value)
        ok = torch.tensor([0.0 if err is not None else 1.0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() == 0:
            for p, b in enumerate(self.bases):
                if b and p != self.rank:
                    lib.qb200_peer_close(b)
            dist.barrier(group=group)
            if self._own:
                lib.qb200_peer_free(self._own)
            self.bases = []
            raise QuantError(L.ERR_NOT_SUPPORTED, "PeerArena: a rank could not allocate or map the peer buffers"
                                                  + (f" ({err})" if err is not None else ""))
        self._bases_c = (L.vp * self.world)(*self.bases)
        self._flags_c = (L.vp * self.world)(*[b + self.data_bytes for b in self.bases])
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._lead = None

    def address(self, name: str, byte_offset: int = 0) -> int:
        """Device address of a byte of this rank's own copy of buffer `name`."""
        return self._own + self.offsets[name] + byte_offset

    def tensor(self, name: str, shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """This rank's copy of buffer `name` as a tensor (aliases the allocation)."""
        if dtype == torch.float32:
            return torch.as_tensor(_RawCuda(self.address(name), shape, "<f4"), device=self.device)
        if dtype == torch.bfloat16:
            return torch.as_tensor(_RawCuda(self.address(name), shape, "<i2"), device=self.device).view(torch.bfloat16)
        raise QuantError(L.ERR_INVALID_PARAM, "PeerArena: buffers are viewed as f32 or bf16")

    def push(self, layers: List[QuantizedLinear], xs: List[torch.Tensor], own_addresses: List[int], m: int,
             out_dtype: torch.dtype = torch.float32, fused_barrier: bool = True) -> None:
        """layers[i](xs[i]) -> `own_addresses[i]` (inside this rank's arena) and the same offset of every peer's
        arena, then the arrival barrier (inside the launch, or as a one-warp kernel after it)."""
        n = len(layers)
        lib = L.load()
        hs = (L.vp * n)(*[ql._h for ql in layers])
        xp = (L.vp * n)(*[x.data_ptr() for x in xs])
        yp = (L.vp * n)(*own_addresses)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _check(lib.qb200_qlinear_forward_many_gather(hs, n, xp, L.BF16, m, yp, L.F32 if out_dtype == torch.float32 else L.BF16,
                                                      self._bases_c, self._flags_c if fused_barrier else None,
                                                      self.world, self.rank, stream))
        if not fused_barrier:
            _check(lib.qb200_peer_signal_wait(self._flags_c, self.world, self.rank, self.status.data_ptr(), stream))
        self._lead = layers[0]

    # ---- pushed exchanges: self-validating 8-byte elements, no barrier (see qb200_qlinear_forward_many_push) ----

    def state_address(self) -> int:
        """This rank's 16-word state array (word 8: the exchanges it has launched)."""
        return self._own + self.data_bytes

    def push_pushed(self, layers: List[QuantizedLinear], xs: List[torch.Tensor], own_addresses: List[int], m: int,
                    slot_stride: int = 0) -> None:
        """layers[i](xs[i]) stored as {f32 bits, exchange number} elements at `own_addresses[i]` of this rank's arena and at
        the same offset of every peer's; the launch neither fences nor waits — the consumers poll the elements.  With
        `slot_stride` (bytes between the ranks' slots; every rank runs the same shapes) the launch itself polls its twins'
        rows before it ends: an all-gather that is complete when the launch is."""
        n = len(layers)
        hs = (L.vp * n)(*[ql._h for ql in layers])
        xp = (L.vp * n)(*[x.data_ptr() for x in xs])
        yp = (L.vp * n)(*own_addresses)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _check(L.load().qb200_qlinear_forward_many_push(hs, n, xp, L.BF16, m, yp, self._bases_c, self.world, self.rank,
                                                        self.state_address(), slot_stride, stream))
        self._lead = layers[0]

    def add_rmsnorm_pushed(self, h: torch.Tensor, name: str, parts: int, gamma: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
        """h += the `parts` pushed arrays of buffer `name` (summed in part order); returns bf16(rmsnorm(h) * gamma)."""
        n, c = h.shape
        _check(L.load().qb200_add_rmsnorm_pushed(h.data_ptr(), self.address(name), parts, self.state_address(), gamma.data_ptr(), n, c, eps,
                                                 out.data_ptr(), self.status.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream))
        return out

    def gather_pushed(self, name: str, parts: int, part_stride: int, rows: int, cols: int, dst: torch.Tensor) -> torch.Tensor:
        """Column shards of a `[rows, cols]` output pushed by the `parts` ranks into buffer `name` -> dense f32 `dst`."""
        _check(L.load().qb200_gather_pushed(self.address(name), parts, part_stride, rows, cols, self.state_address(), dst.data_ptr(),
                                            dst.stride(0), self.status.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream))
        return dst

    def check(self) -> None:
        """Synchronises and raises if a bounded wait of a barrier ran out."""
        if self._lead is not None:
            _check(L.load().qb200_qlinear_check(self._lead._h, torch.cuda.current_stream(self.device).cuda_stream))
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise QuantError(L.ERR_TIMEOUT, "PeerArena: a rank did not arrive within the barrier's poll limit")

    def close(self) -> None:
        if not self.bases:
            return
        lib = L.load()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody unmaps while a peer may still store
        for p, b in enumerate(self.bases):
            if p != self.rank:
                lib.qb200_peer_close(b)
        dist.barrier(group=self.group)
        lib.qb200_peer_free(self._own)
        self.bases = []


class PeerGather:
    """The fused all-gather of a group of column-sharded decode layers.

    Every rank owns TWO receive buffers ``[world, count, m, n_local]`` in a PeerArena and alternates between them
    call by call: a rank that has finished call s may start call s + 1 and store into its peers' buffers while a
    slower peer still reads the outputs of call s, so call s + 1 must not touch the buffer of call s; by the time
    call s + 2 reuses it, call s + 1 has shown that every rank is done reading.  Three mechanisms (``mode``):

    * ``"barrier"``: the kernel stores plain outputs and runs the arrival barrier in the same launch (or as a
      one-warp kernel after it, ``fused_barrier=False``); ``forward_many`` returns the receive buffer itself.
    * ``"pushed"``: the kernel pushes self-validating elements, and each of its CTAs then polls the same rows of its
      twins on the other ranks, so the launch ends when every rank's outputs are here — no fence, no flag, one launch.
      ``forward_many`` returns a strided f32 view of the receive buffer (the values of its 8-byte elements).
    * ``"pushed+gather"``: the kernel only pushes; a second small kernel polls the elements and writes the dense
      gathered outputs into a local buffer, which ``forward_many`` returns.

    Shapes the kernel does not take raise QuantError(NOT_SUPPORTED); callers fall back to ``TensorParallelLinear``."""

    def __init__(self, count: int, m: int, n_local: int, dtype: torch.dtype = torch.float32, group=None,
                 fused_barrier: bool = True, mode: str = "barrier"):
        if mode not in ("barrier", "pushed", "pushed+gather"):
            raise QuantError(L.ERR_INVALID_PARAM, f"PeerGather: unknown mode {mode!r}")
        self.fused_barrier, self.mode, self.pushed = fused_barrier, mode, mode != "barrier"
        if dtype not in (torch.float32, torch.bfloat16) or (self.pushed and dtype != torch.float32):
            raise QuantError(L.ERR_INVALID_PARAM, "PeerGather: outputs are f32 or bf16 (pushed: f32)")
        self.count, self.m, self.n_local, self.dtype = count, m, n_local, dtype
        self.item = 8 if self.pushed else 4 if dtype == torch.float32 else 2
        world = dist.get_world_size(group)
        self.slot_bytes = count * m * n_local * self.item
        self.arena = PeerArena({"g0": world * self.slot_bytes, "g1": world * self.slot_bytes}, group)
        self.world, self.rank, self.device = self.arena.world, self.arena.rank, self.arena.device
        self.dense = torch.empty((self.world, count, m, n_local), dtype=torch.float32, device=self.device) if mode == "pushed+gather" else None
        self.calls = 0

    def view(self, parity: Optional[int] = None) -> torch.Tensor:
        """The gathered outputs ``[world, count, m, n_local]`` of the last call (aliases the buffer)."""
        if self.mode == "pushed+gather":
            return self.dense
        parity = (self.calls - 1) & 1 if parity is None else parity
        shape = (self.world, self.count, self.m, self.n_local)
        if self.mode == "pushed":  # every other 32-bit word of the 8-byte elements
            return self.arena.tensor("g%d" % parity, shape + (2,), torch.float32)[..., 0]
        return self.arena.tensor("g%d" % parity, shape, self.dtype)

    def forward_many(self, layers: List[QuantizedLinear], xs: List[torch.Tensor], parity: Optional[int] = None) -> torch.Tensor:
        """Runs the call into buffer `parity` (default: alternating).  A caller that captures calls into a CUDA graph
        captures an even number of them, so that replays keep alternating."""
        if len(layers) != self.count or len(xs) != self.count:
            raise QuantError(L.ERR_INVALID_PARAM, f"PeerGather: built for {self.count} layers")
        parity = self.calls & 1 if parity is None else parity
        name = "g%d" % parity
        per_layer = self.m * self.n_local * self.item
        own = [self.arena.address(name, self.rank * self.slot_bytes + i * per_layer) for i in range(self.count)]
        self.calls += 1
        if self.mode == "pushed":
            self.arena.push_pushed(layers, xs, own, self.m, self.slot_bytes)
            return self.view(parity)
        if self.mode == "pushed+gather":
            elems = self.count * self.m * self.n_local
            self.arena.push_pushed(layers, xs, own, self.m)
            return self.arena.gather_pushed(name, self.world, elems, 1, self.world * elems, self.dense.view(1, -1)).view_as(self.dense)
        self.arena.push(layers, xs, own, self.m, self.dtype, self.fused_barrier)
        return self.view(parity)

    def check(self) -> None:
        self.arena.check()

    def close(self) -> None:
        self.arena.close()
