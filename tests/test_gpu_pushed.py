"""Pushed exchanges (self-validating 8-byte elements, no barrier) on ONE GPU: the two "ranks" are two sets of
shards and two local arenas; their producer launches run one after the other on the stream (no kernel ever waits
for another launch), each storing its part into both arenas, and the consumers then find every element stamped
with the exchange number they expect.  Also: a rank that never pushes makes the consumer give up after a few
milliseconds with QB200_ERR_TIMEOUT, and the context stays usable."""
import numpy as np
import pytest
import torch

import quanta_b200 as qb
from quanta_b200 import _lib
from quanta_b200.decoder import add_rmsnorm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layers(n_out, k, count, seed, bias=True):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    out = []
    for _ in range(count):
        w = torch.randn(n_out, k, device=DEV, generator=gen) * 0.02
        b = torch.randn(n_out, device=DEV, generator=gen) if bias else None
        out.append(qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128)), b, qb.OUT_IN))
    return out


class _Rank:
    """One emulated rank: its arena (a plain local allocation), its state array and its status word."""

    def __init__(self, nbytes):
        self.arena = torch.zeros(nbytes // 8, dtype=torch.int64, device=DEV)
        self.state = torch.zeros(16, dtype=torch.int64, device=DEV)
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)


def _push(lib, ranks, r, layers, xs, offsets, m, slot_stride=0):
    n = len(layers)
    hs = (_lib.vp * n)(*[ql._h for ql in layers])
    xp = (_lib.vp * n)(*[x.data_ptr() for x in xs])
    yp = (_lib.vp * n)(*[ranks[r].arena.data_ptr() + o for o in offsets])
    bases = (_lib.vp * len(ranks))(*[k.arena.data_ptr() for k in ranks])
    st = lib.qb200_qlinear_forward_many_push(hs, n, xp, _lib.BF16, m, yp, bases, len(ranks), r, ranks[r].state.data_ptr(), slot_stride,
                                             torch.cuda.current_stream().cuda_stream)
    assert st == 0, _lib.last_error()


@pytest.mark.parametrize("M", [1, 6, 16])
def test_row_parallel_partials_pushed_and_summed(M):
    lib = _lib.load()
    d, k_local, world, slices = 768, 512, 2, 2
    part = M * d * 8
    ranks = [_Rank(world * slices * part) for _ in range(world)]
    shards = [_layers(d, k_local, slices, 50 + r, bias=False) for r in range(world)]
    gen = torch.Generator(device=DEV).manual_seed(9)
    gamma = torch.randn(d, device=DEV, generator=gen)
    for step in range(3):  # the exchange number moves on with every push
        xs = [[torch.randn(M, k_local, device=DEV, generator=gen).to(torch.bfloat16) for _ in range(slices)] for _ in range(world)]
        h0 = torch.randn(M, d, device=DEV, generator=gen)
        for r in range(world):
            _push(lib, ranks, r, shards[r], xs[r], [(r * slices + s) * part for s in range(slices)], M)
        assert shards[0][0].last_kernel() == "gemv_mma_grouped_push"
        # reference: the same launches storing plain f32, summed by the plain add + RMSNorm in the same order
        plain = torch.stack([y for r in range(world) for y in qb.QuantizedLinear.forward_many(shards[r], xs[r], out_dtype=torch.float32)])
        h_want = h0.clone()
        out_want = add_rmsnorm(h_want, plain, gamma, 1e-5)
        for r in range(world):
            h = h0.clone()
            out = torch.empty(M, d, dtype=torch.bfloat16, device=DEV)
            st = lib.qb200_add_rmsnorm_pushed(h.data_ptr(), ranks[r].arena.data_ptr(), world * slices, ranks[r].state.data_ptr(),
                                              gamma.data_ptr(), M, d, 1e-5, out.data_ptr(), ranks[r].status.data_ptr(),
                                              torch.cuda.current_stream().cuda_stream)
            assert st == 0, _lib.last_error()
            torch.cuda.synchronize()
            assert int(ranks[r].status.item()) == 0
            assert int(ranks[r].state[8].item()) == step + 1
            assert torch.equal(h, h_want) and torch.equal(out, out_want)   # same values, same order of sums: bit for bit
    assert lib.qb200_qlinear_check(shards[0][0]._h, None) == 0


def test_column_shards_pushed_and_gathered_ragged():
    lib = _lib.load()
    M, K, vocab, world = 5, 256, 1001, 3      # shards of 334, 334, 333 rows
    base, extra = divmod(vocab, world)
    v_max = base + 1
    ranks = [_Rank(world * M * v_max * 8) for _ in range(world)]
    gen = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(M, K, device=DEV, generator=gen).to(torch.bfloat16)
    want = torch.empty(M, vocab, device=DEV)
    lo = 0
    for r in range(world):
        w = base + (1 if r < extra else 0)
        ql = _layers(w, K, 1, 70 + r)[0]
        _push(lib, ranks, r, [ql], [x], [r * M * v_max * 8], M)
        want[:, lo:lo + w] = ql.forward(x, out_dtype=torch.float32)
        lo += w
    for r in range(world):
        dst = torch.full((M, vocab + 3), float("nan"), device=DEV)   # a padded destination: rows 1004 floats apart
        st = lib.qb200_gather_pushed(ranks[r].arena.data_ptr(), world, M * v_max, M, vocab, ranks[r].state.data_ptr(), dst.data_ptr(),
                                     dst.stride(0), ranks[r].status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert st == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert int(ranks[r].status.item()) == 0 and torch.equal(dst[:, :vocab], want) and bool(torch.isnan(dst[:, vocab:]).all())


def test_consumer_gives_up_on_a_rank_that_never_pushes():
    lib = _lib.load()
    assert lib.qb200_peer_set_spin_limit(3000) == 0
    try:
        M, d, k_local, world = 4, 512, 256, 2
        part = M * d * 8
        ranks = [_Rank(world * part) for _ in range(world)]
        ql = _layers(d, k_local, 1, 5, bias=False)[0]
        x = torch.randn(M, k_local, device=DEV).to(torch.bfloat16)
        _push(lib, ranks, 0, [ql], [x], [0], M)            # rank 1 never pushes
        h = torch.zeros(M, d, device=DEV)
        gamma = torch.ones(d, device=DEV)
        out = torch.empty(M, d, dtype=torch.bfloat16, device=DEV)
        st = lib.qb200_add_rmsnorm_pushed(h.data_ptr(), ranks[0].arena.data_ptr(), world, ranks[0].state.data_ptr(), gamma.data_ptr(), M, d,
                                          1e-5, out.data_ptr(), ranks[0].status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()
        assert int(ranks[0].status.item()) == _lib.ERR_TIMEOUT
        # the missing part counted as zeros: h holds rank 0's part alone
        assert torch.equal(h, ql.forward(x, out_dtype=torch.float32))
        ranks[0].status.zero_()
        assert torch.isfinite(ql.forward(x, out_dtype=torch.float32)).all()   # the context is intact
    finally:
        assert lib.qb200_peer_set_spin_limit(4 << 20) == 0


@pytest.mark.parametrize("M", [1, 5, 16])
def test_all_gather_checked_inside_the_launch(M):
    """slot_stride > 0: the launch polls its twins' rows before it ends.  On one GPU the twin cannot run at the same
    time, so rank 1 pushes first (without waiting) and rank 0's launch then finds rank 1's elements in place; a rank 0
    whose twin never pushed gives up after a few milliseconds and the handle reports it once."""
    lib = _lib.load()
    n_local, K, count, world = 200, 512, 2, 2
    slot = count * M * n_local * 8
    ranks = [_Rank(world * slot) for _ in range(world)]
    shards = [_layers(n_local, K, count, 80 + r) for r in range(world)]
    x = torch.randn(M, K, device=DEV, generator=torch.Generator(device=DEV).manual_seed(2)).to(torch.bfloat16)
    offs = lambda r: [r * slot + i * M * n_local * 8 for i in range(count)]
    _push(lib, ranks, 1, shards[1], [x] * count, offs(1), M)                    # the twin's elements, exchange 1
    _push(lib, ranks, 0, shards[0], [x] * count, offs(0), M, slot_stride=slot)  # pushes and checks
    torch.cuda.synchronize()
    assert lib.qb200_qlinear_check(shards[0][0]._h, None) == 0
    want = torch.stack([torch.stack(qb.QuantizedLinear.forward_many(shards[r], [x] * count, out_dtype=torch.float32)) for r in range(world)])
    for k in ranks:   # both arenas hold both ranks' outputs; the values are every other 32-bit word
        got = k.arena.view(torch.float32).view(world, count, M, n_local, 2)[..., 0]
        assert torch.equal(got, want)
    assert lib.qb200_peer_set_spin_limit(3000) == 0
    try:
        _push(lib, ranks, 0, shards[0], [x] * count, offs(0), M, slot_stride=slot)  # exchange 2: the twin never pushes it
        torch.cuda.synchronize()
        assert lib.qb200_qlinear_check(shards[0][0]._h, None) == _lib.ERR_TIMEOUT
        assert lib.qb200_qlinear_check(shards[0][0]._h, None) == 0
    finally:
        assert lib.qb200_peer_set_spin_limit(4 << 20) == 0


def test_push_refuses_what_the_decode_kernel_does_not_take():
    lib = _lib.load()
    ranks = [_Rank(1 << 20)]
    w = torch.randn(64, 256, device=DEV) * 0.02
    q8 = qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int8, qb.PerChannel(0)), None, qb.OUT_IN)
    x = torch.randn(2, 256, device=DEV).to(torch.bfloat16)
    hs, xp = (_lib.vp * 1)(q8._h), (_lib.vp * 1)(x.data_ptr())
    yp, bases = (_lib.vp * 1)(ranks[0].arena.data_ptr()), (_lib.vp * 1)(ranks[0].arena.data_ptr())
    st = lib.qb200_qlinear_forward_many_push(hs, 1, xp, _lib.BF16, 2, yp, bases, 1, 0, ranks[0].state.data_ptr(), 0, None)
    assert st == _lib.ERR_NOT_SUPPORTED and "decode kernel" in _lib.last_error()
    st = lib.qb200_qlinear_forward_many_push(hs, 1, xp, _lib.BF16, 2, yp, bases, 1, 3, ranks[0].state.data_ptr(), 0, None)
    assert st == _lib.ERR_INVALID_PARAM
