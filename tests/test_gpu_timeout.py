"""Bounded device-side waits: a wait that nothing satisfies runs out of polls, the kernel returns, the status word
reads QB200_ERR_TIMEOUT and the context stays usable.  One GPU: both ranks' barrier state and gather buffers are
local allocations, and the second rank simply never launches, so its flag is never set (no kernel waits on another
launch here: the only waiter is the launch under test, and its wait is limited to a few milliseconds)."""
import ctypes

import numpy as np
import pytest
import torch

import quanta_b200 as qb
from quanta_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHORT = 4000  # polls of about a quarter of a microsecond: a few milliseconds


@pytest.fixture()
def short_spin():
    lib = _lib.load()
    assert lib.qb200_peer_set_spin_limit(SHORT) == 0
    yield lib
    assert lib.qb200_peer_set_spin_limit(4 << 20) == 0


def test_spin_limit_setter_rejects_zero():
    lib = _lib.load()
    assert lib.qb200_peer_set_spin_limit(0) == _lib.ERR_INVALID_PARAM
    assert "positive" in _lib.last_error()


def test_peer_barrier_times_out_when_a_rank_never_arrives(short_spin):
    lib = short_spin
    flags = [torch.zeros(16, dtype=torch.int64, device=DEV) for _ in range(2)]
    arr = (_lib.vp * 2)(*[f.data_ptr() for f in flags])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    # rank 0 publishes its arrival to both ranks and waits for rank 1, which never launches
    assert lib.qb200_peer_signal_wait(arr, 2, 0, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.ERR_TIMEOUT
    assert flags[0][0].item() == 1 and flags[1][0].item() == 1 and flags[0][8].item() == 1  # its own side of the barrier ran
    assert flags[0][1].item() == 0
    # the context is intact: rank 1's launch now finds rank 0's flag and completes without a timeout
    status.zero_()
    assert lib.qb200_peer_signal_wait(arr, 2, 1, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and flags[0][1].item() == 1 and flags[1][1].item() == 1


@pytest.mark.parametrize("M", [1, 8, 16])
def test_fused_exchange_stores_both_buffers_and_reports_a_missing_rank(short_spin, M):
    """The decode kernel with peer stores, both "ranks'" buffers on this GPU: every output lands in both buffers and
    equals the plain grouped forward bit for bit; the in-launch barrier gives up on the rank that never arrives and
    qb200_qlinear_check reports it once."""
    lib = short_spin
    K, n_local, count = 1024, 384, 3
    gen = torch.Generator(device=DEV).manual_seed(11)
    layers = []
    for _ in range(count):
        w = torch.randn(n_local, K, device=DEV, generator=gen) * 0.02
        b = torch.randn(n_local, device=DEV, generator=gen)
        layers.append(qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128)), b, qb.OUT_IN))
    x = torch.randn(M, K, device=DEV, generator=gen).to(torch.bfloat16)
    want = torch.stack(qb.QuantizedLinear.forward_many(layers, [x] * count, out_dtype=torch.float32))
    bufs = [torch.zeros(2, count, M, n_local, device=DEV) for _ in range(2)]   # [rank slot][layer][m][n] per "rank"
    flags = [torch.zeros(16, dtype=torch.int64, device=DEV) for _ in range(2)]
    hs = (_lib.vp * count)(*[ql._h for ql in layers])
    xp = (_lib.vp * count)(*[x.data_ptr()] * count)
    yp = (_lib.vp * count)(*[bufs[0][0, i].data_ptr() for i in range(count)])  # rank 0's slot of its own buffer
    bases = (_lib.vp * 2)(*[b.data_ptr() for b in bufs])
    fl = (_lib.vp * 2)(*[f.data_ptr() for f in flags])
    stream = torch.cuda.current_stream().cuda_stream
    st = lib.qb200_qlinear_forward_many_gather(hs, count, xp, _lib.BF16, M, yp, _lib.F32, bases, fl, 2, 0, stream)
    assert st == 0, _lib.last_error()
    assert layers[0].last_kernel() == "gemv_mma_grouped_gather"
    torch.cuda.synchronize()
    assert torch.equal(bufs[0][0], want) and torch.equal(bufs[1][0], want)
    assert float(bufs[0][1].abs().max()) == 0.0 and float(bufs[1][1].abs().max()) == 0.0  # rank 1's slots untouched
    assert lib.qb200_qlinear_check(layers[0]._h, stream) == _lib.ERR_TIMEOUT   # rank 1 never arrived
    assert "wait ran out" in _lib.last_error()
    assert lib.qb200_qlinear_check(layers[0]._h, stream) == 0                  # reported once
    # without flag arrays the launch stores and returns; nothing waits
    for b in bufs:
        b.zero_()
    st = lib.qb200_qlinear_forward_many_gather(hs, count, xp, _lib.BF16, M, yp, _lib.F32, bases, None, 2, 0, stream)
    assert st == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.equal(bufs[0][0], want) and torch.equal(bufs[1][0], want)
    assert lib.qb200_qlinear_check(layers[0]._h, stream) == 0
