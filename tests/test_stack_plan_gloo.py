"""Host-side logic of the tensor-parallel decoder stack on CPU ranks (gloo): the shard maps of `StackPlan`
(whole heads, whole scale groups, vocabulary rows), the slot addressing of the exchange buffers, and the
arithmetic of the two exchanges of a block — row-parallel partial outputs summed over slots equal the unsharded
layer — emulated with the oracle's dequantize and an all_gather in place of the kernels' peer stores."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as o
import quanta_b200 as qb
from quanta_b200 import decoder as dec


def test_shard_units_cover_once_and_differ_by_at_most_one():
    for units, world in [(32, 8), (86, 8), (86, 4), (86, 2), (86, 1), (32000, 8), (5, 4), (7, 7)]:
        spans = [dec.shard_units(units, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == units
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_stack_plan_llama7b_shape(world):
    plans = [dec.StackPlan.make(world, r, 4096, 32, 11008, 32000, 16) for r in range(world)]
    # whole heads, contiguous, covering d; whole scale groups covering the FFN width; vocabulary rows
    assert [p.q_lo for p in plans] == [r * 4096 // world for r in range(world)] and plans[-1].q_hi == 4096
    assert plans[0].f_lo == 0 and plans[-1].f_hi == 11008 and all(a.f_hi == b.f_lo for a, b in zip(plans, plans[1:]))
    assert all(p.f_lo % 128 == 0 and p.f_hi % 128 == 0 for p in plans)
    assert plans[0].v_lo == 0 and plans[-1].v_hi == 32000
    for p in plans:
        # the same number of down slices of one padded width on every rank; each at most 4096 inputs
        assert p.down_slices == plans[0].down_slices and p.down_pad == plans[0].down_pad
        assert sum(p.down_widths) == p.f_hi - p.f_lo and len(p.down_widths) == p.down_slices
        assert all(w % 128 == 0 and w <= p.down_pad <= 4096 for w in p.down_widths) and p.down_pad % 512 == 0
        # slots: the same layout on every rank, disjoint, inside the buffers
        sizes = p.arena_sizes()
        assert sizes == plans[0].arena_sizes()
        o_slots = [p.o_offset(r) for r in range(world)]
        d_slots = [p.d_offset(r, s) for r in range(world) for s in range(p.down_slices)]
        part = 16 * 4096 * p.ELEM
        assert o_slots == [i * part for i in range(world)] and o_slots[-1] + part == sizes["o"]
        assert d_slots == [i * part for i in range(world * p.down_slices)] and d_slots[-1] + part == sizes["d"]
        assert p.v_offset(world - 1) + 16 * p.v_max * p.ELEM == sizes["v"] and p.v_max >= p.v_hi - p.v_lo
    if world == 1:
        assert plans[0].down_widths == (3712, 3712, 3584) and plans[0].down_pad == 4096
    if world == 8:
        assert [p.f_hi - p.f_lo for p in plans] == [1408] * 6 + [1280] * 2 and plans[0].down_pad == 1536


def test_stack_plan_rejects_bad_shapes():
    for args in [(3, 0, 4096, 32, 11008, 32000, 16), (2, 2, 4096, 32, 11008, 32000, 16), (2, 0, 4096, 32, 11000, 32000, 16),
                 (8, 0, 512, 4, 512, 100, 1)]:
        with pytest.raises(qb.QuantError):
            dec.StackPlan.make(*args)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, heads, ffn, vocab, batch = 512, 4, 1280, 101, 3
        p = dec.StackPlan.make(world, rank, d, heads, ffn, vocab, batch)
        rng = np.random.default_rng(21)  # the same full weights on every rank
        w_o = (rng.standard_normal((d, d)) * 0.02).astype(np.float32)
        w_d = (rng.standard_normal((d, ffn)) * 0.02).astype(np.float32)
        w_v = (rng.standard_normal((vocab, d)) * 0.02).astype(np.float32)
        att = rng.standard_normal((batch, d)).astype(np.float32)
        act = rng.standard_normal((batch, ffn)).astype(np.float32)
        xn = rng.standard_normal((batch, d)).astype(np.float32)

        def deq(w):
            c, s = o.quantize_host(w, w.shape[0], w.shape[1], 4, 1, 128)
            return o.dequantize_host(c, s, w.shape[0], w.shape[1], 4, 1, 128)

        dq_o, dq_d, dq_v = deq(w_o), deq(w_d), deq(w_v)
        # exchange 1: the output projection over this rank's heads -> slot `rank` of buffer "o"; sum of slots
        buf_o = np.zeros(p.arena_sizes()["o"] // p.ELEM, np.float32)
        part = att[:, p.q_lo:p.q_hi] @ dq_o[:, p.q_lo:p.q_hi].T
        lo = p.o_offset(rank) // p.ELEM
        mine = torch.from_numpy(part.reshape(-1).copy())
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        for r in range(world):  # what the peers' stores put into this rank's buffer
            buf_o[p.o_offset(r) // p.ELEM: p.o_offset(r) // p.ELEM + mine.numel()] = every[r].numpy()
        assert np.array_equal(buf_o[lo: lo + mine.numel()], mine.numpy())
        got = buf_o.reshape(world, batch, d).sum(0)
        ok = np.allclose(got, att @ dq_o.T, rtol=1e-5, atol=1e-6)
        # exchange 2: the down projection over this rank's FFN columns, in padded slices
        buf_d = np.zeros(p.arena_sizes()["d"] // p.ELEM, np.float32)
        parts, c0 = [], p.f_lo
        for w in p.down_widths:
            xs = np.zeros((batch, p.down_pad), np.float32)
            ws = np.zeros((d, p.down_pad), np.float32)
            xs[:, :w], ws[:, :w] = act[:, c0:c0 + w], dq_d[:, c0:c0 + w]
            parts.append(xs @ ws.T)
            c0 += w
        assert c0 == p.f_hi
        mine = torch.from_numpy(np.stack(parts).reshape(-1).copy())
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        for r in range(world):
            a0 = p.d_offset(r, 0) // p.ELEM
            buf_d[a0: a0 + mine.numel()] = every[r].numpy()
        got = buf_d.reshape(world * p.down_slices, batch, d).sum(0)
        ok = ok and np.allclose(got, act @ dq_d.T, rtol=1e-5, atol=1e-5)
        # the logits: ragged vocabulary shards packed [batch, rows of rank r] in slot r
        buf_v = np.zeros(p.arena_sizes()["v"] // p.ELEM, np.float32)
        mine = np.zeros(batch * p.v_max, np.float32)
        mine[: batch * (p.v_hi - p.v_lo)] = (xn @ dq_v[p.v_lo:p.v_hi].T).reshape(-1)
        mine = torch.from_numpy(mine)
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        logits = np.zeros((batch, vocab), np.float32)
        for r in range(world):
            buf_v[p.v_offset(r) // p.ELEM: p.v_offset(r) // p.ELEM + mine.numel()] = every[r].numpy()
            lo_r, hi_r = dec.shard_units(vocab, world, r)
            slot = buf_v[p.v_offset(r) // p.ELEM:]
            logits[:, lo_r:hi_r] = slot[: batch * (hi_r - lo_r)].reshape(batch, hi_r - lo_r)
        ok = ok and np.allclose(logits, xn @ dq_v.T, rtol=1e-5, atol=1e-6)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_exchanges_of_a_block_on_cpu_ranks(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(180)
        assert pr.exitcode == 0
    assert all(ret.get(r) for r in range(world))
