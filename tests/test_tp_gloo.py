"""Host-side logic of the column-sharded path on CPU ranks (gloo, world size 2 and 3):
shard boundaries, shard views of codes / scales, and the all-gather reassembly, checked
against the oracle's full forward."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as o
import quanta_b200 as qb
from quanta_b200 import tp


def test_shard_range_covers_rows_once():
    for out_dim, world, mult in [(4096, 8, 1), (11008, 8, 32), (100, 3, 32), (37, 4, 1), (64, 8, 32), (5, 8, 1)]:
        seen = []
        for r in range(world):
            lo, hi = tp.shard_range(out_dim, world, r, mult)
            assert lo % mult == 0 or lo == out_dim
            seen += list(range(lo, hi))
        assert seen == list(range(out_dim))
    with pytest.raises(qb.QuantError):
        tp.shard_range(10, 2, 2)


def test_shard_cols_keeps_tiles_and_packed_words_whole():
    from quanta_b200 import _lib
    import ctypes
    lib = _lib.load()
    for cols, gc, bits, world in [(11008, 128, 4, 8), (4096, 32, 8, 4), (100, 4, 4, 3), (64, 3, 4, 2), (64, 3, 8, 2)]:
        seen, mult = [], gc if bits == 8 or gc % 8 == 0 else np.lcm(gc, 8)
        for r in range(world):
            lo, hi = _lib.u64(), _lib.u64()
            assert lib.qb200_shard_cols(cols, gc, bits, world, r, ctypes.byref(lo), ctypes.byref(hi)) == 0
            assert lo.value % mult == 0 or lo.value == cols
            seen += list(range(lo.value, hi.value))
        assert seen == list(range(cols))
    lo, hi = _lib.u64(), _lib.u64()
    assert lib.qb200_shard_cols(64, 0, 4, 2, 0, ctypes.byref(lo), ctypes.byref(hi)) == _lib.ERR_INVALID_PARAM
    assert lib.qb200_shard_rows(64, 1, 2, 2, ctypes.byref(lo), ctypes.byref(hi)) == _lib.ERR_INVALID_PARAM
    assert "outside a world" in _lib.last_error()


def test_tp_create_validates_before_touching_a_device():
    from quanta_b200 import _lib
    import ctypes
    lib = _lib.load()
    h = _lib.vp()
    assert lib.qb200_tp_create(3, 2, None, ctypes.byref(h)) == _lib.ERR_INVALID_PARAM and not h.value
    assert lib.qb200_tp_create(0, 2, None, ctypes.byref(h)) == _lib.ERR_INVALID_PARAM and "unique id" in _lib.last_error()
    assert lib.qb200_qlinear_forward_tp(None, None, 0, 8, 1, None, 0, 1, None, 0, None) == _lib.ERR_INVALID_PARAM


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, N, K, bits, gr, gc, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(11)
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        x = rng.standard_normal((3, K)).astype(np.float32)
        codes, scales = o.quantize_host(w, N, K, bits, gr, gc)
        ct = torch.from_numpy(codes if bits == 8 else codes.view(np.int32))
        gran = qb.granularity_from_grid(N, K, gr, gc, allow_block=True)
        full = qb.QuantizedMatrix.from_parts(ct, [N, K], torch.from_numpy(scales), gran)
        lo, hi = tp.shard_range(N, world, rank, gr)
        want = o.linear_forward(x, o.dequantize_host(codes, scales, N, K, bits, gr, gc), None, o.OUT_IN)
        if hi > lo:
            sh = tp.shard_matrix(full, world, rank)
            sc = sh.codes().numpy()
            sc = sc if bits == 8 else sc.view(np.uint32)
            assert sh.shape() == [hi - lo, K]
            wd = o.dequantize_host(sc, sh.scales().numpy(), hi - lo, K, bits, sh.tile()[0], gc)
            y_local = torch.from_numpy(o.linear_forward(x, wd, None, o.OUT_IN))
        else:
            y_local = torch.empty((3, 0))
        y = tp.gather_columns(y_local, N, multiple=gr)
        ok = y.shape == (3, N) and bool((y.numpy().view(np.uint32) == want.view(np.uint32)).all())
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,N,K,bits,gr,gc", [(2, 64, 256, 4, 1, 128), (2, 96, 64, 8, 32, 32), (3, 100, 128, 4, 1, 128),
                                                  (3, 64, 64, 8, 32, 32)])
def test_sharded_forward_matches_full_forward(world, N, K, bits, gr, gc):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, N, K, bits, gr, gc, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)


def _row_worker(rank, world, port, N, K, bits, gr, gc, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(13)
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        x = rng.standard_normal((3, K)).astype(np.float32)
        codes, scales = o.quantize_host(w, N, K, bits, gr, gc)
        ct = torch.from_numpy(codes if bits == 8 else codes.view(np.int32))
        gran = qb.granularity_from_grid(N, K, gr, gc, allow_block=True)
        full = qb.QuantizedMatrix.from_parts(ct, [N, K], torch.from_numpy(scales), gran)
        wd = o.dequantize_host(codes, scales, N, K, bits, gr, gc)
        want = o.linear_forward_f64(x, wd, None, o.OUT_IN)
        sh, lo, hi = tp.shard_columns(full, world, rank)
        ok = lo % gc == 0 or lo == K
        if sh is not None:
            sc = sh.codes().numpy()
            sc = sc if bits == 8 else sc.view(np.uint32)
            part = o.dequantize_host(sc, sh.scales().numpy(), N, hi - lo, bits, gr, sh.tile()[1])
            ok = ok and np.array_equal(part.view(np.uint32), np.ascontiguousarray(wd[:, lo:hi]).view(np.uint32))  # the shard IS the block
            y = torch.from_numpy(o.linear_forward(np.ascontiguousarray(x[:, lo:hi]), part, None, o.OUT_IN))
        else:
            y = torch.zeros((3, N))
        dist.all_reduce(y)  # what RowParallelLinear.forward does with the local outputs
        ok = ok and bool((np.abs(y.numpy() - want) <= 1e-4 * (1 + np.abs(want))).all())
        cover = torch.zeros(K)
        cover[lo:hi] = 1
        dist.all_reduce(cover)
        ret[rank] = ok and bool((cover == 1).all())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,N,K,bits,gr,gc", [(2, 48, 512, 4, 1, 128), (3, 40, 384, 4, 1, 128), (2, 64, 96, 8, 32, 32),
                                                  (3, 32, 128, 8, 1, 128)])
def test_row_parallel_shards_sum_to_the_full_forward(world, N, K, bits, gr, gc):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_row_worker, args=(r, world, port, N, K, bits, gr, gc, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)
