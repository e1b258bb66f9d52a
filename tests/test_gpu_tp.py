"""Column-sharded QuantizedLinear over 2 GPUs (NCCL), against the single-GPU forward.
Runs as child processes; skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    import quanta_b200 as qb
    from quanta_b200 import tp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ok = True
        for N, K, dt, gran in [(4096, 1024, qb.QuantDtype.Int4, qb.Group(1, 128)), (200, 256, qb.QuantDtype.Int8, qb.Block(32, 32))]:
            gen = torch.Generator(device=dev).manual_seed(5)
            w = torch.randn(N, K, device=dev, generator=gen) * 0.02
            b = torch.randn(N, device=dev, generator=gen)
            qm = qb.QuantizedMatrix.quantize(w, dt, gran)
            full = qb.QuantizedLinear.new(qm, b, qb.OUT_IN)
            tpl = tp.TensorParallelLinear.new(qm, b)
            for M in (1, 16, 128):
                x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
                want = full.forward(x, out_dtype=torch.float32)
                got = tpl.forward(x, out_dtype=torch.float32)
                ok = ok and got.shape == want.shape and bool(((got - want).abs() <= 1e-4 * (1 + want.abs())).all())
            rpl = tp.RowParallelLinear.new(qm, b)  # input features sharded, partial outputs summed
            for M in (1, 16, 128):
                x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
                want = full.forward(x, out_dtype=torch.float32)
                got = rpl.forward(x)
                sliced = rpl.forward(x[:, rpl.lo: rpl.hi].contiguous(), sliced=True)
                ok = ok and got.shape == want.shape and bool(((got - want).abs() <= 1e-4 * (1 + want.abs())).all())
                ok = ok and bool(torch.equal(got, sliced))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_linear_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert ret.get(0) and ret.get(1)


def _gather_worker(rank, world, port, ret):
    import torch.distributed as dist

    import quanta_b200 as qb
    from quanta_b200 import tp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ok = True
        K, n_local, count = 1024, 512, 3
        gen = torch.Generator(device=dev).manual_seed(100 + rank)  # every rank owns different shards
        layers = []
        for _ in range(count):
            w = torch.randn(n_local, K, device=dev, generator=gen) * 0.02
            b = torch.randn(n_local, device=dev, generator=gen)
            layers.append(qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128)), b, qb.OUT_IN))
        for M in (1, 4, 8):
            xg = torch.Generator(device=dev).manual_seed(7 + M)  # the same activations on every rank
            x = torch.randn(M, K, device=dev, generator=xg).to(torch.bfloat16)
            own = torch.stack([ql.forward(x, out_dtype=torch.float32) for ql in layers])  # [count, M, n_local]
            want = torch.empty(world, count, M, n_local, device=dev)
            dist.all_gather_into_tensor(want, own)  # the collective the fused path replaces
            for fused_barrier in (True, False):  # the barrier inside the launch, or as its own kernel
                pg = tp.PeerGather(count, M, n_local, torch.float32, fused_barrier=fused_barrier)
                for _ in range(3):  # the barrier counts steps: repeated use must keep working
                    got = pg.forward_many(layers, [x] * count)
                pg.check()
                ok = ok and layers[0].last_kernel() == "gemv_mma_grouped_gather" and torch.equal(got, want)
                pg.close()
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_all_gather_two_gpus():
    """The decode kernel's peer stores plus the arrival barrier against NCCL's all-gather of the same outputs."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert ret.get(0) and ret.get(1)
