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
        comm = tp.TpComm()   # the library's own NCCL communicator behind the C ABI
        for N, K, dt, gran in [(4096, 1024, qb.QuantDtype.Int4, qb.Group(1, 128)), (200, 256, qb.QuantDtype.Int8, qb.Block(32, 32))]:
            gen = torch.Generator(device=dev).manual_seed(5)
            w = torch.randn(N, K, device=dev, generator=gen) * 0.02
            b = torch.randn(N, device=dev, generator=gen)
            qm = qb.QuantizedMatrix.quantize(w, dt, gran)
            full = qb.QuantizedLinear.new(qm, b, qb.OUT_IN)
            tpl = tp.TensorParallelLinear.new(qm, b)
            tplc = tp.TensorParallelLinear.new(qm, b, comm=comm)   # the same through qb200_qlinear_forward_tp
            for M in (1, 16, 128):
                x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
                want = full.forward(x, out_dtype=torch.float32)
                got = tpl.forward(x, out_dtype=torch.float32)
                ok = ok and got.shape == want.shape and bool(((got - want).abs() <= 1e-4 * (1 + want.abs())).all())
                gotc = tplc.forward(x, out_dtype=torch.float32)
                ok = ok and torch.equal(gotc, got)   # the same shard kernels; the collective only moves bytes
                gotb = tplc.forward(x, out_dtype=torch.bfloat16)
                ok = ok and bool(((gotb.float() - want).abs() <= 1e-2 * (1 + want.abs())).all())
            rpl = tp.RowParallelLinear.new(qm, b)  # input features sharded, partial outputs summed
            rplc = tp.RowParallelLinear.new(qm, b, comm=comm)
            for M in (1, 16, 128):
                x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
                want = full.forward(x, out_dtype=torch.float32)
                got = rpl.forward(x)
                sliced = rpl.forward(x[:, rpl.lo: rpl.hi].contiguous(), sliced=True)
                ok = ok and got.shape == want.shape and bool(((got - want).abs() <= 1e-4 * (1 + want.abs())).all())
                ok = ok and bool(torch.equal(got, sliced))
                gotc = rplc.forward(x)
                ok = ok and bool(((gotc - want).abs() <= 1e-4 * (1 + want.abs())).all())
        comm.close()
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
        for M in (1, 4, 8, 11, 16):
            xg = torch.Generator(device=dev).manual_seed(7 + M)  # the same activations on every rank
            xs = [torch.randn(M, K, device=dev, generator=xg).to(torch.bfloat16) for _ in range(5)]  # another x every step
            wants = []
            for x in xs:
                own = torch.stack([ql.forward(x, out_dtype=torch.float32) for ql in layers])  # [count, M, n_local]
                want = torch.empty(world, count, M, n_local, device=dev)
                dist.all_gather_into_tensor(want, own)  # the collective the fused path replaces
                wants.append(want)
            # the barrier inside the launch, the barrier as its own kernel, pushed elements validated by the launch itself,
            # or pushed elements and a polling consumer kernel
            for fused_barrier, mode in ((True, "barrier"), (False, "barrier"), (True, "pushed"), (True, "pushed+gather")):
                pushed = mode != "barrier"
                pg = tp.PeerGather(count, M, n_local, torch.float32, fused_barrier=fused_barrier, mode=mode)
                # every step's gathered buffer is read while the next step may already be storing into the peers:
                # the two receive buffers used in turn keep a step's outputs intact until they have been compared
                gots = []
                for x in xs:  # the barrier counts steps: repeated use must keep working
                    gots.append(pg.forward_many(layers, [x] * count).clone())
                pg.check()
                ok = ok and layers[0].last_kernel() == ("gemv_mma_grouped_push" if pushed else "gemv_mma_grouped_gather")
                ok = ok and all(torch.equal(g, w) for g, w in zip(gots, wants))
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


def _stack_worker(rank, world, port, ret):
    import torch.distributed as dist

    from quanta_b200 import decoder as dec
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # a small Llama-shaped stack: 8 heads of 128, FFN of 21 scale groups (ragged over 2 ranks), ragged vocabulary
        args = dict(n_layers=2, d=1024, heads=8, ffn=2688, vocab=1001, batch=16, ctx_max=65, device=dev, seed=4)
        single = dec.DecoderStack(**args)
        sharded = dec.DecoderStack(**args, group=dist.group.WORLD)
        h0 = torch.randn(16, 1024, device=dev, generator=torch.Generator(device=dev).manual_seed(3)) * 0.5
        ok = True
        for pos in (63, 64):
            single.set_position(pos)
            sharded.set_position(pos)
            want = single.step(h0).clone()
            got = sharded.step(h0).clone()
            sharded.arena.check()
            # the same codes and scales, the f32 sums over ranks in another order; logits are O(1)
            ok = ok and bool(((got - want).abs() <= 1e-2 * (1 + want.abs())).all())
            ref = got.clone()
            dist.broadcast(ref, 0)
            ok = ok and torch.equal(ref, got)  # bit-identical on every rank: all ranks sum the slots in one order
        # the step as a CUDA graph, replayed: the barrier's step counter lives in device memory
        sharded.set_position(64)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            sharded.step(h0)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        sharded.arena.check()
        ok = ok and bool(((sharded.logits - want).abs() <= 1e-2 * (1 + want.abs())).all())
        del g
        sharded.close()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_decoder_stack_two_gpus():
    """The tensor-parallel decoder stack (whole heads per rank, fused exchanges) against the single-GPU stack that
    holds the same codes."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_stack_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert ret.get(0) and ret.get(1)
