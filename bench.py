#!/usr/bin/env python
"""Benchmark of the quantized-inference hot path on B200.

  python bench.py --gpus N --steps K --warmup W            (this build's CUDA path)
  python bench.py --impl reference --gpus N --steps K ...  (the reference's CPU algorithm)

Headline workload: the int4 decode GEMV configuration — QuantizedLinear forward over
resident int4 codes `[4096, 4096]` (packed, low nibble = even k) with a 1x128 f32 scale
grid, X bf16 `[M=1, 4096]`, f32 out.  One "step" is one pass over LAYERS distinct weight
matrices that read the same X (independent projections, as fused QKV / gate+up are): by
default one grouped call (qb200_qlinear_forward_many, one persistent launch), with
--launch per-layer one qb200_qlinear_forward launch per matrix.  The matrices together
exceed L2, so their codes stream from HBM.  Inputs are seeded synthetic data of the stated shapes.

Metric: weight GB/s = algorithmic bytes (codes + scales + X + Y) of all launches / time.
With N > 1 every rank holds its own `[4096, 4096]` column shard of a `[4096*N, 4096]` layer
(weak scaling) and the shards' outputs are all-gathered after every layer.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_OUT, K_IN, GROUP = 4096, 4096, 128
LAYERS = 32  # 32 x 8.9 MB = 286 MB of codes + scales, larger than the 126 MB L2
METRIC = "QuantizedLinear weight GB/s (int4 decode GEMV)"
NOMINAL_HBM_GBS = 8000.0  # the figure the workload's target is quoted against
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch divided by the layers it processed, from the
# ncu capture summarised in profiles/gemv_i4_grouped_decode.md (an 8-layer launch; traffic grows in proportion to the
# layers).  It describes the kernel as captured then; a changed kernel needs a new capture.
TRAFFIC_PER_LAYER = {1: 72.13e6 / 8, 16: 73.43e6 / 8}
TRAFFIC_SOURCE = "ncu capture of an 8-layer launch (profiles/gemv_i4_grouped_decode.md), scaled by the layers per launch"


def workload_name(m: int) -> str:
    """The workload both arms name in `config.workload` (the reference arm times a bounded sample of it)."""
    return f"int4 decode GEMV W[{N_OUT},{K_IN}] grid 1x{GROUP}, X bf16 [{m},{K_IN}], f32 out"


def bench_config(m: int, world: int) -> dict:
    """`config` of the JSON line, the same in both arms."""
    return {"workload": workload_name(m), "layers_per_step": LAYERS,
            "l2": f"inputs larger than L2 ({LAYERS} distinct weight matrices, {layer_bytes(m) * LAYERS / 1e6:.0f} MB)",
            "parallelism": "single GPU" if world == 1 else f"column-sharded x{world} (weak scaling: one [{N_OUT},{K_IN}] shard per GPU), outputs all-gathered"}


def layer_bytes(m: int) -> int:
    """Algorithmic bytes of one forward launch: codes N*K/2 + scales N*(K/128)*4 + X m*K*2 + Y m*N*4."""
    return N_OUT * K_IN // 2 + N_OUT * (K_IN // GROUP) * 4 + m * K_IN * 2 + m * N_OUT * 4


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.stop, self.thread = index, [], threading.Event(), None

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                if len(f) >= 6:
                    self.samples.append(f)
            except Exception:
                pass
            self.stop.wait(0.1)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": float(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}


def make_inputs(m: int, layers: int, seed: int):
    """Seeded synthetic weights ~ N(0, 0.02) and X ~ N(0, 1) (bf16 by round-to-nearest-even)."""
    rng = np.random.default_rng(seed)
    w = [rng.standard_normal((N_OUT, K_IN), dtype=np.float32) * np.float32(0.02) for _ in range(layers)]
    x = rng.standard_normal((16, K_IN), dtype=np.float32)[:m]
    return w, x


# ---------------------------------------------------------------------------------------
# reference arm: the reference's CPU algorithm (dequantize the whole weight, then the
# sequential-k f32 GEMM) on the host cores, timed on a bounded sample of the same workload
# ---------------------------------------------------------------------------------------

def cpu_forward_gbs(m: int, threads: int, layers: int, reps: int):
    import oracle as o
    w, x = make_inputs(m, layers, seed=1)
    xq = o.bf16_to_f32(o.f32_to_bf16(x))
    quant = [o.quantize_host(wi, N_OUT, K_IN, 4, 1, GROUP) for wi in w]
    scratch = np.empty(N_OUT * K_IN, dtype=np.float32)
    o.qlinear_apply(quant[0][0], quant[0][1], N_OUT, K_IN, 4, 1, GROUP, o.OUT_IN, xq, None, threads, scratch)
    t0 = time.perf_counter()
    for _ in range(reps):
        for c, s in quant:
            o.qlinear_apply(c, s, N_OUT, K_IN, 4, 1, GROUP, o.OUT_IN, xq, None, threads, scratch)
    dt = time.perf_counter() - t0
    return layer_bytes(m) * layers * reps / dt / 1e9, dt


def cpu_quantize_baseline():
    """quantize_host / dequantize_host of the CPU restatement on ONE thread (the reference's loops are single-threaded:
    crates/sci/quanta-array/src/quant.rs:293-413), on one [4096, 4096] matrix of the checkpoint workload."""
    import oracle as o
    rng = np.random.default_rng(3)
    w = rng.standard_normal((4096, 4096), dtype=np.float32) * np.float32(0.02)
    res = {"cores": 1, "kind": "port", "sample": "1 of the 64 matrices ([4096, 4096] f32, 67 MB read), single thread"}
    for name, bits, gr, gc in [("int4_1x128", 4, 1, 128), ("int8_32x32", 8, 32, 32)]:
        t0 = time.perf_counter()
        c, sc = o.quantize_host(w, 4096, 4096, bits, gr, gc)
        t1 = time.perf_counter()
        o.dequantize_host(c, sc, 4096, 4096, bits, gr, gc)
        t2 = time.perf_counter()
        res["quantize_" + name + "_read_GB/s"] = w.nbytes / (t1 - t0) / 1e9
        res["dequantize_" + name + "_write_GB/s"] = w.nbytes / (t2 - t1) / 1e9
    return res


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as o
    threads = o.max_threads()
    layers = 2
    for _ in range(max(args.warmup, 1)):
        cpu_forward_gbs(args.m, threads, 1, 1)
    vals, t_total = [], 0.0
    _, probe = cpu_forward_gbs(args.m, threads, layers, 1)
    reps = max(1, int(1.0 / max(probe, 1e-3)))   # about one second of CPU work per step
    steps = min(args.steps, 60)                  # bounded: the whole run stays within minutes
    for _ in range(steps):
        v, dt = cpu_forward_gbs(args.m, threads, layers, reps)
        vals.append(v)
        t_total += dt
    value = float(np.mean(vals))
    sample = f"{layers} of {LAYERS} layers x {reps} passes per step, dequantize + sequential-k f32 GEMM, {threads} OpenMP threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t_total / max(steps, 1), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.m, max(args.gpus, 1)),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# this build's arm
# ---------------------------------------------------------------------------------------

def measure_decode_step(torch, dev, gen, hbm, n_layers, world=1):
    """Whole-model decode step: `n_layers` Llama-7B-shaped blocks + vocabulary projection, int4 1x128 linears,
    batch 16, 1024 cached positions (KV bf16), random-initialised; one step = one CUDA graph replay.  With
    world > 1 the stack is tensor-parallel over the ranks (whole heads per rank, two fused exchanges per block)."""
    import torch.distributed as dist
    stack = None
    try:
        from quanta_b200 import decoder as dec
        torch.cuda.empty_cache()
        if world > 1:
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        stack = dec.DecoderStack(n_layers, 4096, 32, 11008, 32000, 16, 1025, dev, seed=4, group=dist.group.WORLD if world > 1 else None)
        stack.set_position(1024)
        h0 = torch.randn(16, 4096, device=dev, generator=torch.Generator(device=dev).manual_seed(5)) * 0.02

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)

        for _ in range(2):
            stack.step(h0)
        barrier()
        if stack.arena is not None:
            stack.arena.check()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            stack.step(h0)
        for _ in range(3):
            g.replay()
        iters = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(iters):
            g.replay()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / iters
        logits_ok = bool(torch.isfinite(stack.logits).all().item())
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            stack.arena.check()  # a consumer that gave up waiting would have let the step run on missing partial sums
            # every rank must hold the same logits after the last exchange
            ref = stack.logits.clone()
            dist.broadcast(ref, 0)
            same = torch.tensor([1.0 if torch.equal(ref, stack.logits) and logits_ok else 0.0], device=dev)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            logits_ok = bool(same.item() == 1.0)
        by = stack.weight_bytes + stack.kv_bytes(1025)  # per GPU
        res = {"tokens/s": 16 / ms * 1e3, "ms_per_step": ms, "layers": n_layers, "batch": 16, "context": 1024, "n_gpus": world,
               "bytes_per_step_per_gpu": by, "GB/s_per_gpu": by / ms / 1e6, "roofline_frac": by / ms / 1e6 / hbm,
               "launch": "cuda graph replay of the step", "logits_finite_and_equal_on_all_ranks": logits_ok}
        if world > 1:
            # the exchanges' share of the step: the same graph with every exchange switched off (each rank stores only
            # into its own buffer and nothing waits; the logits of that run mean nothing, only its time does)
            stack.exchange = False
            for _ in range(2):
                stack.step(h0)
            barrier()
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2):
                stack.step(h0)
            for _ in range(3):
                g2.replay()
            barrier()
            e0.record()
            for _ in range(iters):
                g2.replay()
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            del g2
            stack.exchange = True
            res["ms_per_step_without_exchanges"] = float(t.item())
            res["exchange_share_of_step"] = max(0.0, 1.0 - float(t.item()) / ms)
            res["exchanges_per_step"] = 2 * n_layers + 1
            res["nvlink_bytes_per_step_per_gpu"] = stack.exchange_bytes() * (world - 1)
            res["parallelism"] = (f"tensor-parallel x{world}: whole heads per rank, row-parallel output and down projections; the producing "
                                  "kernels push their partial sums to every rank as self-validating elements, the consumers poll (no barrier)")
        del g
        return res
    except Exception as e:  # the rest of the line must survive
        return {"skipped": f"{type(e).__name__}: {str(e)[:160]}"}
    finally:
        if stack is not None:
            try:
                stack.close()
            except Exception:
                pass
        del stack
        torch.cuda.empty_cache()


def measure_int8_decode(torch, qb, dev, gen, timed, hbm, n_layers):
    """The decode workload over int8 codes with 32 x 32 blocks (the grid of the quantize-on-load workload's int8 half):
    `n_layers` distinct [4096, 4096] matrices per grouped launch, X bf16 [M, 4096], M = 1 and 8."""
    out = {}
    try:
        lys = [qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(torch.randn(4096, 4096, device=dev, generator=gen) * 0.02,
                                                                   qb.QuantDtype.Int8, qb.Block(32, 32)), None, qb.OUT_IN)
               for _ in range(n_layers)]
        from quanta_b200 import _lib
        lib = _lib.load()
        hs = (_lib.vp * n_layers)(*[ql._h for ql in lys])
        for mm in (1, 8):
            xm = torch.randn(mm, 4096, device=dev, generator=gen).to(torch.bfloat16)
            ym = torch.empty(n_layers, mm, 4096, device=dev, dtype=torch.float32)
            xp = (_lib.vp * n_layers)(*[xm.data_ptr()] * n_layers)
            yp = (_lib.vp * n_layers)(*[ym[i].data_ptr() for i in range(n_layers)])

            def run8():
                st = lib.qb200_qlinear_forward_many(hs, n_layers, xp, _lib.BF16, mm, yp, _lib.F32, torch.cuda.current_stream(dev).cuda_stream)
                if st:
                    raise RuntimeError(_lib.last_error())
            ms = timed(run8, 200 if n_layers == 32 else 5)
            by = n_layers * (4096 * 4096 + 128 * 128 * 4 + mm * 4096 * 2 + mm * 4096 * 4)
            out[f"decode_gemv_int8_32x32_M{mm}"] = {"GB/s": by / ms / 1e6, "ms": ms, "roofline_frac": by / ms / 1e6 / hbm,
                                                    "kernel": lys[0].last_kernel(), "bytes": by,
                                                    "launch": f"grouped, {n_layers} matrices per launch"}
        del lys
    except Exception as e:
        out["decode_gemv_int8"] = {"skipped": str(e)[:80]}
    return out


def measure_extras(torch, qb, dev, only=None, small=False, world=1):
    """Secondary numbers of the same path on one GPU (device-resident inputs, CUDA events):
    the int4 prefill GEMM configuration and quantize-on-load, each with its roofline fraction."""
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm, tf = float(peaks.get("hbm_gbs", 6650.0)), float(peaks.get("bf16_tflops", 1590.0))

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / iters

    def timed_replay(fn, reps, iters=5):
        """Device time of one `fn()`: `reps` calls captured into a CUDA graph, the graph replayed.  A quantize or
        dequantize call is one 15 - 45 us kernel behind a Python wrapper whose own cost is of that order, so eager
        calls leave the GPU idle between launches and would time the host."""
        fn()
        torch.cuda.synchronize(dev)
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(reps):
                    fn()
        except Exception:  # capture not possible: eager calls, host gaps included
            torch.cuda.synchronize(dev)
            return timed(fn, reps), "eager calls"
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            g.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / iters / reps
        del g
        return ms, f"cuda graph replay of {reps} calls"

    out = {}
    gen = torch.Generator(device=dev).manual_seed(2)
    if only == "int8_decode":
        return measure_int8_decode(torch, qb, dev, gen, timed, hbm, 8 if small else 32)
    if only == "decode_step" or world > 1:  # the one side workload that shards: the whole-model decode step
        return {"decode_step_llama7b_shape": measure_decode_step(torch, dev, gen, hbm, 2 if small else 32, world)}
    M, N, K = (512, 2048, 4096) if small else (2048, 11008, 4096)
    w = torch.randn(N, K, device=dev, generator=gen) * 0.02
    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
    # quantize-on-load: f32 [11008, 4096] (180 MB, larger than L2) -> int4 1x128 and int8 32x32
    if only in ("blas_quant", "blas_quant_brief"):
        brief = only == "blas_quant_brief"
        # the quantized BLAS entries: int codes for both operands, one per i32 word (the reference's storage), so a call
        # is two packing passes over 4 B per code and the tcgen05 kind::i8 GEMM; the GEMV entry reads A's codes once
        from quanta_b200 import blas
        del w, x
        res = {}
        q8 = blas.GemmQuantType.Q8Symmetric
        for m, n, k in ([(1024, 1024, 2048)] if small else [(4096, 4096, 4096)] if brief else [(4096, 4096, 4096), (8192, 8192, 8192)]):
            a = torch.randint(-128, 128, (m * k,), dtype=torch.int32, device=dev, generator=gen)
            b = torch.randint(-128, 128, (k * n,), dtype=torch.int32, device=dev, generator=gen)
            c = torch.zeros(m * n, device=dev)
            ms = timed(lambda: blas.gemm_quant(q8, m, n, k, 1.0, 0.01, 0.01, a, b, 0.0, c), 3 if small else 10)
            blas.check_stream(c)
            res[f"gemm_quant_{m}x{n}x{k}"] = {"TOP/s": 2.0 * m * n * k / ms / 1e9, "ms": ms, "launches_per_call": 3,
                                               "code_bytes_read": 4 * (m * k + k * n)}
            del a, b, c
        m, n = (4096, 4096) if small else (16384, 8192)
        a = torch.randint(-128, 128, (m * n,), dtype=torch.int32, device=dev, generator=gen)
        xq = torch.randint(-128, 128, (n,), dtype=torch.int32, device=dev, generator=gen)
        y = torch.zeros(m, device=dev)
        ms = timed(lambda: blas.gemv_quant(q8, m, n, 1.0, 0.01, 0.01, a, xq, 0.0, y), 3 if small else 10)
        blas.check_stream(y)
        res[f"gemv_quant_{m}x{n}"] = {"GB/s": 4.0 * m * n / ms / 1e6, "ms": ms, "roofline_frac": 4.0 * m * n / ms / 1e6 / hbm,
                                      "bytes": 4 * m * n}
        return res
    if only == "prefill":
        qm = qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128))
        ql = qb.QuantizedLinear.new(qm, None, qb.OUT_IN)
        ms = timed(lambda: ql.forward(x), 3 if small else 10)
        res = {"prefill_int4_gemm": {"TFLOP/s": 2.0 * M * N * K / ms / 1e9, "ms": ms, "roofline_frac": 2.0 * M * N * K / ms / 1e9 / tf,
                                     "peak_TFLOP/s": tf, "shape": {"M": M, "N": N, "K": K}, "kernel": ql.last_kernel()}}
        del ql, qm
        # the same shape over int8 codes: the 32 x 32 grid closes an accumulator every 32 k, a 1 x 128 grid every 128
        for name, gran in [("prefill_int8_32x32_gemm", qb.Block(32, 32)), ("prefill_int8_1x128_gemm", qb.Group(1, 128))]:
            ql = qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int8, gran), None, qb.OUT_IN)
            ms = timed(lambda: ql.forward(x), 3 if small else 10)
            res[name] = {"TFLOP/s": 2.0 * M * N * K / ms / 1e9, "ms": ms, "roofline_frac": 2.0 * M * N * K / ms / 1e9 / tf,
                         "shape": {"M": M, "N": N, "K": K}, "kernel": ql.last_kernel()}
            del ql
        return res
    for name, dt, gran, wbytes in [("quantize_int4_1x128", qb.QuantDtype.Int4, qb.Group(1, 128), N * K // 2 + N * (K // 128) * 4),
                                   ("quantize_int8_32x32", qb.QuantDtype.Int8, qb.Block(32, 32), N * K + (N // 32) * (K // 32) * 4)]:
        ms, how = timed_replay(lambda: qb.QuantizedMatrix.quantize(w, dt, gran), 10)
        out[name] = {"read_GB/s": N * K * 4 / ms / 1e6, "ms": ms, "roofline_frac": (N * K * 4 + wbytes) / ms / 1e6 / hbm,
                     "shape": [N, K], "launch": how}
    qm = qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128))
    ms, how = timed_replay(lambda: qm.dequantize(), 10)
    out["dequantize_int4_1x128"] = {"write_GB/s": N * K * 4 / ms / 1e6, "ms": ms,
                                    "roofline_frac": (N * K * 4.5 + N * (K // 128) * 4) / ms / 1e6 / hbm, "shape": [N, K],
                                    "launch": how}
    # quantize-on-load at the whole checkpoint's size: 32 x [4096, 4096] + 32 x [11008, 4096] f32 (7.92 GB read),
    # input resident in HBM, one quantize call per matrix
    try:
        mats = [torch.randn(4096, 4096, device=dev, generator=gen) * 0.02 for _ in range(32)]
        mats += [torch.randn(11008, 4096, device=dev, generator=gen) * 0.02 for _ in range(32)]
        elems = sum(t.numel() for t in mats)
        for name, dt, gran, per_elem in [("checkpoint_int4_1x128", qb.QuantDtype.Int4, qb.Group(1, 128), 0.5 + 4 / 128),
                                         ("checkpoint_int8_32x32", qb.QuantDtype.Int8, qb.Block(32, 32), 1 + 4 / 1024)]:
            def run():
                for t in mats:
                    qb.QuantizedMatrix.quantize(t, dt, gran)
            ms, how = timed_replay(run, 1, iters=3)
            out["quantize_" + name] = {"read_GB/s": elems * 4 / ms / 1e6, "ms": ms, "matrices": len(mats), "read_bytes": elems * 4,
                                       "roofline_frac": elems * (4 + per_elem) / ms / 1e6 / hbm,
                                       "launch": how.replace("1 calls", "the 64 quantize calls")}
        del mats
    except torch.OutOfMemoryError as e:  # a smaller device: report why the line is missing
        out["quantize_checkpoint"] = {"skipped": str(e)[:80]}
    # decode GEMV at the other batch sizes of the configuration (M = 4, 16), grouped launch over 32 matrices
    try:
        lys = [qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(torch.randn(4096, 4096, device=dev, generator=gen) * 0.02,
                                                                   qb.QuantDtype.Int4, qb.Group(1, 128)), None, qb.OUT_IN)
               for _ in range(32)]
        from quanta_b200 import _lib
        lib = _lib.load()
        hs = (_lib.vp * 32)(*[ql._h for ql in lys])
        for mm in (4, 16):
            xm = torch.randn(mm, 4096, device=dev, generator=gen).to(torch.bfloat16)
            ym = torch.empty(32, mm, 4096, device=dev, dtype=torch.float32)
            xp = (_lib.vp * 32)(*[xm.data_ptr()] * 32)
            yp = (_lib.vp * 32)(*[ym[i].data_ptr() for i in range(32)])

            def run():
                st = lib.qb200_qlinear_forward_many(hs, 32, xp, _lib.BF16, mm, yp, _lib.F32, torch.cuda.current_stream(dev).cuda_stream)
                if st:
                    raise RuntimeError(_lib.last_error())
            ms = timed(run, 200)
            by = 32 * (4096 * 4096 // 2 + 4096 * 32 * 4 + mm * 4096 * 2 + mm * 4096 * 4)
            out[f"decode_gemv_M{mm}"] = {"GB/s": by / ms / 1e6, "ms": ms, "roofline_frac": by / ms / 1e6 / hbm,
                                         "kernel": lys[0].last_kernel(), "launch": "grouped, 32 matrices per launch"}
        del lys
    except Exception as e:
        out["decode_gemv_M"] = {"skipped": str(e)[:80]}
    out.update(measure_int8_decode(torch, qb, dev, gen, timed, hbm, 32))
    try:  # the reference's CPU-runnable configuration as it is: int8 [1024, 1024], 32 x 32 blocks, X f32 [8, 1024], one call
        w1 = torch.randn(1024, 1024, device=dev, generator=gen) * 0.02
        x1 = torch.randn(8, 1024, device=dev, generator=gen)
        ql1 = qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w1, qb.QuantDtype.Int8, qb.Block(32, 32)), None, qb.OUT_IN)
        ms, how = timed_replay(lambda: ql1.forward(x1, out_dtype=torch.float32), 10)
        out["config1_int8_32x32_f32_x8"] = {"us_per_call": ms * 1e3, "kernel": ql1.last_kernel(), "launch": how,
                                             "note": "1 MB of codes: launch-bound, not an HBM measurement; f32 activations as three bf16 parts"}
        del ql1, w1, x1
    except Exception as e:
        out["config1_int8_32x32_f32_x8"] = {"skipped": str(e)[:80]}
    out["decode_step_llama7b_shape"] = measure_decode_step(torch, dev, gen, hbm, 32, 1)
    try:  # the reference's quantize / dequantize are single-threaded host loops: the restatement timed the same way
        out["cpu_quantize_baseline"] = cpu_quantize_baseline()
    except Exception as e:
        out["cpu_quantize_baseline"] = {"skipped": f"{type(e).__name__}: {str(e)[:120]}"}
    try:  # the quantized BLAS entries (int codes for both operands): one GEMM size and the GEMV
        out["blas_quant"] = measure_extras(torch, qb, dev, only="blas_quant_brief")
    except Exception as e:
        out["blas_quant"] = {"skipped": f"{type(e).__name__}: {str(e)[:120]}"}
    ql = qb.QuantizedLinear.new(qm, None, qb.OUT_IN)
    ms = timed(lambda: ql.forward(x), 10)
    out["prefill_int4_gemm"] = {"TFLOP/s": 2.0 * M * N * K / ms / 1e9, "ms": ms, "roofline_frac": 2.0 * M * N * K / ms / 1e9 / tf,
                                "peak_TFLOP/s": tf, "shape": {"M": M, "N": N, "K": K}, "kernel": ql.last_kernel()}
    del ql
    try:  # the same shape over int8 codes with 32 x 32 blocks (an accumulator every 32 k)
        ql8 = qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int8, qb.Block(32, 32)), None, qb.OUT_IN)
        ms = timed(lambda: ql8.forward(x), 10)
        out["prefill_int8_32x32_gemm"] = {"TFLOP/s": 2.0 * M * N * K / ms / 1e9, "ms": ms, "roofline_frac": 2.0 * M * N * K / ms / 1e9 / tf,
                                          "shape": {"M": M, "N": N, "K": K}, "kernel": ql8.last_kernel()}
        del ql8
    except Exception as e:
        out["prefill_int8_32x32_gemm"] = {"skipped": f"{type(e).__name__}: {str(e)[:120]}"}
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    import quanta_b200 as qb
    from quanta_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device — this build has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # the ranks' own kernels store into peer memory; keep NVLink multicast objects out of it
        dist.init_process_group("nccl", device_id=dev)

    global LAYERS
    LAYERS = args.layers
    m = args.m
    lib = _lib.load()
    if args.only:  # side workloads alone (used for profiling): prefill GEMM, quantize / dequantize, the decode step
        ex = measure_extras(torch, qb, dev, only=args.only, small=args.small, world=world)
        if rank == 0:
            print(json.dumps({"only": args.only, "extras": ex}), flush=True)
        if world > 1:
            _leave(torch, dist, dev)
        return
    # device-side quantize-on-load of this rank's shards (seeded per rank)
    gen = torch.Generator(device=dev).manual_seed(1 + rank)
    layers = []
    for _ in range(LAYERS):
        w = torch.randn(N_OUT, K_IN, device=dev, generator=gen) * 0.02
        qm = qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, GROUP))
        layers.append(qb.QuantizedLinear.new(qm, None, qb.OUT_IN))
        del w
    x = torch.randn(m, K_IN, device=dev, generator=torch.Generator(device=dev).manual_seed(99)).to(torch.bfloat16)  # the same on every rank
    y_all = torch.empty(world, m, N_OUT, device=dev, dtype=torch.float32) if world > 1 else None
    stream = torch.cuda.current_stream(dev)

    y_cat = torch.empty(LAYERS, m, N_OUT, device=dev, dtype=torch.float32)
    ys = [y_cat[i] for i in range(LAYERS)]
    y_cat_all = torch.empty(world * LAYERS, m, N_OUT, device=dev, dtype=torch.float32) if world > 1 else None
    hs = (_lib.vp * LAYERS)(*[ql._h for ql in layers])
    xp = (_lib.vp * LAYERS)(*[x.data_ptr()] * LAYERS)
    yp = (_lib.vp * LAYERS)(*[t.data_ptr() for t in ys])
    grouped = args.launch == "grouped"
    # N > 1, grouped: the kernel stores the step's outputs into every rank's buffer itself (peer memory) and the
    # arrival barrier runs in the same launch; --gather nccl keeps the library all-gather for comparison
    fused = world > 1 and grouped and args.gather in ("fused", "pushed", "pushed+gather") and m <= 16
    pg = None
    if fused:
        # every rank must take the same path: the ranks agree on whether all of them could map the peers' buffers
        from quanta_b200 import tp as _tp
        ok = torch.ones(1, device=dev)
        try:
            pg = _tp.PeerGather(LAYERS, m, N_OUT, torch.float32, mode={"fused": "barrier", "pushed": "pushed", "pushed+gather": "pushed+gather"}[args.gather])
        except Exception as e:  # no peer access between these devices, or IPC refused: the library collective serves
            print(f"bench.py: rank {rank}: fused all-gather unavailable ({type(e).__name__}: {str(e)[:100]}); using NCCL", file=sys.stderr)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            fused, pg = False, None

    def one(parity=None):
        cur = torch.cuda.current_stream(dev).cuda_stream  # the capture stream while a graph is recorded
        if fused:
            pg.forward_many(layers, [x] * LAYERS, parity)
            return
        if grouped:  # the 32 layers read the same x: one persistent launch streams all their codes
            st = lib.qb200_qlinear_forward_many(hs, LAYERS, xp, _lib.BF16, m, yp, _lib.F32, cur)
            if st:
                raise RuntimeError(_lib.last_error())
            if world > 1:  # the step's outputs are independent: one all-gather for all of them
                dist.all_gather_into_tensor(y_cat_all, y_cat)
            return
        for ql, t in zip(layers, ys):
            st = lib.qb200_qlinear_forward(ql._h, x.data_ptr(), _lib.BF16, m, t.data_ptr(), _lib.F32, cur)
            if st:
                raise RuntimeError(_lib.last_error())
            if world > 1:
                dist.all_gather_into_tensor(y_all, t)

    # A graph replay is TWO steps: the fused exchange alternates between two receive buffers step by step, and
    # a replayed graph must keep that alternation, so the unit that is captured and timed is a pair.
    def pair():
        one(0)
        one(1)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(2):
        pair()
    barrier()
    run_pair = pair
    if not args.no_graph:
        # the launches keep their programmatic-dependency edges inside the graph, so the next launch's weight
        # prefetch overlaps the current one's tail
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            pair()
        run_pair = graph.replay
        stream = torch.cuda.current_stream(dev)
    steps = max(2, args.steps + (args.steps & 1))  # whole pairs
    pairs = steps // 2

    def block():
        for _ in range(pairs):
            run_pair()

    # spin the clocks up for at least half a second before timing; the clock sampler runs from here
    # to the end of the timed region (same kernel, same load)
    clocks = ClockSampler(local)
    clocks.__enter__()
    # every rank must run the same number of steps (they hold collectives): rank 0 sizes the
    # spin-up and the number of timed blocks from a probe and broadcasts the counts
    for _ in range(max(args.warmup, 3)):
        run_pair()
    barrier()
    t_probe = time.perf_counter()
    block()
    barrier()
    block_s = max(time.perf_counter() - t_probe, 1e-6)
    n_spin = 0 if args.profile else int(min(max(0.5 / block_s, 1), 20000))
    # the timed region is `n_blocks` blocks of `steps` steps, at least a quarter of a second in all; the block
    # with the median time is the one reported
    n_blocks = 1 if args.profile else int(min(max(0.25 / block_s, 3), 5000))
    if world > 1:
        cnt = torch.tensor([n_spin, n_blocks], device=dev, dtype=torch.int64)
        dist.broadcast(cnt, 0)
        n_spin, n_blocks = int(cnt[0].item()), int(cnt[1].item())
    for i in range(n_spin):
        block()
        if i % 16 == 15:
            torch.cuda.synchronize(dev)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_blocks + 1)]
    barrier()
    evs[0].record(stream)
    for i in range(n_blocks):
        block()
        evs[i + 1].record(stream)
    barrier()
    clocks.__exit__()
    times = torch.tensor([evs[i].elapsed_time(evs[i + 1]) for i in range(n_blocks)], device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)  # per block, the slowest rank
    ms = float(times.median().item())
    timed_region_s = float(times.sum().item()) * 1e-3
    # fused exchange: the arrival barrier runs inside the GEMV launch; pushed exchange: the gathering kernel is a second launch
    launches = ((1 if grouped else LAYERS) + (1 if fused and args.gather == "pushed+gather" else 0)) * steps * n_blocks
    total_bytes = layer_bytes(m) * LAYERS * steps * world
    value = total_bytes / (ms * 1e-3) / 1e9

    # the multi-GPU numbers are only worth printing if the exchange delivered: no barrier timed out, and the
    # gathered buffer equals an NCCL all-gather of the same outputs
    gather_checked, device_status = None, 0
    if world > 1:
        try:
            if fused:
                pg.check()
            else:
                st = lib.qb200_qlinear_check(layers[0]._h, torch.cuda.current_stream(dev).cuda_stream)
                if st:
                    raise RuntimeError(_lib.last_error())
        except Exception as e:
            device_status = getattr(e, "code", -1)
            print(f"bench.py: rank {rank}: device status after the timed region: {e}", file=sys.stderr)
        st = lib.qb200_qlinear_forward_many(hs, LAYERS, xp, _lib.BF16, m, yp, _lib.F32, torch.cuda.current_stream(dev).cuda_stream)
        if st:
            raise RuntimeError(_lib.last_error())
        dist.all_gather_into_tensor(y_cat_all, y_cat)
        if fused:
            got = pg.forward_many(layers, [x] * LAYERS)
            pg.check()
            same = torch.equal(got.reshape(world * LAYERS, m, N_OUT), y_cat_all)
        else:
            same = True  # the timed path IS the library collective
        flag = torch.tensor([1.0 if same and device_status == 0 else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        gather_checked = bool(flag.item() == 1.0)

    # end to end through host buffers: pinned host X in, every layer's (at N > 1: every rank's) Y back on the host
    xh = torch.empty(m, K_IN, dtype=torch.bfloat16).pin_memory()
    xh.copy_(x.cpu())
    xd = torch.empty_like(x)
    xdp = (_lib.vp * LAYERS)(*[xd.data_ptr()] * LAYERS)
    # on one GPU every layer's output goes to the host; on N the host reads every output ONCE across the job: each rank
    # copies out the rows another rank computed (its neighbour's), as they arrived in its own gathered buffer
    yh = torch.empty(LAYERS, m, N_OUT, dtype=torch.float32).pin_memory()
    peer = (rank + 1) % world
    xhp = (_lib.vp * LAYERS)(*[xh.data_ptr()] * LAYERS)
    yhp = (_lib.vp * LAYERS)(*[yh[i].data_ptr() for i in range(LAYERS)])

    # the fused step at N > 1 as two CUDA graphs (the exchange alternates between two receive buffers): copy in, forward
    # with its exchange, copy out — one graph launch and one synchronize per step, the Python wrappers out of the way
    e2e_graphs = []
    if world > 1 and fused and not args.no_graph:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for parity in (0, 1):
                    xd.copy_(xh, non_blocking=True)
                    yh.copy_(pg.forward_many(layers, [xd] * LAYERS, parity=parity)[peer], non_blocking=True)
                torch.cuda.synchronize(dev)
                for parity in (0, 1):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        xd.copy_(xh, non_blocking=True)
                        yh.copy_(pg.forward_many(layers, [xd] * LAYERS, parity=parity)[peer], non_blocking=True)
                    e2e_graphs.append(g)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
        except Exception:
            e2e_graphs = []
            torch.cuda.synchronize(dev)
    e2e_calls = [0]

    def step_host():
        if world > 1:  # copy in, the forward with its exchange, copy the neighbour's rows of the gathered outputs out
            if e2e_graphs:
                e2e_graphs[e2e_calls[0] & 1].replay()
                e2e_calls[0] += 1
                torch.cuda.synchronize(dev)
                return
            cur = torch.cuda.current_stream(dev).cuda_stream
            xd.copy_(xh, non_blocking=True)
            if fused:
                got = pg.forward_many(layers, [xd] * LAYERS)
                yh.copy_(got[peer], non_blocking=True)  # (pushed: a strided read of the values)
            else:
                st = lib.qb200_qlinear_forward_many(hs, LAYERS, xdp, _lib.BF16, m, yp, _lib.F32, cur)
                if st:
                    raise RuntimeError(_lib.last_error())
                dist.all_gather_into_tensor(y_cat_all, y_cat)
                yh.copy_(y_cat_all.view(world, LAYERS, m, N_OUT)[peer], non_blocking=True)
            torch.cuda.synchronize(dev)
            return
        if grouped:  # one call: x copied once, one persistent launch, every layer's y copied back
            st = lib.qb200_qlinear_forward_many_host(hs, LAYERS, xhp, _lib.BF16, m, yhp, _lib.F32)
            if st:
                raise RuntimeError(_lib.last_error())
            return
        for i, ql in enumerate(layers):
            st = lib.qb200_qlinear_forward_host(ql._h, xh.data_ptr(), _lib.BF16, m, yh[i].data_ptr(), _lib.F32)
            if st:
                raise RuntimeError(_lib.last_error())

    for _ in range(0 if args.profile else 4):
        step_host()
    barrier()
    t0 = time.perf_counter()
    step_host()
    step_host()
    probe = max((time.perf_counter() - t0) / 2, 1e-6)
    e2e_steps = 2 if args.profile else int(min(max(0.2 / probe, 20), 20000)) & ~1
    if world > 1:
        cnt = torch.tensor([e2e_steps], device=dev, dtype=torch.int64)
        dist.broadcast(cnt, 0)
        e2e_steps = int(cnt.item())
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_host()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        tmax = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_s = float(tmax.item())
    e2e = layer_bytes(m) * LAYERS * e2e_steps * world / e2e_s / 1e9

    extras = None
    if not args.profile and not args.no_extras:
        extras = measure_extras(torch, qb, dev, world=world)
    if rank == 0:
        peak, which = measured_peak_gbs()
        # the dominant kernel is launched once per step (grouped) or once per layer; at N > 1 the step's time also
        # holds the exchange, so the fraction below is a lower bound there
        per_launch_s = ms * 1e-3 / ((1 if grouped else LAYERS) * steps)
        achieved = layer_bytes(m) * (LAYERS if grouped else 1) / per_launch_s / 1e9
        par = "single GPU" if world == 1 else f"column-sharded x{world}, every rank's outputs on every rank after each step"
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 x int4 -> f32", "data": "synthetic",
            "config": bench_config(m, world),
            "timing": {"blocks": n_blocks, "steps_per_block": steps, "reported": "median block, max over ranks per block",
                       "timed_region_s": timed_region_s, "block_ms_min": float(times.min().item()), "block_ms_max": float(times.max().item())},
            "impl_detail": {"kernel": layers[0].last_kernel(),
                            "launch": ("one persistent launch per step" if grouped else "one launch per layer") +
                                      (", eager" if args.no_graph else ", cuda graph replay of two steps"),
                            "exchange": None if world == 1 else (
                                ("pushed to every rank's buffer by the kernel as {value, exchange number} elements (peer memory), two receive buffers "
                                 "used in turn; every CTA polls its twins' rows before the launch ends" if args.gather == "pushed" else
                                 "pushed to every rank's buffer by the kernel as {value, exchange number} elements (peer memory), two receive buffers "
                                 "used in turn; a second kernel polls them into the dense gathered outputs" if args.gather == "pushed+gather" else
                                 "stored to every rank's buffer by the kernel (peer memory), two receive buffers used in turn, arrival barrier in the same launch") if fused
                                else "one NCCL all-gather of the step's outputs" if grouped else "NCCL all-gather per layer")},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": (1 if grouped or world > 1 else LAYERS) * m * K_IN * 2,
                    "d2h_bytes_per_step": LAYERS * m * N_OUT * 4, "steps": e2e_steps,
                    "call": ("per rank: copy in + fused forward / exchange + copy out of the rows its neighbour computed, from its own gathered "
                             "buffer (the job reads every output once)" + (", one CUDA graph launch and one synchronize per step" if e2e_graphs else "")
                             if world > 1 else
                             "qb200_qlinear_forward_many_host" if grouped else "qb200_qlinear_forward_host")},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "frac_nominal": achieved / NOMINAL_HBM_GBS, "nominal_peak": NOMINAL_HBM_GBS,
                         "traffic": TRAFFIC_PER_LAYER.get(m) * (LAYERS if grouped else 1) if TRAFFIC_PER_LAYER.get(m) else None,
                         "traffic_source": TRAFFIC_SOURCE if TRAFFIC_PER_LAYER.get(m) else None,
                         "peak_source": which, "launch_us": per_launch_s * 1e6},
        }
        if world > 1:
            line["gather_checked"] = gather_checked
            line["device_status"] = device_status
        if extras is not None:
            line["extras"] = extras
        if world == 1 and not args.no_cpu and not args.profile:
            import oracle as o
            threads = o.max_threads()
            v, dt = cpu_forward_gbs(m, threads, 2, 2)
            reps = max(2, int(10.0 / max(dt / 2, 1e-3)))  # about ten seconds of CPU work
            v, dt = cpu_forward_gbs(m, threads, 2, reps)
            line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"2 of {LAYERS} layers x {reps} passes ({dt:.1f} s), dequantize + sequential-k "
                                              f"f32 GEMM, {threads} OpenMP threads"}
            # the same on ONE thread: the reference's host loops are single-threaded, the threaded figure above is the
            # parallel restatement (its CPU lane spreads workgroups over the host's threads)
            v1, dt1 = cpu_forward_gbs(m, 1, 1, 3)
            line["cpu_baseline"]["single_thread"] = {"value": v1, "unit": "GB/s", "cores": 1,
                                                     "sample": f"1 of {LAYERS} layers x 3 passes ({dt1:.1f} s)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        if gather_checked is False:
            print("bench.py: the gathered outputs differ from the NCCL all-gather, or a device wait timed out", file=sys.stderr)
        _leave(torch, dist, dev, 0 if gather_checked else 3)


def _leave(torch, dist, dev, code=0):
    """Leaves a multi-rank run without tearing the process group down: destroying it while a captured graph that
    holds collectives is alive can block."""
    dist.barrier()
    torch.cuda.synchronize(dev)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="activation rows (1, 4 or 16 for the decode configuration)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--profile", action="store_true", help="short run for a profiler: no clock spin-up, no CPU leg")
    ap.add_argument("--launch", default="grouped", choices=["grouped", "per-layer"],
                    help="grouped: the step's layers go through qb200_qlinear_forward_many (one persistent launch); "
                         "per-layer: one qb200_qlinear_forward launch per layer")
    ap.add_argument("--gather", default="pushed", choices=["pushed", "pushed+gather", "fused", "nccl"],
                    help="N > 1, grouped launch: pushed = the kernel pushes {value, exchange number} elements to every rank and its "
                         "CTAs poll their twins' rows before the launch ends; pushed+gather = push only, a second kernel polls the "
                         "elements into dense outputs; fused = plain peer stores + arrival barrier in the launch; nccl = all-gather "
                         "after the kernel")
    ap.add_argument("--layers", type=int, default=LAYERS, help="distinct weight matrices per step")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill / quantize side measurements")
    ap.add_argument("--only", default=None, choices=["prefill", "quantize", "decode_step", "blas_quant", "int8_decode"], help="run only a side workload and print its numbers")
    ap.add_argument("--small", action="store_true", help="with --only: a reduced shape, for profiler captures")
    ap.add_argument("--no-graph", action="store_true", help="launch every layer eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
