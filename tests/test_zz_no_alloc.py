"""The allocation-free forward, qb200_qlinear_forward_static.

Who needs it: a caller that must not allocate device memory while it issues work — a serving
loop whose memory budget is frozen after start-up, a host that owns every device buffer through
another runtime, latency-critical code that cannot take cudaMalloc's implicit synchronisation.  The ordinary forward may grow a scratch
buffer (cudaMalloc) for the split-K partial sums of `[in, out]` weights; this entry point keeps
those partial sums in a 2 MiB array built into the library instead.

Checked here, through the C ABI: two calls in a row give exactly the ordinary entry point's
output (the array is shared and keeps the previous call's contents, so the second call proves
nothing has to be cleared), other shapes reuse the array correctly, and a call that would not
fit is refused with the sizes in the message.  This file is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

import quanta_b200 as qb
from quanta_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layer(in_dim, out_dim, dtype, gran, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    w = torch.randn(in_dim, out_dim, device=DEV, generator=gen) * 0.02
    b = torch.randn(out_dim, device=DEV, generator=gen)
    return qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, dtype, gran), b, qb.IN_OUT)


def _static(ql, x, out_dtype):
    y = torch.empty((x.shape[0], ql.out_dim()), dtype=out_dtype, device=x.device)
    act = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]  # the driver's count of free device bytes, after the output exists
    st = _lib.load().qb200_qlinear_forward_static(ql._h, x.data_ptr(), act[x.dtype], x.shape[0], y.data_ptr(),
                                                  act[out_dtype], ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
    return st, y


def test_static_forward_matches_the_ordinary_forward_twice_in_a_row():
    lib = _lib.load()
    cases = [(4096, 256, qb.QuantDtype.Int4, qb.Group(0, 40)),    # small out, long K: K is split, scratch in use (groups of 40: no fast kernel)
             (1024, 520, qb.QuantDtype.Int8, qb.Block(8, 8)),         # tiles no fast kernel takes: the ordinary forward is generic too
             (512, 4096, qb.QuantDtype.Int4, qb.Group(0, 8))]     # wide out: one slice, no scratch
    for in_dim, out_dim, dt, gran in cases:
        ql = _layer(in_dim, out_dim, dt, gran, seed=in_dim + out_dim)
        for m, xdt, ydt in [(3, torch.float32, torch.float32), (9, torch.bfloat16, torch.float32), (1, torch.float32, torch.bfloat16)]:
            x = torch.randn(m, in_dim, device=DEV).to(xdt)
            want = ql.forward(x, out_dtype=ydt)
            assert ql.last_kernel() == "generic_cols"
            for call in range(2):
                st, got = _static(ql, x, ydt)
                assert st == 0, _lib.last_error()
                torch.cuda.synchronize()
                # same kernels, same K slicing: the tolerance of the forward tests (1e-4) is met with equality
                assert torch.equal(got, want), (in_dim, out_dim, m, call)
                assert ql.last_kernel() == "generic_cols"
    assert lib.qb200_qlinear_check(ql._h, None) == 0


def test_static_forward_refuses_what_does_not_fit_and_other_layouts():
    ql = _layer(4096, 2048, qb.QuantDtype.Int4, qb.Group(0, 64), seed=1)
    m = 72  # 4 K slices x 72 x 2048 partial sums = 589 824 > 2^19
    x = torch.zeros(m, 4096, device=DEV)
    st, _ = _static(ql, x, torch.float32)
    assert st == _lib.ERR_INVALID_PARAM
    msg = _lib.last_error()
    assert "2 MiB" in msg and str(m) in msg and "2048" in msg
    st, y = _static(ql, x[:64].contiguous(), torch.float32)   # 4 x 64 x 2048 = 2^19 fits exactly
    assert st == 0 and torch.equal(y, ql.forward(x[:64].contiguous(), out_dtype=torch.float32))
    w = torch.randn(64, 256, device=DEV) * 0.02
    rows = qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int8, qb.PerTensor()), None, qb.OUT_IN)
    st, _ = _static(rows, torch.zeros(2, 256, device=DEV), torch.float32)
    assert st == _lib.ERR_NOT_SUPPORTED and "qb200_qlinear_forward" in _lib.last_error()
