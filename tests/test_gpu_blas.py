"""quanta-blas's quantized entries on the GPU against the oracle: the reference's own test cases
(crates/sci/quanta-blas/tests/gemm_quant.rs) at its tolerance, bit for bit where the sums stay below 2^24,
plus ragged and multi-tile shapes, the GEMV entries and the loud errors."""
import numpy as np
import pytest
import torch

import quanta_b200 as qb
from oracle import blas_oracle as bo
from quanta_b200 import blas
from tests.golden import kats

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
Q8, Q4 = blas.GemmQuantType.Q8Symmetric, blas.GemmQuantType.Q4Symmetric

Q8_CASES = [(4, 4, 4, 1.0, 0.0, 0.05, 0.05), (3, 5, 7, 1.0, 0.0, 0.1, 0.02), (6, 4, 5, 2.0, -1.0, 0.05, 0.05),
            (1, 8, 6, 1.0, 0.0, 0.05, 0.05), (8, 1, 6, 1.0, 0.0, 0.05, 0.05), (32, 24, 40, 1.0, 0.5, 0.02, 0.03)]
Q4_CASES = [(4, 4, 4, 1.0, 0.0, 0.1, 0.1), (3, 5, 7, 1.0, 0.0, 0.2, 0.05), (6, 4, 5, 2.0, -1.0, 0.1, 0.1),
            (16, 16, 24, 1.0, 0.5, 0.05, 0.08)]


def _dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32).reshape(-1)).to(DEV)


def _close(got, want):
    return bool((np.abs(got - want) <= 1e-3 * (1 + np.abs(want))).all())  # gemm_quant.rs:76


def _c0(m, n):
    return np.arange(m * n, dtype=np.float32) * np.float32(0.25) - np.float32(1.0)


@pytest.mark.parametrize("m,n,k,alpha,beta,sa,sb", Q8_CASES)
def test_q8_reference_cases(m, n, k, alpha, beta, sa, sb):
    a, b, c0 = bo.test_matrix(m, k, 1, 8), bo.test_matrix(k, n, 2, 8), _c0(m, n)
    c = torch.from_numpy(c0.copy()).to(DEV)
    blas.gemm_quant(Q8, m, n, k, alpha, sa, sb, _dev_i32(a), _dev_i32(b), beta, c)
    blas.check_stream(c)
    want = bo.gemm_q8_sym(m, n, k, alpha, sa, sb, a, b, beta, c0)
    got = c.cpu().numpy().reshape(m, n)
    assert _close(got, want)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # sums below 2^24: f32 accumulation is exact too


@pytest.mark.parametrize("m,n,k,alpha,beta,sa,sb", Q4_CASES)
def test_q4_reference_cases(m, n, k, alpha, beta, sa, sb):
    a, b, c0 = bo.test_matrix(m, k, 1, 4), bo.test_matrix(k, n, 2, 4), _c0(m, n)
    aw, bw = bo.int4_pack_flat(a), bo.int4_pack_flat(b)
    c = torch.from_numpy(c0.copy()).to(DEV)
    blas.gemm_quant4(Q4, m, n, k, alpha, sa, sb, _dev_i32(aw), _dev_i32(bw), beta, c)
    blas.check_stream(c)
    want = bo.gemm_q4_sym(m, n, k, alpha, sa, sb, aw, bw, beta, c0)
    got = c.cpu().numpy().reshape(m, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("m,n,k", [(300, 520, 1000), (129, 257, 131), (128, 256, 128), (1024, 1024, 2048), (5, 1030, 77)])
def test_q8_full_range_codes_multi_tile(m, n, k):
    rng = np.random.default_rng(m + n + k)
    span = 128 if k <= 1000 else 32  # keeps every running sum below 2^24, where the oracle is exact as well
    a = rng.integers(-span, span, size=(m, k), dtype=np.int32)
    b = rng.integers(-span, span, size=(k, n), dtype=np.int32)
    c0 = rng.standard_normal(m * n).astype(np.float32)
    c = torch.from_numpy(c0.copy()).to(DEV)
    blas.gemm_quant(Q8, m, n, k, 1.5, 0.01, 0.02, _dev_i32(a), _dev_i32(b), -0.5, c)
    blas.check_stream(c)
    want = bo.gemm_q8_sym(m, n, k, 1.5, 0.01, 0.02, a, b, -0.5, c0)
    got = c.cpu().numpy().reshape(m, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q8_beyond_exact_f32_sums_meets_the_reference_tolerance():
    m, n, k = 64, 96, 4096  # sums up to 4096 * 127^2: the reference's f32 accumulation rounds, the integer sum does not
    rng = np.random.default_rng(9)
    a = rng.integers(100, 128, size=(m, k), dtype=np.int32)
    b = rng.integers(100, 128, size=(k, n), dtype=np.int32)
    c = torch.zeros(m * n, device=DEV)
    blas.gemm_quant(Q8, m, n, k, 1.0, 0.01, 0.01, _dev_i32(a), _dev_i32(b), 0.0, c)
    blas.check_stream(c)
    got = c.cpu().numpy().reshape(m, n)
    assert _close(got, bo.gemm_q8_sym(m, n, k, 1.0, 0.01, 0.01, a, b, 0.0, np.zeros(m * n, np.float32)))
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32) * (np.float32(np.float32(1.0) * np.float32(0.01)) * np.float32(0.01))
    assert np.array_equal(got.view(np.uint32), exact.astype(np.float32).view(np.uint32))


@pytest.mark.parametrize("m,n,k", [(130, 260, 300), (64, 40, 1001)])
def test_q4_ragged_rows_start_inside_words(m, n, k):
    rng = np.random.default_rng(k)
    a = rng.integers(-8, 8, size=(m, k), dtype=np.int32)
    b = rng.integers(-8, 8, size=(k, n), dtype=np.int32)
    aw, bw = bo.int4_pack_flat(a), bo.int4_pack_flat(b)
    c0 = rng.standard_normal(m * n).astype(np.float32)
    c = torch.from_numpy(c0.copy()).to(DEV)
    blas.gemm_quant4(Q4, m, n, k, 1.0, 0.1, 0.2, _dev_i32(aw), _dev_i32(bw), 1.0, c)
    blas.check_stream(c)
    want = bo.gemm_q4_sym(m, n, k, 1.0, 0.1, 0.2, aw, bw, 1.0, c0)
    assert np.array_equal(c.cpu().numpy().reshape(m, n).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("m,n", [(7, 5), (1000, 4096), (33, 1027)])
def test_gemv_entries(m, n):
    rng = np.random.default_rng(m * n)
    a8, x8 = bo.test_matrix(m, n, 4, 8), bo.test_matrix(n, 1, 5, 8)
    y0 = (np.arange(m, dtype=np.float32) * np.float32(0.1))
    y = torch.from_numpy(y0.copy()).to(DEV)
    blas.gemv_quant(Q8, m, n, 1.0, 0.05, 0.04, _dev_i32(a8), _dev_i32(x8), 0.5, y)
    want = bo.gemm_q8_sym(m, 1, n, 1.0, 0.05, 0.04, a8, x8, 0.5, y0)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.reshape(-1).view(np.uint32))
    a4 = rng.integers(-8, 8, size=(m, n), dtype=np.int32)
    x4 = rng.integers(-8, 8, size=n, dtype=np.int32)
    aw, xw = bo.int4_pack_flat(a4), bo.int4_pack_flat(x4)
    y = torch.from_numpy(y0.copy()).to(DEV)
    blas.gemv_quant4(Q4, m, n, 2.0, 0.1, 0.3, _dev_i32(aw), _dev_i32(xw), -1.0, y)
    blas.check_stream(y)
    want = bo.gemm_q4_sym(m, 1, n, 2.0, 0.1, 0.3, aw, xw, -1.0, y0)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.reshape(-1).view(np.uint32))


def test_loud_errors():
    a = torch.zeros(4, dtype=torch.int32, device=DEV)
    c = torch.zeros(4, device=DEV)
    with pytest.raises(qb.QuantError, match="only Q8Symmetric"):  # gemm_quant.rs:215-238
        blas.gemm_quant(Q4, 2, 2, 2, 1.0, 0.1, 0.1, a, a, 0.0, c)
    with pytest.raises(qb.QuantError, match="only Q4Symmetric"):
        blas.gemm_quant4(Q8, 2, 2, 2, 1.0, 0.1, 0.1, a[:1], a[:1], 0.0, c)
    with pytest.raises(qb.QuantError) as e:
        blas.gemm_quant(Q8, 2, 2, 3, 1.0, 0.1, 0.1, a, a, 0.0, c)
    assert e.value.kind == "LengthMismatch"
    with pytest.raises(qb.QuantError):
        blas.gemm_quant(Q8, 2, 2, 2, 1.0, 0.1, 0.1, a.cpu(), a, 0.0, c)
    bad = torch.tensor([1, 2, 300, 4], dtype=torch.int32, device=DEV)
    blas.gemm_quant(Q8, 2, 2, 2, 1.0, 0.1, 0.1, bad, a, 0.0, c)
    with pytest.raises(qb.QuantError, match="outside"):
        blas.check_stream(c)
    blas.check_stream(c)  # reported once, then clear


def test_reference_literal_cases_on_the_gpu():
    """The reference's own literal cases (crates/sci/quanta-blas/src/reference.rs:1119-1148) through the C ABI."""
    c8 = kats.GEMM_Q8_SYM_BASIC
    c = torch.zeros(4, device=DEV)
    blas.gemm_quant(Q8, c8["m"], c8["n"], c8["k"], c8["alpha"], c8["a_scale"], c8["b_scale"], _dev_i32(np.array(c8["a"], np.int32)),
                    _dev_i32(np.array(c8["b"], np.int32)), c8["beta"], c)
    blas.check_stream(c)
    assert c.cpu().tolist() == c8["c"]
    c4 = kats.GEMM_Q4_SYM_BASIC
    c = torch.zeros(4, device=DEV)
    blas.gemm_quant4(Q4, c4["m"], c4["n"], c4["k"], c4["alpha"], c4["a_scale"], c4["b_scale"],
                     _dev_i32(bo.int4_pack_flat(np.array(c4["a"]))), _dev_i32(bo.int4_pack_flat(np.array(c4["b"]))), c4["beta"], c)
    blas.check_stream(c)
    assert c.cpu().tolist() == c4["c"]
