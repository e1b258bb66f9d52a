"""The quantized-GEMM oracle against the two literal cases the reference's own tests hold
(crates/sci/quanta-blas/src/reference.rs:1119-1148) and against exact integer arithmetic on the input family and
shapes of crates/sci/quanta-blas/tests/gemm_quant.rs, where every running sum is far below 2^24."""
import numpy as np
import pytest

import oracle as o
from oracle import blas_oracle as bo
from tests.golden import kats

Q8_CASES = [(4, 4, 4, 1.0, 0.0, 0.05, 0.05), (3, 5, 7, 1.0, 0.0, 0.1, 0.02), (6, 4, 5, 2.0, -1.0, 0.05, 0.05),
            (1, 8, 6, 1.0, 0.0, 0.05, 0.05), (8, 1, 6, 1.0, 0.0, 0.05, 0.05), (32, 24, 40, 1.0, 0.5, 0.02, 0.03)]
Q4_CASES = [(4, 4, 4, 1.0, 0.0, 0.1, 0.1), (3, 5, 7, 1.0, 0.0, 0.2, 0.05), (6, 4, 5, 2.0, -1.0, 0.1, 0.1),
            (16, 16, 24, 1.0, 0.5, 0.05, 0.08)]


def _exact(m, n, k, alpha, sa, sb, a, b, beta, c0):
    s = a.reshape(m, k).astype(np.int64) @ b.reshape(k, n).astype(np.int64)
    ae = np.float32(np.float32(alpha) * np.float32(sa)) * np.float32(sb)
    return ae * s.astype(np.float32) + np.float32(beta) * c0.reshape(m, n)


def test_input_family_is_its_own_quantization():
    L = o.lib()
    for bits, scale in [(8, 0.05), (8, 0.02), (4, 0.1), (4, 0.08)]:
        q = bo.test_matrix(16, 24, 2, bits)
        for v in q.reshape(-1)[:200]:
            assert L.qo_quantize_sym(np.float32(np.float32(v) * np.float32(scale)), np.float32(scale), bits) == v


@pytest.mark.parametrize("m,n,k,alpha,beta,sa,sb", Q8_CASES)
def test_q8_oracle_is_exact_on_the_reference_cases(m, n, k, alpha, beta, sa, sb):
    a, b = bo.test_matrix(m, k, 1, 8), bo.test_matrix(k, n, 2, 8)
    c0 = (np.arange(m * n, dtype=np.float32) * np.float32(0.25) - np.float32(1.0))
    got = bo.gemm_q8_sym(m, n, k, alpha, sa, sb, a, b, beta, c0)
    assert np.array_equal(got.view(np.uint32), _exact(m, n, k, alpha, sa, sb, a, b, beta, c0).astype(np.float32).view(np.uint32))


@pytest.mark.parametrize("m,n,k,alpha,beta,sa,sb", Q4_CASES)
def test_q4_oracle_unpacks_by_flat_index(m, n, k, alpha, beta, sa, sb):
    a, b = bo.test_matrix(m, k, 1, 4), bo.test_matrix(k, n, 2, 4)
    aw, bw = bo.int4_pack_flat(a), bo.int4_pack_flat(b)
    assert aw.size == (m * k + 7) // 8 and np.array_equal(bo.int4_unpack_flat(aw, m * k), a)
    c0 = (np.arange(m * n, dtype=np.float32) * np.float32(0.25) - np.float32(1.0))
    got = bo.gemm_q4_sym(m, n, k, alpha, sa, sb, aw, bw, beta, c0)
    assert np.array_equal(got.view(np.uint32), _exact(m, n, k, alpha, sa, sb, a, b, beta, c0).astype(np.float32).view(np.uint32))


def test_int4_flat_packing_matches_the_scalar_pack():
    L = o.lib()
    q = bo.test_matrix(3, 7, 5, 4)
    words = [0] * 3
    for i, v in enumerate(q.reshape(-1)):
        words[i // 8] = L.qo_int4_pack(words[i // 8], i % 8, int(v))
    assert list(bo.int4_pack_flat(q)) == words


def test_reference_literal_cases_pin_the_oracle():
    """gemm_q8_sym_basic / gemm_q4_sym_basic: literal inputs and outputs from the reference's tests."""
    c8 = kats.GEMM_Q8_SYM_BASIC
    got = bo.gemm_q8_sym(c8["m"], c8["n"], c8["k"], c8["alpha"], c8["a_scale"], c8["b_scale"], np.array(c8["a"], np.int32),
                         np.array(c8["b"], np.int32), c8["beta"], np.zeros(4, np.float32))
    assert got.reshape(-1).tolist() == c8["c"]
    c4 = kats.GEMM_Q4_SYM_BASIC
    L = o.lib()

    def pack(codes):  # int4_pack over nibbles 0..3 of one word, as the reference's test does
        w = 0
        for i, q in enumerate(codes):
            w = L.qo_int4_pack(w, i, q)
        return np.array([w], np.uint32)

    aw, bw = pack(c4["a"]), pack(c4["b"])
    assert np.array_equal(aw, bo.int4_pack_flat(np.array(c4["a"]))) and np.array_equal(bw, bo.int4_pack_flat(np.array(c4["b"])))
    got = bo.gemm_q4_sym(c4["m"], c4["n"], c4["k"], c4["alpha"], c4["a_scale"], c4["b_scale"], aw, bw, c4["beta"], np.zeros(4, np.float32))
    assert got.reshape(-1).tolist() == c4["c"]
