"""CPU restatement of the reference's quantized-GEMM oracle (TEST INFRASTRUCTURE ONLY).

``gemm_q8_sym`` / ``gemm_q4_sym`` follow crates/sci/quanta-blas/src/reference.rs:104-131 (the shared narrow GEMM:
codes cast to f32, the inner product accumulated in f32 left to right, ``alpha_eff * acc + beta * c`` in f32),
:212-226 and :235-262.  The loop over k is kept sequential; rows and columns are vectorised, which does not
change any entry's order of operations.

Parity pin: the two literal cases of the reference's own tests for these functions (``gemm_q8_sym_basic`` and
``gemm_q4_sym_basic``, crates/sci/quanta-blas/src/reference.rs:1119-1148) are reproduced in ``tests/golden/kats.py`` and
checked in ``tests/test_blas_oracle.py``; the device tests of the reference (crates/sci/quanta-blas/tests/gemm_quant.rs)
compare the device with this very function on inputs whose running sums stay far below 2^24, where f32 accumulation
is integer arithmetic, and the same file checks the restatement against exact integer sums on those inputs.
"""
from __future__ import annotations

import numpy as np


def int4_unpack_flat(words: np.ndarray, count: int) -> np.ndarray:
    """Element i = nibble ``i % 8`` of word ``i // 8``, sign extended (reference.rs:248-249)."""
    w = np.ascontiguousarray(words).view(np.uint32).reshape(-1)
    idx = np.arange(count, dtype=np.int64)
    nib = ((w[idx >> 3] >> (4 * (idx & 7)).astype(np.uint32)) & 0xF).astype(np.int32)
    return np.where(nib >= 8, nib - 16, nib).astype(np.int32)


def int4_pack_flat(codes: np.ndarray) -> np.ndarray:
    q = np.asarray(codes, dtype=np.int64).reshape(-1)
    out = np.zeros((q.size + 7) // 8, dtype=np.uint32)
    for j in range(8):
        part = (q[j::8] & 0xF).astype(np.uint32) << np.uint32(4 * j)
        out[: part.size] |= part
    return out


def _gemm_narrow(m, n, k, alpha_eff, a_codes, b_codes, beta, c):
    a = np.asarray(a_codes, dtype=np.int32).reshape(m, k).astype(np.float32)
    b = np.asarray(b_codes, dtype=np.int32).reshape(k, n).astype(np.float32)
    acc = np.zeros((m, n), dtype=np.float32)
    for p in range(k):
        acc = acc + a[:, p: p + 1] * b[p: p + 1, :]  # product exact in f32 for 8-bit codes; one rounding per add
    c = np.asarray(c, dtype=np.float32).reshape(m, n)
    return (np.float32(alpha_eff) * acc + np.float32(beta) * c).astype(np.float32)


def gemm_q8_sym(m, n, k, alpha, a_scale, b_scale, a, b, beta, c):
    """reference.rs:212-226.  Returns the new C ``[m, n]``."""
    alpha_eff = np.float32(np.float32(alpha) * np.float32(a_scale)) * np.float32(b_scale)
    return _gemm_narrow(m, n, k, alpha_eff, a, b, beta, c)


def gemm_q4_sym(m, n, k, alpha, a_scale, b_scale, a_words, b_words, beta, c):
    """reference.rs:235-262: packed words, unpacked by flat index."""
    a_words, b_words = np.asarray(a_words), np.asarray(b_words)
    assert a_words.size == (m * k + 7) // 8 and b_words.size == (k * n + 7) // 8
    alpha_eff = np.float32(np.float32(alpha) * np.float32(a_scale)) * np.float32(b_scale)
    return _gemm_narrow(m, n, k, alpha_eff, int4_unpack_flat(a_words, m * k), int4_unpack_flat(b_words, k * n), beta, c)


def test_matrix(rows: int, cols: int, seed: int, bits: int) -> np.ndarray:
    """The input family of the reference's tests (gemm_quant.rs:26-35, 124-132): code i is
    ``x = ((i * 2654435761 mod 2^32) xor seed) mod span - span / 2`` with span 64 (int8) or 16 (int4), then
    ``quantize_sym(x * s, s, bits)``, which is x itself for these integers (checked in the CPU tests)."""
    span = 64 if bits == 8 else 16
    i = np.arange(rows * cols, dtype=np.uint64)
    x = (((i * np.uint64(2654435761)) & np.uint64(0xFFFFFFFF)) ^ np.uint64(seed)) % np.uint64(span)
    q = x.astype(np.int32) - span // 2
    lo, hi = (-128, 127) if bits == 8 else (-8, 7)
    return np.clip(q, lo, hi).astype(np.int32)
