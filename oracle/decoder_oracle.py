"""CPU restatement of the decode step's support ops (TEST INFRASTRUCTURE ONLY; parity unpinned:
the reference holds no golden vectors for these ops on this path, so the checks are against this
restatement of its kernels' arithmetic, at a stated tolerance).

Each function follows the reference kernel it cites, in float32 with the reference's order of
operations where that matters (the online-softmax recurrence), vectorised over what is
independent.
"""
from __future__ import annotations

import numpy as np

F = np.float32


def rmsnorm(x, gamma, eps):
    """crates/ml/quanta-nn/src/norm.rs:192-225: rrms = 1 / sqrt(sum(x^2) / c + eps); out = x * rrms * gamma."""
    x = np.asarray(x, F)
    c = F(x.shape[-1])
    sq = np.zeros(x.shape[:-1], F)
    for p in range(x.shape[-1]):  # the reference accumulates sequentially in f32
        sq = (sq + x[..., p] * x[..., p]).astype(F)
    rrms = (F(1.0) / np.sqrt((sq / c + F(eps)).astype(F))).astype(F)
    return ((x * rrms[..., None]).astype(F) * np.asarray(gamma, F)).astype(F)


def rope_rows(pos, d, base=10000.0):
    """crates/sci/quanta-array/src/autograd/rope.rs:43-63: theta_i = pos * base^(-2i/d) in f64, cast to f32,
    the same value at i and i + d/2."""
    half = d // 2
    i = np.arange(half, dtype=np.float64)
    theta = float(pos) * np.power(float(base), -2.0 * i / float(d))
    c, s = np.cos(theta), np.sin(theta)
    return np.concatenate([c, c]).astype(F), np.concatenate([s, s]).astype(F)


def rope_apply(x, cosv, sinv):
    """crates/ml/quanta-nn/src/rope.rs:23-58 (sign = +1): out[j] = x[j] cos[j] + pm x[partner] sin[j],
    partner = j + d/2 with pm = -1 for j < d/2, partner = j - d/2 with pm = +1 otherwise."""
    x = np.asarray(x, F)
    d = x.shape[-1]
    half = d // 2
    partner = np.concatenate([x[..., half:], x[..., :half]], axis=-1)
    pm = np.concatenate([-np.ones(half, F), np.ones(half, F)])
    return ((x * cosv).astype(F) + ((pm * partner).astype(F) * sinv).astype(F)).astype(F)


def sdpa_one_query(q, k, v, scale, kv_len):
    """crates/ml/quanta-nn/src/kernel.rs:64-175 for one query row, no causal mask: the online-softmax
    recurrence over the keys in order, float32, masked keys biased by -1e9."""
    q, k, v = np.asarray(q, F), np.asarray(k, F), np.asarray(v, F)
    m, l = F(0), F(0)
    acc = np.zeros(v.shape[-1], F)
    for kj in range(k.shape[0]):
        dot = F(0)
        for p in range(q.shape[0]):
            dot = F(dot + q[p] * k[kj, p])
        raw = F(scale) * dot
        valid = F(1.0) if kj < kv_len else F(0.0)
        sk = F(raw + (F(1.0) - valid) * F(-1000000000.0))
        if kj == 0:
            m_new, a = sk, F(0)
        else:
            m_new = max(m, sk)
            a = F(np.exp(min(F(m - m_new), F(0))))
        b = F(np.exp(min(F(sk - m_new), F(0))))
        l = F(l * a + b)
        acc = (acc * a + b * v[kj]).astype(F)
        m = m_new
    return (acc / l).astype(F)


def swiglu(a, b):
    """crates/ml/quanta-nn/src/activation.rs:145-162: s = 1 / (1 + exp(min(-a, 30))); out = a * s * b."""
    a, b = np.asarray(a, F), np.asarray(b, F)
    s = (F(1.0) / (F(1.0) + np.exp(np.minimum(-a, F(30.0))).astype(F))).astype(F)
    return ((a * s).astype(F) * b).astype(F)
