"""Host-side pieces of the decode step that need no GPU: the RoPE table and the column slicing of a wide linear."""
import numpy as np

from oracle import decoder_oracle as do
from quanta_b200 import decoder as dec


def test_rope_rows_match_the_restatement_and_the_reference_formula():
    for pos, d in [(0, 128), (1, 128), (1024, 128), (77, 64)]:
        c, s = dec.rope_rows(pos, d)
        c2, s2 = do.rope_rows(pos, d)
        assert c.dtype == np.float32 and np.array_equal(c, c2) and np.array_equal(s, s2)
        half = d // 2
        assert np.array_equal(c[:half], c[half:]) and np.array_equal(s[:half], s[half:])  # a pair shares its angle
        theta = pos * 10000.0 ** (-2.0 * 3 / d)  # crates/sci/quanta-array/src/autograd/rope.rs:52-60, i = 3
        assert c[3] == np.float32(np.cos(theta)) and s[3] == np.float32(np.sin(theta))
    c, s = dec.rope_rows(0, 128)
    assert (c == 1).all() and (s == 0).all()


def test_split_groups_covers_the_width_in_whole_groups():
    for width, n in [(128, 1), (4096, 1), (4224, 2), (11008, 3), (14336, 4), (28672, 7), (1408, 1)]:
        w = dec._split_groups(width // 128, n)
        assert sum(w) == width and all(x % 128 == 0 and 0 < x <= 4096 for x in w)
        assert len(w) == n and max(w) - min(w) <= 128
    assert dec._split_groups(86, 3) == [3712, 3712, 3584]


def test_oracle_ops_agree_with_float64_math():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 64)).astype(np.float32)
    g = rng.standard_normal(64).astype(np.float32)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * g
    assert np.allclose(do.rmsnorm(x, g, 1e-5), want, rtol=1e-5, atol=1e-6)
    q = rng.standard_normal(16).astype(np.float32)
    k = rng.standard_normal((9, 16)).astype(np.float32)
    v = rng.standard_normal((9, 16)).astype(np.float32)
    sc = (k[:7].astype(np.float64) @ q) * 0.25
    p = np.exp(sc - sc.max())
    assert np.allclose(do.sdpa_one_query(q, k, v, 0.25, 7), (p / p.sum()) @ v[:7], rtol=1e-5, atol=1e-6)  # keys 7, 8 masked
    a = np.array([-100.0, -1.0, 0.0, 2.0, 100.0], np.float32)
    assert np.allclose(do.swiglu(a, np.ones(5, np.float32)), a / (1 + np.exp(np.minimum(-a.astype(np.float64), 30))), rtol=1e-6, atol=1e-12)
    c, s = do.rope_rows(5, 8)
    xr = do.rope_apply(x[:, :8], c, s)
    assert np.allclose((xr ** 2).sum(-1), (x[:, :8] ** 2).sum(-1), rtol=1e-5)  # a rotation keeps the norm
