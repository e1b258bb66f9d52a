"""The decode step's support ops against the CPU restatement of the reference kernels, and the
Llama-shaped stack end to end against the same ops composed in torch."""
import math

import numpy as np
import pytest
import torch

import oracle as o
from oracle import decoder_oracle as do
import quanta_b200 as qb
from quanta_b200 import decoder as dec

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bf(a):
    return o.bf16_to_f32(o.f32_to_bf16(np.asarray(a, np.float32)))


def close(got, want, tol):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want) - tol * (1 + np.abs(want))
    assert (err <= 0).all(), f"max excess {err.max():.3e}"


def test_add_rmsnorm_against_reference_arithmetic():
    rng = np.random.default_rng(1)
    for n, c in [(1, 128), (16, 4096), (3, 1000)]:
        h = rng.standard_normal((n, c)).astype(np.float32)
        d = rng.standard_normal((n, c)).astype(np.float32)
        g = rng.standard_normal(c).astype(np.float32)
        ht = torch.from_numpy(h).to(DEV)
        out = dec.add_rmsnorm(ht, torch.from_numpy(d).to(DEV), torch.from_numpy(g).to(DEV), 1e-5)
        s = (h + d).astype(np.float32)
        assert np.array_equal(ht.cpu().numpy(), s)  # the residual sum is one f32 add
        want = do.rmsnorm(s, g, 1e-5)
        close(out.to(torch.float32).cpu().numpy(), want, 1e-2)  # bf16 output: 2^-8 relative
        out2 = dec.add_rmsnorm(ht, None, torch.from_numpy(g).to(DEV), 1e-5)
        assert torch.equal(out, out2)
        # a delta in parts is summed first
        parts = rng.standard_normal((3, n, c)).astype(np.float32)
        h3 = torch.from_numpy(h).to(DEV)
        dec.add_rmsnorm(h3, torch.from_numpy(parts).to(DEV), torch.from_numpy(g).to(DEV), 1e-5)
        assert np.array_equal(h3.cpu().numpy(), (h + ((parts[0] + parts[1]).astype(np.float32) + parts[2]).astype(np.float32)).astype(np.float32))


def test_rope_append_and_sdpa_decode():
    rng = np.random.default_rng(2)
    b, heads, hd, ctx_max, pos = 3, 4, 128, 300, 257
    q = rng.standard_normal((b, heads * hd)).astype(np.float32)
    k = rng.standard_normal((b, heads * hd)).astype(np.float32)
    v = rng.standard_normal((b, heads * hd)).astype(np.float32)
    kc = bf(rng.standard_normal((b, ctx_max, heads, hd)))
    vc = bf(rng.standard_normal((b, ctx_max, heads, hd)))
    c, s = dec.rope_rows(pos, hd)
    c2, s2 = do.rope_rows(pos, hd)
    assert np.array_equal(c, c2) and np.array_equal(s, s2)
    t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).to(DEV) if dt is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dt)
    kct, vct = t(kc, torch.bfloat16), t(vc, torch.bfloat16)
    q_out = torch.empty(b, heads * hd, dtype=torch.bfloat16, device=DEV)
    dec.rope_append(t(q), t(k), t(v), t(c), t(s), heads, q_out, kct, vct, pos)
    q_want = bf(do.rope_apply(q.reshape(b, heads, hd), c, s)).reshape(b, heads * hd)
    k_want = bf(do.rope_apply(k.reshape(b, heads, hd), c, s))
    assert np.array_equal(q_out.to(torch.float32).cpu().numpy(), q_want)  # f32 mul/add in the reference's order, then bf16
    assert np.array_equal(kct[:, pos].to(torch.float32).cpu().numpy(), k_want)
    assert np.array_equal(vct[:, pos].to(torch.float32).cpu().numpy(), bf(v).reshape(b, heads, hd))
    kc[:, pos], vc[:, pos] = k_want, bf(v).reshape(b, heads, hd)
    assert np.array_equal(kct.to(torch.float32).cpu().numpy(), kc)  # nothing else was touched
    # attention over the first pos + 1 cache rows
    kv_len, scale = pos + 1, 1.0 / math.sqrt(hd)
    out = torch.empty(b, heads * hd, dtype=torch.bfloat16, device=DEV)
    dec.sdpa_decode(q_out, kct, vct, kv_len, scale, dec.sdpa_scratch(b, heads, kv_len, DEV), out)
    got = out.to(torch.float32).cpu().numpy().reshape(b, heads, hd)
    for bi in range(b):
        for h in range(heads):
            want = do.sdpa_one_query(q_want.reshape(b, heads, hd)[bi, h], kc[bi, :, h], vc[bi, :, h], scale, kv_len)
            close(got[bi, h], want, 1e-2)


@pytest.mark.parametrize("b,heads,kv_len", [(16, 16, 200), (8, 40, 3), (2, 4, 1025), (1, 1, 130), (37, 7, 65)])
def test_sdpa_decode_shapes(b, heads, kv_len):
    """Many and few (row, head) pairs, one key split and many, a ragged last split: against the restatement."""
    rng = np.random.default_rng(b * 100 + heads)
    hd, ctx_max = 128, kv_len + 3
    q = bf(rng.standard_normal((b, heads, hd)))
    kc = bf(rng.standard_normal((b, ctx_max, heads, hd)))
    vc = bf(rng.standard_normal((b, ctx_max, heads, hd)))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty(b, heads * hd, dtype=torch.bfloat16, device=DEV)
    dec.sdpa_decode(t(q.reshape(b, heads * hd)), t(kc), t(vc), kv_len, scale, dec.sdpa_scratch(b, heads, kv_len, DEV), out)
    got = out.to(torch.float32).cpu().numpy().reshape(b, heads, hd)
    for bi in range(0, b, max(1, b // 3)):
        for h in range(0, heads, max(1, heads // 3)):
            close(got[bi, h], do.sdpa_one_query(q[bi, h], kc[bi, :, h], vc[bi, :, h], scale, kv_len), 1e-2)


def test_swiglu_sliced_and_sum():
    rng = np.random.default_rng(3)
    n, h, widths = 5, 1408, [512, 512, 384]
    a = (rng.standard_normal((n, h)) * 8).astype(np.float32)
    a[0, :4] = [40.0, -40.0, 100.0, -100.0]  # the clamp
    b = rng.standard_normal((n, h)).astype(np.float32)
    out = torch.empty(n * h, dtype=torch.bfloat16, device=DEV)
    dec.swiglu_sliced(torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV), widths, out)
    want = do.swiglu(a, b)
    got = out.to(torch.float32).cpu().numpy()
    off, col = 0, 0
    for w in widths:
        close(got[off: off + n * w].reshape(n, w), want[:, col: col + w], 1e-2)
        off, col = off + n * w, col + w
    padded = torch.full((3, n, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    dec.swiglu_sliced(torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV), widths, padded, 512)
    pg = padded.to(torch.float32).cpu().numpy()
    col = 0
    for i, w in enumerate(widths):
        close(pg[i, :, :w], want[:, col: col + w], 1e-2)
        assert (pg[i, :, w:] == 7.0).all()  # padding columns untouched
        col += w
    parts = rng.standard_normal((3, n, 64)).astype(np.float32)
    y = torch.empty(n, 64, device=DEV)
    dec.sum_arrays(torch.from_numpy(parts).to(DEV), y)
    assert np.array_equal(y.cpu().numpy(), ((parts[0] + parts[1]).astype(np.float32) + parts[2]).astype(np.float32))


def test_decoder_stack_against_torch_composition():
    """Two blocks of a small Llama-shaped stack: the kernels strung together against torch ops over the
    bit-exact dequantized weights with bf16 rounding at the same places."""
    torch.manual_seed(0)
    st = dec.DecoderStack(n_layers=2, d=256, heads=2, ffn=1408, vocab=640, batch=4, ctx_max=40, device=torch.device(DEV))
    pos = 17
    st.set_position(pos)
    h0 = torch.randn(4, 256, device=DEV)
    k0, v0 = st.kcache.clone(), st.vcache.clone()
    logits = st.step(h0).clone()

    def rb(x):
        return x.to(torch.bfloat16).to(torch.float32)

    def lin(ql, x):
        return x @ ql._w.dequantize().t()

    def norm(h, g):
        return rb(h * torch.rsqrt((h * h).mean(-1, keepdim=True) + st.eps) * g)

    c, s = [torch.from_numpy(a).to(DEV) for a in dec.rope_rows(pos, 128)]

    def rope(x):
        x = x.view(4, 2, 128)
        partner = torch.cat([x[..., 64:], x[..., :64]], -1)
        pm = torch.cat([-torch.ones(64, device=DEV), torch.ones(64, device=DEV)])
        return x * c + pm * partner * s

    h = h0.clone()
    for li, blk in enumerate(st.layers):
        xn = norm(h, blk["g1"])
        q, k, v = [lin(ql, xn) for ql in blk["qkv"]]
        qr, kr = rb(rope(q)), rb(rope(k))
        kc, vc = k0[li].to(torch.float32), v0[li].to(torch.float32)
        kc[:, pos], vc[:, pos] = kr, rb(v).view(4, 2, 128)
        att = torch.einsum("bhd,bthd->bht", qr, kc[:, : pos + 1]) / math.sqrt(128)
        att = torch.einsum("bht,bthd->bhd", torch.softmax(att, -1), vc[:, : pos + 1])
        h = h + lin(blk["o"], rb(att.reshape(4, 256)))
        xn = norm(h, blk["g2"])
        g, u = [lin(ql, xn) for ql in blk["gate_up"]]
        act = rb(g * torch.sigmoid(g) * u)
        col, down = 0, 0
        for ql, w in zip(blk["down"], st.down_widths):
            down = down + act[:, col: col + w] @ ql._w.dequantize().t()[:w]
            col += w
        h = h + down
    want = lin(st.lm_head, norm(h, st.g_final))
    assert bool(((logits - want).abs() <= 2e-2 * (1 + want.abs())).all()), float((logits - want).abs().max())
