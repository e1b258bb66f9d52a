"""Parity of the CUDA path (through the C ABI) against the CPU oracle.

Bit-exact for codes, scales and dequantized weights; the reference's own tolerance form
|got - want| <= tol * (1 + |want|) (crates/sci/quanta-blas/tests/gemm_quant.rs:74-79) for
the forward: 1e-4 for f32 activations, 1e-3 where bf16 staging is involved."""
import numpy as np
import pytest
import torch

import oracle as o
import quanta_b200 as qb
from tests.golden import kats

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def codes_np(m):
    c = m.codes().cpu().numpy()
    return c if c.dtype == np.int8 else c.view(np.uint32)


def gran_of(kind, axis, size):
    return qb.Granularity(kind, axis, size)


def quantize_both(w, rows, cols, dtype, gran):
    """(device QuantizedMatrix, oracle codes, oracle scales) on the same input."""
    gr, gc = gran.tile(rows, cols)
    m = qb.QuantizedMatrix.quantize(t(np.asarray(w, np.float32).reshape(rows, cols)), dtype, gran)
    oc, os_ = o.quantize_host(w, rows, cols, dtype.bits(), gr, gc)
    return m, oc, os_


def assert_quant_equal(m, oc, os_, ctx=""):
    assert (codes_np(m) == oc).all(), f"{ctx}: codes differ"
    assert (bits(m.scales().cpu().numpy()) == bits(os_)).all(), f"{ctx}: scales differ"


def close(got, want, tol):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want) - tol * (1 + np.abs(want))
    assert (err <= 0).all(), f"max excess {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}"


# ---- quantize / dequantize: the reference's own shape grid -------------------

@pytest.mark.parametrize("r,c,g", kats.DEVICE_HOST_SHAPES)
def test_device_matches_host_shape_grid(r, c, g):
    # quanta-array/tests/quant.rs:75-115 — 2 dtypes x 5 spellings
    w = kats.weights(r * c)
    for dtype in (qb.QuantDtype.Int8, qb.QuantDtype.Int4):
        for kind, axis, size in kats.spellings(g):
            gran = gran_of(kind, axis, size)
            m, oc, os_ = quantize_both(w, r, c, dtype, gran)
            ctx = f"[{r},{c}] {dtype.name} {gran!r}"
            assert_quant_equal(m, oc, os_, ctx)
            gr, gc = gran.tile(r, c)
            host = o.dequantize_host(oc, os_, r, c, dtype.bits(), gr, gc)
            dev = m.dequantize().cpu().numpy()
            assert dev.shape == (r, c)
            assert (bits(dev) == bits(host)).all(), ctx


@pytest.mark.parametrize("case,dtype", [(kats.RTE_INT8, qb.QuantDtype.Int8), (kats.RTE_INT4, qb.QuantDtype.Int4)])
def test_ties_to_even_pinned(case, dtype):
    m = qb.QuantizedMatrix.quantize(t(np.array(case["w"], np.float32).reshape(2, 4)), dtype, qb.PerTensor())
    assert m.scales().cpu().tolist() == [[case["scale"]]]
    assert (bits(m.dequantize().cpu().numpy().reshape(-1)) == bits(case["deq"])).all()


@pytest.mark.parametrize("case", [kats.NIBBLE_ORDER, kats.ROW_PACKING])
def test_int4_nibble_contract(case):
    r, c = case["rows"], case["cols"]
    m = qb.QuantizedMatrix.quantize(t(np.array(case["w"], np.float32).reshape(r, c)), qb.QuantDtype.Int4, qb.PerTensor())
    assert codes_np(m).reshape(-1).tolist() == case["words"]
    assert (bits(m.dequantize().cpu().numpy().reshape(-1)) == bits(case["w"])).all()


def test_exact_multiples_and_op_matrix():
    for ints, dtype in [(kats.EXACT_INT8, qb.QuantDtype.Int8), (kats.EXACT_INT4, qb.QuantDtype.Int4)]:
        m = qb.QuantizedMatrix.quantize(t(np.array(ints, np.float32).reshape(2, 4)), dtype, qb.PerTensor())
        assert m.scales().cpu().reshape(-1).tolist() == [1.0]
        assert (bits(m.dequantize().cpu().numpy().reshape(-1)) == bits(ints)).all()
    # op-matrix: every representable code dequantizes exactly at scale 0.5
    for b, dt in [(8, torch.int8), (4, torch.int32)]:
        lo, hi = kats.QUANT_RANGES[b]
        vals = list(range(lo, hi + 1))
        n = len(vals)
        if b == 8:
            codes = torch.tensor(vals, dtype=torch.int8).reshape(1, n)
        else:
            words = []
            for i in range(0, n, 8):
                w = 0
                for j, v in enumerate(vals[i:i + 8]):
                    w |= (v & 0xF) << (4 * j)
                words.append(w)
            codes = torch.from_numpy(np.array(words, np.uint32).view(np.int32)).reshape(1, -1)
        m = qb.QuantizedMatrix.from_parts(codes.to(DEV), [1, n], torch.tensor([[0.5]], device=DEV), qb.PerTensor())
        want = np.float32(0.5) * np.array(vals, np.float32)
        assert (bits(m.dequantize().cpu().numpy().reshape(-1)) == bits(want)).all()


def test_from_parts_dequantizes():
    c8 = torch.tensor(kats.FROM_PARTS_INT8["codes"], dtype=torch.int8).reshape(2, 2).to(DEV)
    s = torch.tensor(kats.FROM_PARTS_INT8["scales"]).reshape(2, 1).to(DEV)
    assert qb.QuantizedMatrix.from_parts(c8, [2, 2], s, qb.PerChannel(0)).dequantize().cpu().reshape(-1).tolist() == \
        kats.FROM_PARTS_INT8["deq"]
    c4 = torch.tensor(kats.FROM_PARTS_INT4["words"], dtype=torch.int32).reshape(2, 1).to(DEV)
    assert qb.QuantizedMatrix.from_parts(c4, [2, 2], s, qb.PerChannel(0)).dequantize().cpu().reshape(-1).tolist() == \
        kats.FROM_PARTS_INT4["deq"]


def test_all_zero_tile_and_specials():
    w = kats.weights(16)
    w[8] = w[9] = 0.0
    m, oc, os_ = quantize_both(w, 4, 4, qb.QuantDtype.Int8, qb.Group(1, 2))
    assert_quant_equal(m, oc, os_)
    assert m.scales().cpu()[2, 0] == 0.0
    d = m.dequantize().cpu().numpy()
    assert bits(d)[2, 0] == 0 and bits(d)[2, 1] == 0
    # NaN contributes nothing to the scale and quantizes to 0; inf gives s = inf, codes 0
    for special in (np.nan, np.inf, -np.inf):
        for shape, gran in [((4, 64), qb.Group(1, 16)), ((5, 7), qb.PerChannel(0)), ((64, 64), qb.Block(32, 32))]:
            w = np.random.default_rng(3).standard_normal(shape).astype(np.float32)
            w[1, 3] = special
            w[shape[0] - 1, shape[1] - 1] = -0.0
            for dtype in (qb.QuantDtype.Int8, qb.QuantDtype.Int4):
                m, oc, os_ = quantize_both(w, *shape, dtype, gran)
                assert_quant_equal(m, oc, os_, f"{special} {shape} {gran!r}")
    # denormal scales survive (no flush-to-zero)
    w = (np.random.default_rng(4).standard_normal((8, 128)) * 1e-39).astype(np.float32)
    m, oc, os_ = quantize_both(w, 8, 128, qb.QuantDtype.Int4, qb.Group(1, 128))
    assert_quant_equal(m, oc, os_, "denormal")


@pytest.mark.parametrize("shape,gran", [
    ((256, 512), qb.Group(1, 128)), ((256, 512), qb.Block(32, 32)), ((96, 200), qb.Block(32, 32)),
    ((64, 1024), qb.Group(1, 256)), ((64, 1024), qb.PerChannel(0)), ((300, 72), qb.Group(0, 128)),
    ((128, 136), qb.Group(1, 64)), ((33, 130), qb.Group(1, 128)), ((1, 8), qb.PerTensor()), ((130, 9), qb.Block(64, 4)),
    ((512, 64), qb.Block(256, 8)), ((77, 4096), qb.Group(1, 2048)),
])
def test_quantize_paths_bit_exact(shape, gran):
    rng = np.random.default_rng(hash(shape) & 0xFFFF)
    w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    for dtype in (qb.QuantDtype.Int8, qb.QuantDtype.Int4):
        m, oc, os_ = quantize_both(w, *shape, dtype, gran)
        assert_quant_equal(m, oc, os_, f"{shape} {gran!r} {dtype.name}")
        gr, gc = gran.tile(*shape)
        assert (bits(m.dequantize().cpu().numpy()) == bits(o.dequantize_host(oc, os_, *shape, dtype.bits(), gr, gc))).all()


@pytest.mark.parametrize("dtype,gran", [(qb.QuantDtype.Int4, qb.Group(1, 128)), (qb.QuantDtype.Int8, qb.Block(32, 32)),
                                        (qb.QuantDtype.Int8, qb.Group(1, 128))])
def test_quantize_near_ties_bit_exact(dtype, gran):
    """The tile kernel rounds x * (1 / s) and falls back to the exact divide near half-integers: weights placed
    on and within a few ulps of every rounding boundary k + 0.5 (and of every integer), for scales across the
    f32 range, must still give the reference's codes bit for bit."""
    hi = 127 if dtype.bits() == 8 else 7
    rows, cols = 256, 256
    rng = np.random.default_rng(17)
    w = np.zeros((rows, cols), np.float32)
    for r in range(rows):
        # per row: a scale magnitude anywhere from subnormal-ish to huge, every column block shares it
        m = np.float32(rng.uniform(0.5, 2.0) * 2.0 ** int(rng.integers(-120, 100)))
        s = np.float32(m / np.float32(hi))
        ks = rng.integers(-hi - 1, hi + 1, size=cols).astype(np.float32)
        frac = rng.choice(np.array([0.5, 0.5, 0.5, 0.0, 0.25], np.float32), size=cols)
        x = (ks + frac).astype(np.float32) * s
        ulps = rng.integers(-6, 7, size=cols)
        xi = x.view(np.int32) + ulps.astype(np.int32)  # step by a few ulps either way
        x = np.clip(xi.view(np.float32), -m, m).astype(np.float32)
        x[::32] = m  # every tile of either grid holds the row's maximum, so s is the tile's scale
        w[r] = x
    m_, oc, os_ = quantize_both(w, rows, cols, dtype, gran)
    assert_quant_equal(m_, oc, os_, f"near ties {dtype.name} {gran!r}")


def test_quantize_from_half_sources():
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((64, 256)) * 0.02).astype(np.float32)
    for tdt in (torch.bfloat16, torch.float16):
        src = torch.from_numpy(w).to(tdt)
        exact = src.to(torch.float32).numpy()
        for dtype, gran in [(qb.QuantDtype.Int4, qb.Group(1, 128)), (qb.QuantDtype.Int8, qb.PerTensor())]:
            m = qb.QuantizedMatrix.quantize(src.to(DEV), dtype, gran)
            gr, gc = gran.tile(64, 256)
            oc, os_ = o.quantize_host(exact, 64, 256, dtype.bits(), gr, gc)
            assert_quant_equal(m, oc, os_, f"{tdt}")


# ---- the benchmark workloads at oracle-sized inputs -----------------------------------

def test_config1_int8_block32_cpu_runnable():
    g = np.random.default_rng(0)
    w = (g.standard_normal((1024, 1024), dtype=np.float32) * np.float32(0.02))
    x = g.standard_normal((8, 1024), dtype=np.float32)
    m, oc, os_ = quantize_both(w, 1024, 1024, qb.QuantDtype.Int8, qb.Block(32, 32))
    assert_quant_equal(m, oc, os_)
    assert codes_np(m).min() >= -127 and codes_np(m).max() <= 127
    wd = o.dequantize_host(oc, os_, 1024, 1024, 8, 32, 32)
    assert (bits(m.dequantize().cpu().numpy()) == bits(wd)).all()
    ql = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
    y = ql.forward(t(x)).cpu().numpy()
    close(y, o.linear_forward(x, wd, None, o.OUT_IN, threads=8), 1e-4)
    yh = ql.forward_host(x)
    assert (bits(yh) == bits(y)).all()


@pytest.mark.parametrize("M", [1, 4, 16])
def test_config2_int4_decode_shapes(M):
    g = np.random.default_rng(1)
    w = g.standard_normal((4096, 4096), dtype=np.float32) * np.float32(0.02)
    x = g.standard_normal((16, 4096), dtype=np.float32)
    xb = o.f32_to_bf16(x)[:M]
    m, oc, os_ = quantize_both(w, 4096, 4096, qb.QuantDtype.Int4, qb.Group(1, 128))
    assert_quant_equal(m, oc, os_)
    assert m.scales().shape == (4096, 32)
    wd = o.dequantize_host(oc, os_, 4096, 4096, 4, 1, 128)
    ql = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
    xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
    y = ql.forward(xt, out_dtype=torch.float32).cpu().numpy()
    want = o.linear_forward(o.bf16_to_f32(xb), wd, None, o.OUT_IN, threads=8)
    close(y, want, 1e-3)


# ---- QuantizedLinear == Linear(deq w), every orientation / dtype / grid ---------

@pytest.mark.parametrize("layout", [qb.IN_OUT, qb.OUT_IN])
@pytest.mark.parametrize("dtype,gran,shape", [
    (qb.QuantDtype.Int8, qb.PerChannel(1), (6, 4)), (qb.QuantDtype.Int4, qb.Group(0, 3), (6, 4)),
    (qb.QuantDtype.Int4, qb.Group(0, 8), (64, 40)), (qb.QuantDtype.Int8, qb.PerTensor(), (33, 17)),
    (qb.QuantDtype.Int4, qb.Group(1, 128), (96, 256)), (qb.QuantDtype.Int8, qb.Block(32, 32), (128, 96)),
    (qb.QuantDtype.Int4, qb.Group(0, 128), (1024, 520)), (qb.QuantDtype.Int8, qb.Group(1, 64), (40, 1024)),
])
def test_quantized_linear_matches_linear_of_dequantized(layout, dtype, gran, shape):
    # quanta-nn/tests/quant.rs:467-524 (the reference claims bitwise for its f32 chain; the fused
    # kernels accumulate in a different order, so the stated 1e-4 bound applies)
    r, c = shape
    w = kats.fill(r * c, 21).reshape(r, c)
    in_dim, out_dim = (r, c) if layout == qb.IN_OUT else (c, r)
    b = kats.fill(out_dim, 22)
    m, oc, os_ = quantize_both(w, r, c, dtype, gran)
    gr, gc = gran.tile(r, c)
    wd = o.dequantize_host(oc, os_, r, c, dtype.bits(), gr, gc)
    for M in (1, 3, 9):
        x = kats.fill(M * in_dim, 9 + M).reshape(M, in_dim)
        want = o.linear_forward(x, wd, b, layout)
        ql = qb.QuantizedLinear.new(m, t(b), layout)
        assert ql.in_dim() == in_dim and ql.out_dim(in_dim) == out_dim and ql.init() == ()
        y = ql.apply(None, (), t(x)).cpu().numpy()
        close(y, want, 1e-4)
        # Mode A (dequantized once) agrees with Mode B
        ya = qb.QuantizedLinear.dequantized(m, t(b), layout).forward(t(x)).cpu().numpy()
        close(ya, want, 1e-4)
        # bf16 activations in / out
        xb = o.f32_to_bf16(x)
        yb = ql.forward(torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV))
        wantb = o.linear_forward(o.bf16_to_f32(xb), wd, b, layout)
        close(yb.to(torch.float32).cpu().numpy(), wantb, 1e-2)  # bf16 output rounding: 2^-9 relative
        assert yb.dtype == torch.bfloat16


def test_trained_linear_round_trip_bound():
    # quanta-nn/tests/quant.rs:543-663, with the trained weight replaced by a seeded one:
    # |dy| <= sum_k |x_k| s/2 * 1.001 + 1e-6
    n, k, mo = 8, 4, 3
    x = kats.fill(n * k, 11).reshape(n, k)
    w = kats.fill(k * mo, 12).reshape(k, mo)
    b = kats.fill(mo, 13)
    y_f = o.linear_forward(x, w, b, o.IN_OUT)
    for dtype, gran in [(qb.QuantDtype.Int8, qb.PerChannel(1)), (qb.QuantDtype.Int4, qb.Group(0, 2))]:
        entries = qb.quantize_named([("w", t(w)), ("b", t(b))], lambda name, a: (dtype, gran) if name == "w" else None)
        data = qb.save_named(entries, None)
        restored = qb.load(DEV, {"w": torch.zeros(k, mo), "b": torch.zeros(mo)}, data)
        y_a = (t(x) @ restored["w"] + restored["b"]).cpu().numpy()
        loaded = qb.load_named(DEV, data)
        leaves = dict(loaded.leaves)
        mq = leaves["w"].value
        ql = qb.QuantizedLinear.new(mq, leaves["b"].value)
        y_b = ql.forward(t(x)).cpu().numpy()
        close(y_b, y_a, 1e-5)
        gr, gc = mq.tile()
        s = mq.scales().cpu().numpy()
        for i in range(n):
            for j in range(mo):
                bound = sum(abs(float(x[i, kk])) * float(s[kk // gr, j // gc]) / 2 for kk in range(k))
                assert abs(float(y_b[i, j]) - float(y_f[i, j])) <= bound * 1.001 + 1e-6


def test_mode_a_load_equals_device_dequantize_bitwise():
    # quanta-nn/tests/quant.rs:239-276
    entries = []
    for name, kind, shape, vals in kats.REFERENCE_ENTRIES:
        a = t(np.array(vals, np.float32).reshape(shape))
        if kind == "f32":
            entries.append((name, qb.QuantLeaf.F32(a)))
        else:
            dt = qb.QuantDtype.Int8 if kind == "q8" else qb.QuantDtype.Int4
            entries.append((name, qb.QuantLeaf.Quantized(qb.QuantizedMatrix.quantize(a, dt, qb.PerTensor()))))
    data = qb.save_named(entries, None)
    assert data == kats.reference_quantized_bytes()
    loaded = qb.load_named_f32(DEV, data)
    for (name, leaf), (lname, arr) in zip(entries, loaded.tensors):
        assert name == lname
        want = leaf.value.dequantize() if leaf.is_quantized else leaf.value
        assert list(arr.shape) == list(want.shape)
        assert torch.equal(arr.view(torch.int32), want.view(torch.int32))


# ---- size-independent properties at the full workload sizes -------------------------

def test_full_size_properties_config3_shape():
    """int4 1x128 over [11008, 4096]: the s/2 round-trip bound, clamp-freeness, idempotence of
    re-quantizing the dequantized weight, and linearity of the forward in x."""
    gen = torch.Generator(device=DEV).manual_seed(2)
    w = torch.randn(11008, 4096, device=DEV, generator=gen) * 0.02
    m = qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128))
    d = m.dequantize()
    s = m.scales().repeat_interleave(128, dim=1)
    assert bool(((d - w).abs() <= s * (0.5 + 1e-4)).all())
    words = m.codes()
    nib = torch.stack([(words >> (4 * j)) & 0xF for j in range(8)], dim=-1)
    assert int((nib == 8).sum()) == 0  # code -8 is never produced
    m2 = qb.QuantizedMatrix.quantize(d, qb.QuantDtype.Int4, qb.Group(1, 128))
    assert torch.equal(m2.codes(), m.codes())  # codes are a fixed point (the scale may move one ulp)
    assert bool(((m2.dequantize() - d).abs() <= d.abs() * 2.0 ** -22).all())
    ql = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
    x1 = torch.randn(4, 4096, device=DEV, generator=gen)
    x2 = torch.randn(4, 4096, device=DEV, generator=gen)
    y12 = ql.forward(x1 + x2)
    ysum = ql.forward(x1) + ql.forward(x2)
    assert bool(((y12 - ysum).abs() <= 1e-4 * (1 + ysum.abs())).all())
    ref = x1 @ d.t()
    y1 = ql.forward(x1)
    assert bool(((y1 - ref).abs() <= 1e-3 * (1 + ref.abs())).all())


# ---- the decode GEMV on the tensor pipe ---------------------------------------

@pytest.mark.parametrize("N,K", [(4096, 4096), (1000, 1024), (37, 128), (4096, 11008), (11008, 4096), (16, 256), (300, 2560)])
def test_decode_gemv_shapes(N, K):
    rng = np.random.default_rng(N * 7 + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    m, oc, os_ = quantize_both(w, N, K, qb.QuantDtype.Int4, qb.Group(1, 128))
    wd = o.dequantize_host(oc, os_, N, K, 4, 1, 128)
    ql = qb.QuantizedLinear.new(m, t(bias), qb.OUT_IN)
    for M in (1, 2, 5, 8, 9, 16):
        xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
        y = ql.forward(xt, out_dtype=torch.float32)
        # the tensor-pipe GEMV keeps the activations of at most 4096 inputs in registers; wider inputs run as column
        # slices of the weight (one grouped launch over the slices and a fold)
        assert ql.last_kernel() == ("gemv_mma" if K <= 4096 else "gemv_mma_sliced")
        want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.OUT_IN, threads=8)
        close(y.cpu().numpy(), want, 1e-4)   # exact codes, f32 accumulate: far inside the stated 1e-3
        yb = ql.forward(xt)                  # bf16 out
        close(yb.to(torch.float32).cpu().numpy(), want, 1e-2)
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


def test_decode_gemv_under_graph_replay_matches_eager():
    rng = np.random.default_rng(77)
    qls, outs = [], []
    for i in range(4):
        w = torch.randn(1024, 2048, device=DEV) * 0.02
        qls.append(qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128)), None, qb.OUT_IN))
    x = torch.randn(4, 2048, device=DEV).to(torch.bfloat16)
    eager = [ql.forward(x, out_dtype=torch.float32) for ql in qls]
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        outs = [torch.empty(4, 1024, device=DEV) for _ in qls]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            cap = [ql.forward(x, out_dtype=torch.float32) for ql in qls]
        for _ in range(3):
            g.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, cap):
        assert torch.equal(a, b)


def test_forward_many_matches_per_layer_forward():
    rng = np.random.default_rng(5)
    shapes = [(1024, 1024), (3000, 1024), (37, 1024), (4096, 1024)]
    qls = []
    for N, K in shapes:
        w = torch.from_numpy((rng.standard_normal((N, K)) * 0.02).astype(np.float32)).to(DEV)
        b = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(DEV)
        qls.append(qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128)), b, qb.OUT_IN))
    for M in (1, 3, 8, 16):
        x_shared = torch.randn(M, 1024, device=DEV).to(torch.bfloat16)
        x_other = torch.randn(M, 1024, device=DEV).to(torch.bfloat16)
        xs = [x_shared, x_shared, x_other, x_shared]
        want = [ql.forward(x, out_dtype=torch.float32) for ql, x in zip(qls, xs)]
        got = qb.QuantizedLinear.forward_many(qls, xs, out_dtype=torch.float32)
        assert qls[0].last_kernel() == "gemv_mma_grouped"
        for a, b_ in zip(got, want):
            assert torch.equal(a, b_)
    # a mix the grouped kernel cannot take falls back to the per-layer loop
    w8 = torch.randn(64, 1024, device=DEV) * 0.02
    q8 = qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w8, qb.QuantDtype.Int8, qb.PerChannel(0)), None, qb.OUT_IN)
    x = torch.randn(2, 1024, device=DEV).to(torch.bfloat16)
    got = qb.QuantizedLinear.forward_many([qls[0], q8], [x, x], out_dtype=torch.float32)
    # (an int4 and an int8 layer cannot share a launch; each takes its own decode kernel through the per-layer loop)
    assert torch.equal(got[1], q8.forward(x, out_dtype=torch.float32)) and q8.last_kernel() == "gemv_mma_i8"
    assert torch.equal(got[0], qls[0].forward(x, out_dtype=torch.float32)) and qls[0].last_kernel() == "gemv_mma"


# ---- the prefill GEMM on tcgen05 -------------------------------------------------

@pytest.mark.parametrize("M,N,K", [(17, 256, 512), (40, 384, 1024), (128, 128, 128), (128, 256, 256), (256, 384, 1024), (200, 300, 512), (64, 130, 2048), (333, 128, 4096)])
def test_prefill_gemm_against_oracle(M, N, K):
    """Stated staging: codes enter the tensor core as exact integers, activations as exact bf16, f32
    accumulation per 128-k group, the f32 scale applied to the group sum.  Checker: f64 accumulation of
    bf16(x) * (s * q) — no rounding of the weights — at the 1e-3 bound."""
    rng = np.random.default_rng(M * 31 + N * 7 + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    m, oc, os_ = quantize_both(w, N, K, qb.QuantDtype.Int4, qb.Group(1, 128))
    wd = o.dequantize_host(oc, os_, N, K, 4, 1, 128)
    xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
    want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.OUT_IN, threads=8)
    ql = qb.QuantizedLinear.new(m, t(bias), qb.OUT_IN)
    y = ql.forward(xt, out_dtype=torch.float32)
    assert ql.last_kernel() == "gemm_tcgen05"
    close(y.cpu().numpy(), want, 1e-3)
    yb = ql.forward(xt)
    assert yb.dtype == torch.bfloat16
    close(yb.to(torch.float32).cpu().numpy(), want, 1e-2)
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


@pytest.mark.parametrize("M,N,K,gran,layout", [
    (17, 256, 512, qb.Group(1, 64), qb.OUT_IN), (256, 1000, 1024, qb.Group(1, 32), qb.OUT_IN), (64, 130, 2048, qb.Group(1, 256), qb.OUT_IN),
    (128, 384, 1024, qb.PerChannel(0), qb.OUT_IN), (40, 256, 256, qb.PerTensor(), qb.OUT_IN), (200, 300, 512, qb.Block(5, 16), qb.OUT_IN),
    (96, 257, 384, qb.Group(1, 48), qb.OUT_IN), (300, 264, 1024, qb.Group(0, 64), qb.IN_OUT), (33, 520, 512, qb.Group(0, 256), qb.IN_OUT)])
def test_int4_prefill_gemm_other_grids(M, N, K, gran, layout):
    """int4 grids other than 1x128 whose tile width (along the inputs) is a whole number of 16-k MMA steps: the same tcgen05
    kernel with an accumulator per scale group of that width; `[in, out]` weights through the transposed copy.  f64 checker
    at 1e-3, one-hot activations bit for bit."""
    rng = np.random.default_rng(M * 31 + N * 7 + K)
    r, c = (N, K) if layout == qb.OUT_IN else (K, N)
    w = (rng.standard_normal((r, c)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    gr, gc = gran.tile(r, c)
    m, oc, os_ = quantize_both(w, r, c, qb.QuantDtype.Int4, gran)
    wd = o.dequantize_host(oc, os_, r, c, 4, gr, gc)
    xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
    want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, layout, threads=8)
    ql = qb.QuantizedLinear.new(m, t(bias), layout)
    y = ql.forward(xt, out_dtype=torch.float32)
    assert ql.last_kernel() == "gemm_tcgen05"
    close(y.cpu().numpy(), want, 1e-3)
    close(ql.forward(xt).to(torch.float32).cpu().numpy(), want, 1e-2)
    ks = sorted(set(int(k) for k in rng.integers(0, K, 40)) | {0, 15, 16, 31, 32, 63, K - 1})[:48]
    plain = qb.QuantizedLinear.new(m, None, layout)
    y1 = plain.forward(_one_hot_rows(ks, K), out_dtype=torch.float32)
    assert plain.last_kernel() == "gemm_tcgen05"
    ref = wd[:, ks].T.copy() if layout == qb.OUT_IN else wd[ks, :].copy()
    assert (bits(y1.cpu().numpy()) == bits(ref)).all()
    # a decode batch: grids whose scale is constant over whole 128-column runs are served as 1 x 128 (the decode kernel),
    # the others keep the generic kernel
    vgc = gc if layout == qb.OUT_IN else gr      # tile width along the inputs
    y4 = plain.forward(xt[:4], out_dtype=torch.float32)
    if vgc % 128 == 0 or vgc >= K:
        assert plain.last_kernel() == "gemv_mma", gran
    else:
        assert plain.last_kernel().startswith("generic"), gran
    close(y4.cpu().numpy(), want[:4] - bias[None, :], 1e-4)
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


def test_prefill_gemm_config3_full_size_properties():
    """int4 prefill at the full workload size (X [2048, 4096], W [11008, 4096]): against an f32 matmul over the
    bit-exact dequantized weight, and linearity in x."""
    gen = torch.Generator(device=DEV).manual_seed(2)
    w = torch.randn(11008, 4096, device=DEV, generator=gen) * 0.02
    x = torch.randn(2048, 4096, device=DEV, generator=gen).to(torch.bfloat16)
    m = qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128))
    ql = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
    y = ql.forward(x, out_dtype=torch.float32)
    assert ql.last_kernel() == "gemm_tcgen05"
    ref = x.to(torch.float32) @ m.dequantize().t()
    assert bool(((y - ref).abs() <= 1e-3 * (1 + ref.abs())).all())
    y2 = ql.forward((x.to(torch.float32) * 2).to(torch.bfloat16), out_dtype=torch.float32)  # exact doubling in bf16
    assert bool(((y2 - 2 * y).abs() <= 1e-5 * (1 + y.abs())).all())
    yb = ql.forward(x)
    assert bool(((yb.to(torch.float32) - ref).abs() <= 1e-2 * (1 + ref.abs())).all())


def test_forward_many_host_pinned_and_pageable_outputs():
    """qb200_qlinear_forward_many_host with outputs in pinned (device-mapped) memory, which the decode kernels write
    directly, and in pageable memory, which goes through the staging buffer: both equal the device-side call."""
    from quanta_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(11)
    qls = []
    for N in (512, 96, 1024):
        w = torch.from_numpy((rng.standard_normal((N, 1024)) * 0.02).astype(np.float32)).to(DEV)
        b = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(DEV)
        qls.append(qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int4, qb.Group(1, 128)), b, qb.OUT_IN))
    for M in (1, 5):
        x = torch.randn(M, 1024).to(torch.bfloat16)
        want = qb.QuantizedLinear.forward_many(qls, [x.to(DEV)] * 3, out_dtype=torch.float32)
        n = len(qls)
        hs = (_lib.vp * n)(*[q._h for q in qls])
        xp = (_lib.vp * n)(*[x.data_ptr()] * n)
        for pinned in (True, False):
            ys = [torch.full((M, q.out_dim()), float("nan")) for q in qls]
            if pinned:
                ys = [y.pin_memory() for y in ys]
            yp = (_lib.vp * n)(*[y.data_ptr() for y in ys])
            assert lib.qb200_qlinear_forward_many_host(hs, n, xp, _lib.BF16, M, yp, _lib.F32) == 0, _lib.last_error()
            for got, w_ in zip(ys, want):
                assert torch.equal(got, w_.cpu()), f"pinned={pinned} M={M}"
            one = torch.full((M, qls[0].out_dim()), float("nan"))
            one = one.pin_memory() if pinned else one
            assert lib.qb200_qlinear_forward_host(qls[0]._h, x.data_ptr(), _lib.BF16, M, one.data_ptr(), _lib.F32) == 0, _lib.last_error()
            assert torch.equal(one, qls[0].forward(x.to(DEV), out_dtype=torch.float32).cpu())


@pytest.mark.parametrize("shape,dtype,gran", [
    ((64, 256), qb.QuantDtype.Int4, qb.Group(1, 128)), ((96, 512), qb.QuantDtype.Int8, qb.Block(32, 32)),
    ((33, 768), qb.QuantDtype.Int4, qb.Group(1, 96)), ((33, 768), qb.QuantDtype.Int8, qb.Group(1, 96)),
    ((40, 1024), qb.QuantDtype.Int4, qb.PerTensor()), ((7, 256), qb.QuantDtype.Int8, qb.PerChannel(0)),
    ((300, 2048), qb.QuantDtype.Int4, qb.Block(32, 32)),
])
def test_dequantize_row_segment_path_is_bit_exact(shape, dtype, gran):
    # cols % 256 == 0: the kernel whose warps take 256 elements of a row per step; power-of-two and other tile widths
    r, c = shape
    w = np.random.default_rng(r + c).standard_normal(shape).astype(np.float32)
    m, oc, os_ = quantize_both(w, r, c, dtype, gran)
    gr, gc = gran.tile(r, c)
    want = o.dequantize_host(oc, os_, r, c, dtype.bits(), gr, gc)
    got = m.dequantize().cpu().numpy()
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("shape,dtype,gran", [
    ((64, 4096), qb.QuantDtype.Int8, qb.PerChannel(0)), ((64, 4096), qb.QuantDtype.Int4, qb.PerChannel(0)),
    ((300, 512), qb.QuantDtype.Int8, qb.PerTensor()), ((300, 512), qb.QuantDtype.Int4, qb.PerTensor()),
    ((130, 192), qb.QuantDtype.Int4, qb.Block(64, 64)), ((9, 2056), qb.QuantDtype.Int8, qb.Group(1, 2056)),
])
def test_quantize_large_tiles_chunk_path_is_bit_exact(shape, dtype, gran):
    # tiles of more than 2048 elements (whole rows, the whole matrix, big blocks): the two-pass chunk kernels
    r, c = shape
    w = (np.random.default_rng(r * c).standard_normal(shape) * 0.05).astype(np.float32)
    w[1, 8] = np.nan
    w[2, 16] = -3.75  # the tile's (or a tile's) maximum
    m, oc, os_ = quantize_both(w, r, c, dtype, gran)
    assert_quant_equal(m, oc, os_)
    # bf16 source through the same path
    wb = o.f32_to_bf16(w)
    mb = qb.QuantizedMatrix.quantize(torch.from_numpy(wb.view(np.int16)).view(torch.bfloat16).to(DEV), dtype, gran)
    gr, gc = gran.tile(r, c)
    oc2, os2 = o.quantize_host(o.bf16_to_f32(wb), r, c, dtype.bits(), gr, gc)
    assert_quant_equal(mb, oc2, os2)


# ---- bit-for-bit at the full sizes of the quantize-on-load and prefill workloads ------------------

@pytest.mark.parametrize("shape,dtype,gran", [
    ((11008, 4096), qb.QuantDtype.Int4, qb.Group(1, 128)),
    ((11008, 4096), qb.QuantDtype.Int8, qb.Block(32, 32)),
    ((4096, 4096), qb.QuantDtype.Int8, qb.Block(32, 32)),
    ((4096, 4096), qb.QuantDtype.Int4, qb.Group(1, 128)),
])
def test_full_size_codes_scales_and_dequantize_bit_exact(shape, dtype, gran):
    """The checkpoint's two matrix shapes, both grids: every code, every scale and every dequantized weight against
    the oracle (45 M elements take the CPU restatement about a second)."""
    r, c = shape
    g = np.random.default_rng(3 + r)
    w = g.standard_normal((r, c), dtype=np.float32) * np.float32(0.02)
    m, oc, os_ = quantize_both(w, r, c, dtype, gran)
    assert_quant_equal(m, oc, os_, f"{shape} {dtype.name}")
    gr, gc = gran.tile(r, c)
    host = o.dequantize_host(oc, os_, r, c, dtype.bits(), gr, gc)
    assert (bits(m.dequantize().cpu().numpy()) == bits(host)).all()


# ---- the reference's own orientation, `[in, out]` with groups along the inputs, on the fast kernels ---------

def _one_hot_rows(ks, K):
    x = np.zeros((len(ks), K), np.float32)
    for i, k in enumerate(ks):
        x[i, k] = 1.0
    return torch.from_numpy(o.f32_to_bf16(x).view(np.int16)).view(torch.bfloat16).to(DEV)


@pytest.mark.parametrize("K,N", [(1024, 520), (4096, 264), (256, 136), (11008, 72)])
def test_in_out_int4_takes_the_fast_kernels_and_its_execution_copy_is_a_permutation(K, N):
    """QuantizedLinear::new(w: [in, out]) with Group{axis: 0, size: 128} (crates/ml/quanta-nn/src/quant.rs:853-862):
    the handle transposes codes and scales once.  One-hot activations read single weights back through the decode
    kernel: 1.0 * (s * q) with every other product zero is exact, so the outputs must equal the oracle's dequantized
    weights of the ORIGINAL record bit for bit."""
    rng = np.random.default_rng(K + N)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    m, oc, os_ = quantize_both(w, K, N, qb.QuantDtype.Int4, qb.Group(0, 128))
    wd = o.dequantize_host(oc, os_, K, N, 4, 128, 1)   # [in, out]
    ql = qb.QuantizedLinear.new(m, None, qb.IN_OUT)
    ks = sorted(set([0, 1, 2, 3, 4, 5, 6, 7, 127, 128 % K, K // 2 + 3, K - 8, K - 1] + list(rng.integers(0, K, 3))))
    ks = [int(k) for k in ks][:16]
    y = ql.forward(_one_hot_rows(ks, K), out_dtype=torch.float32)
    assert ql.last_kernel() == ("gemv_mma" if K <= 4096 else "gemv_mma_sliced")
    assert (bits(y.cpu().numpy()) == bits(wd[ks])).all()
    # dense activations, decode and prefill batch sizes, against the f64 checker over the dequantized record
    bias = rng.standard_normal(N).astype(np.float32)
    qlb = qb.QuantizedLinear.new(m, t(bias), qb.IN_OUT)
    for M, kernel, tol in [(3, "gemv_mma" if K <= 4096 else "gemv_mma_sliced", 1e-4), (16, None, 1e-4), (40, "gemm_tcgen05", 1e-3)]:
        xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
        got = qlb.forward(xt, out_dtype=torch.float32).cpu().numpy()
        if kernel:
            assert qlb.last_kernel() == kernel
        close(got, o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.IN_OUT, threads=8), tol)
    # f32 activations (the reference's own dtype) ride the same kernels as three exact bf16 parts
    mf = max(1, -(-2 ** 24 // (K * N)))   # enough rows for the three-part path (at least 2^24 multiply-adds)
    xf = rng.standard_normal((mf, K)).astype(np.float32)
    got = qlb.forward(t(xf), out_dtype=torch.float32).cpu().numpy()
    assert qlb.last_kernel() == (("gemv_mma" if K <= 4096 else "gemv_mma_sliced") if 3 * mf <= 16 else "gemm_tcgen05")
    close(got, o.linear_forward_f64(xf, wd, bias, o.IN_OUT, threads=8), 1e-5)
    # the record itself is untouched: it still dequantizes to the oracle's matrix
    assert (bits(m.dequantize().cpu().numpy()) == bits(wd)).all()
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(qlb._h, None) == 0


@pytest.mark.parametrize("K,N,gran", [(1024, 520, qb.Block(32, 32)), (512, 264, qb.Group(0, 128)), (256, 136, qb.PerChannel(1)),
                                      (2048, 300, qb.Block(16, 8)), (192, 72, qb.Group(0, 48)), (320, 100, qb.PerTensor())])
def test_in_out_int8_takes_the_fast_kernels_through_its_transposed_copy(K, N, gran):
    """An `[in, out]` int8 weight whose tile height is a whole number of 16-row steps: the handle transposes codes and
    scale grid once and the int8 decode and prefill kernels serve it.  One-hot activations read single weights back
    bit for bit against the oracle's dequantize of the ORIGINAL record; random activations against the f64 checker."""
    rng = np.random.default_rng(K + N)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    gr, gc = gran.tile(K, N)
    m, oc, os_ = quantize_both(w, K, N, qb.QuantDtype.Int8, gran)
    wd = o.dequantize_host(oc, os_, K, N, 8, gr, gc)   # [in, out]
    plain = qb.QuantizedLinear.new(m, None, qb.IN_OUT)
    ql = qb.QuantizedLinear.new(m, t(bias), qb.IN_OUT)
    decode = gr % 32 == 0 and K % 128 == 0 and K <= 4096
    prefill = K % 64 == 0 and (gr >= K or K % gr == 0)
    ks = sorted(set(int(k) for k in rng.integers(0, K, 40)) | {0, 15, 16, 31, 32, 63, K - 1})
    for rows, kernel in [(ks[:8], "gemv_mma_i8" if decode else "gemm_tcgen05_i8" if prefill else "generic_cols"),
                         (ks[:40], "gemm_tcgen05_i8" if prefill else "generic_cols")]:
        y = plain.forward(_one_hot_rows(rows, K), out_dtype=torch.float32)
        assert plain.last_kernel() == kernel, (gran, len(rows))
        assert (bits(y.cpu().numpy()) == bits(wd[rows, :].copy())).all()
    for M in (3, 8, 12, 50):
        xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
        want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.IN_OUT, threads=8)
        close(ql.forward(xt, out_dtype=torch.float32).cpu().numpy(), want, 1e-3)
        assert not ql.last_kernel().startswith("generic") or not (decode or (prefill and M > 4))
    assert (bits(m.dequantize().cpu().numpy()) == bits(wd)).all()   # the record itself is untouched
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


@pytest.mark.parametrize("N,K,gran,layout", [
    (1000, 1024, qb.PerChannel(0), qb.OUT_IN), (264, 2048, qb.PerTensor(), qb.OUT_IN), (130, 1024, qb.Group(1, 256), qb.OUT_IN),
    (300, 512, qb.Block(4, 128), qb.OUT_IN), (520, 1024, qb.PerChannel(1), qb.IN_OUT), (136, 512, qb.PerTensor(), qb.IN_OUT),
    (72, 11008, qb.PerChannel(0), qb.OUT_IN), (264, 1024, qb.Group(0, 512), qb.IN_OUT)])
def test_int4_grids_constant_over_128_column_runs_take_the_1x128_kernels(N, K, gran, layout):
    """Per-row, per-tensor and wide-tile int4 grids: the handle spells the scales out per 128-column run (the same scale
    on the same codes), after which the decode kernel, its sliced form and the prefill kernel of the 1 x 128 grid serve the
    layer.  One-hot activations read single weights back bit for bit against the oracle's dequantize of the stored record."""
    rng = np.random.default_rng(N + K)
    r, c = (N, K) if layout == qb.OUT_IN else (K, N)
    w = (rng.standard_normal((r, c)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    gr, gc = gran.tile(r, c)
    m, oc, os_ = quantize_both(w, r, c, qb.QuantDtype.Int4, gran)
    wd = o.dequantize_host(oc, os_, r, c, 4, gr, gc)
    ql = qb.QuantizedLinear.new(m, t(bias), layout)
    plain = qb.QuantizedLinear.new(m, None, layout)
    decode = "gemv_mma" if K <= 4096 else "gemv_mma_sliced"
    ks = sorted(set(int(k) for k in rng.integers(0, K, 40)) | {0, 127, 128, K - 1})
    for rows, kernel in [(ks[:8], decode), (ks[:40], "gemm_tcgen05")]:
        y = plain.forward(_one_hot_rows(rows, K), out_dtype=torch.float32)
        assert plain.last_kernel() == kernel, (gran, len(rows))
        ref = wd[:, rows].T.copy() if layout == qb.OUT_IN else wd[rows, :].copy()
        assert (bits(y.cpu().numpy()) == bits(ref)).all()
    for M, kernel, tol in [(1, decode, 1e-4), (16, decode, 1e-4), (50, "gemm_tcgen05", 1e-3)]:
        xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
        y = ql.forward(xt, out_dtype=torch.float32)
        assert ql.last_kernel() == kernel, (gran, M)
        close(y.cpu().numpy(), o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, layout, threads=8), tol)
    assert (bits(m.dequantize().cpu().numpy()) == bits(wd)).all()   # the record itself is untouched
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


def test_sliced_decode_of_a_wide_layer_matches_per_slice_sums():
    """A `[4096, 11008]` layer at M <= 16 (a feed-forward down projection called on its own): three column slices in one
    launch plus the fold; with bf16 output; through the host-buffer entry point with pinned outputs."""
    rng = np.random.default_rng(12)
    N, K = 512, 11008
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    m, oc, os_ = quantize_both(w, N, K, qb.QuantDtype.Int4, qb.Group(1, 128))
    wd = o.dequantize_host(oc, os_, N, K, 4, 1, 128)
    ql = qb.QuantizedLinear.new(m, t(bias), qb.OUT_IN)
    ks = [0, 3711, 3712, 7423, 7424, 11007, 5000, 1]    # first and last column of every slice
    y = ql.forward(_one_hot_rows(ks, K), out_dtype=torch.float32)
    assert ql.last_kernel() == "gemv_mma_sliced"
    want = wd[:, ks].T + bias[None, :]
    assert (bits(y.cpu().numpy()) == bits(want.astype(np.float32))).all()
    for M in (1, 7, 16):
        xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
        want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.OUT_IN, threads=8)
        yd = ql.forward(xt, out_dtype=torch.float32).cpu().numpy()
        close(yd, want, 1e-4)
        close(ql.forward(xt).to(torch.float32).cpu().numpy(), want, 1e-2)
        assert (bits(ql.forward_host(xb)) == bits(yd)).all()   # host buffers in and out: the same kernels
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


@pytest.mark.parametrize("gran,layout", [(qb.Block(32, 32), qb.OUT_IN), (qb.Group(1, 128), qb.OUT_IN), (qb.Block(32, 32), qb.IN_OUT)])
def test_int8_sliced_decode_of_a_wide_layer(gran, layout):
    """An int8 layer with 11008 inputs at M <= 16: three column slices in one launch (two launches for 9..16 rows) plus
    the fold; one-hot activations at the slices' edges bit for bit; f32 activations as three parts."""
    rng = np.random.default_rng(13)
    N, K = 392, 11008
    r, c = (N, K) if layout == qb.OUT_IN else (K, N)
    w = (rng.standard_normal((r, c)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    gr, gc = gran.tile(r, c)
    m, oc, os_ = quantize_both(w, r, c, qb.QuantDtype.Int8, gran)
    wd = o.dequantize_host(oc, os_, r, c, 8, gr, gc)
    ql = qb.QuantizedLinear.new(m, t(bias), layout)
    ks = [0, 3711, 3712, 7423, 7424, 11007, 5000, 1]    # first and last column of every slice
    y = ql.forward(_one_hot_rows(ks, K), out_dtype=torch.float32)
    assert ql.last_kernel() == "gemv_mma_i8_sliced"
    want = (wd[:, ks].T if layout == qb.OUT_IN else wd[ks, :]) + bias[None, :]
    assert (bits(y.cpu().numpy()) == bits(want.astype(np.float32))).all()
    for M in (1, 7, 8, 12, 16):
        xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
        want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, layout, threads=8)
        yd = ql.forward(xt, out_dtype=torch.float32).cpu().numpy()
        assert ql.last_kernel() == "gemv_mma_i8_sliced"
        close(yd, want, 1e-4)
        close(ql.forward(xt).to(torch.float32).cpu().numpy(), want, 1e-2)
    xf = rng.standard_normal((4, K)).astype(np.float32)
    yf = ql.forward(t(xf), out_dtype=torch.float32).cpu().numpy()
    assert ql.last_kernel() == "gemv_mma_i8_sliced"
    close(yf, o.linear_forward_f64(xf, wd, bias, layout, threads=8), 1e-5)
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


def test_decode_domain_limit_is_checked():
    """The decode kernel scales activations by 2^40 inside bf16: |x| < 2^87 is its domain.  Just inside, the result
    matches the oracle; at 2^87 and for non-finite activations the call is flagged and qb200_qlinear_check reports
    it (the reference's f32 path would return a finite number for a finite x: the difference is loud, not silent)."""
    from quanta_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(8)
    N, K = 256, 512
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    m, oc, os_ = quantize_both(w, N, K, qb.QuantDtype.Int4, qb.Group(1, 128))
    wd = o.dequantize_host(oc, os_, N, K, 4, 1, 128)
    ql = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
    x = rng.standard_normal((2, K)).astype(np.float32)
    x[0, 5] = 2.0 ** 86
    x[1, 300] = -(2.0 ** 86) * 1.5
    xb = o.f32_to_bf16(x)
    xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
    y = ql.forward(xt, out_dtype=torch.float32).cpu().numpy()
    assert ql.last_kernel() == "gemv_mma" and lib.qb200_qlinear_check(ql._h, None) == 0
    want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, None, o.OUT_IN, threads=2)
    assert np.isfinite(y).all()
    close(y / 2.0 ** 80, want / 2.0 ** 80, 1e-4)
    for bad in (2.0 ** 87, np.inf, np.nan):
        x2 = x.copy()
        x2[1, 17] = bad
        xb2 = o.f32_to_bf16(x2)
        ql.forward(torch.from_numpy(xb2.view(np.int16)).view(torch.bfloat16).to(DEV), out_dtype=torch.float32)
        assert lib.qb200_qlinear_check(ql._h, None) == _lib.ERR_INVALID_PARAM
        assert "2^87" in _lib.last_error()
        assert lib.qb200_qlinear_check(ql._h, None) == 0   # reported once


def test_host_entry_with_unaligned_scales_keeps_the_staging_path():
    """Scales that are not 16-byte aligned take the layer off the decode kernel (the tcgen05 GEMM serves it); the
    host-buffer entry point must then not hand pinned host memory to that kernel's TMA stores but stage the outputs
    on the device, and still return the right numbers."""
    from quanta_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(31)
    N, K, M = 384, 1024, 4
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    m, oc, os_ = quantize_both(w, N, K, qb.QuantDtype.Int4, qb.Group(1, 128))
    wd = o.dequantize_host(oc, os_, N, K, 4, 1, 128)
    base = torch.zeros(N * (K // 128) + 4, device=DEV)
    shifted = base[1: 1 + N * (K // 128)].view(N, K // 128)
    shifted.copy_(m.scales())
    assert shifted.data_ptr() % 16 == 4
    odd = qb.QuantizedMatrix.from_parts(m.codes(), [N, K], shifted, qb.Group(1, 128))
    ql = qb.QuantizedLinear.new(odd, None, qb.OUT_IN)
    xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, None, o.OUT_IN, threads=4)
    xh = torch.from_numpy(xb.view(np.int16).copy()).view(torch.bfloat16).pin_memory()
    yh = torch.full((M, N), float("nan")).pin_memory()
    hs, xp, yp = (_lib.vp * 1)(ql._h), (_lib.vp * 1)(xh.data_ptr()), (_lib.vp * 1)(yh.data_ptr())
    assert lib.qb200_qlinear_forward_many_host(hs, 1, xp, _lib.BF16, M, yp, _lib.F32) == 0, _lib.last_error()
    assert ql.last_kernel() == "gemm_tcgen05"
    close(yh.numpy(), want, 1e-3)
    y2 = np.full((M, N), np.nan, np.float32)
    assert (bits(ql.forward_host(xb, y2)) == bits(yh.numpy())).all()


# ---- the int8 decode GEMV on the tensor pipe (any grid whose tile width is a multiple of 32) ------------------

I8_GRIDS = [qb.Block(32, 32), qb.Group(1, 128), qb.PerChannel(0), qb.PerTensor(), qb.Group(1, 32), qb.Block(16, 64), qb.Block(5, 96)]


@pytest.mark.parametrize("N,K", [(4096, 4096), (1000, 1024), (37, 128), (300, 2560), (16, 256)])
def test_int8_decode_gemv_shapes(N, K):
    rng = np.random.default_rng(N * 3 + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    from quanta_b200 import _lib
    for gran in I8_GRIDS[: (7 if N <= 1000 else 3)]:
        try:
            gr, gc = gran.tile(N, K)
        except qb.QuantError:   # a block larger than this matrix is not a valid spelling
            continue
        m, oc, os_ = quantize_both(w, N, K, qb.QuantDtype.Int8, gran)
        wd = o.dequantize_host(oc, os_, N, K, 8, gr, gc)
        ql = qb.QuantizedLinear.new(m, t(bias), qb.OUT_IN)
        for M in (1, 2, 5, 8):
            xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
            xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
            y = ql.forward(xt, out_dtype=torch.float32)
            assert ql.last_kernel() == "gemv_mma_i8", (gran, M)
            want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.OUT_IN, threads=8)
            close(y.cpu().numpy(), want, 1e-4)
            close(ql.forward(xt).to(torch.float32).cpu().numpy(), want, 1e-2)
        # one-hot activations read single weights back: 1.0 * (s * q) is exact, every other product is zero
        ks = sorted({0, 1, 2, 3, 31, 32 % K, 127, K // 2 + 5, K - 1})[:8]
        y = qb.QuantizedLinear.new(m, None, qb.OUT_IN).forward(_one_hot_rows(ks, K), out_dtype=torch.float32)
        assert (bits(y.cpu().numpy()) == bits(wd[:, ks].T.copy())).all(), gran
        for M in (9, 16):   # batches of 9..16: two launches of eight rows at most
            xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
            xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
            y = ql.forward(xt, out_dtype=torch.float32)
            assert ql.last_kernel() == "gemv_mma_i8_x2"
            close(y.cpu().numpy(), o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.OUT_IN, threads=8), 1e-4)
        ql.forward(torch.randn(17, K, device=DEV).to(torch.bfloat16), out_dtype=torch.float32)   # a prefill batch
        tensor_core = K % 64 == 0 and (gc >= K or (gc % 16 == 0 and K % gc == 0))
        assert ql.last_kernel() == ("gemm_tcgen05_i8" if tensor_core else "generic_rows"), (gran, K)
        assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


# ---- the int8 prefill GEMM on tcgen05 (tile widths that are whole 16-k MMA steps) ------------------------------

@pytest.mark.parametrize("M,N,K,gran", [
    (17, 256, 512, qb.Block(32, 32)), (256, 1024, 1024, qb.Block(32, 32)), (300, 1000, 1024, qb.Block(32, 32)),
    (64, 130, 2048, qb.Group(1, 128)), (128, 384, 1024, qb.PerChannel(0)), (40, 256, 256, qb.PerTensor()),
    (200, 300, 512, qb.Block(5, 16)), (96, 257, 192, qb.Group(1, 48)), (333, 128, 4096, qb.Block(16, 64)),
    (513, 515, 576, qb.Group(1, 192)), (32, 64, 64, qb.Block(32, 32))])
def test_int8_prefill_gemm_against_oracle(M, N, K, gran):
    """Codes enter the tensor core as the exact bf16 values q / 64, activations as exact bf16, f32 accumulation per scale
    group, the f32 scale applied to the group sum.  Checker: f64 accumulation of bf16(x) * (s * q) at the 1e-3 bound;
    one-hot activations read single weights back bit for bit (1.0 * q / 64 * 64 s rounds once, like s * q)."""
    rng = np.random.default_rng(M * 31 + N * 7 + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    gr, gc = gran.tile(N, K)
    m, oc, os_ = quantize_both(w, N, K, qb.QuantDtype.Int8, gran)
    wd = o.dequantize_host(oc, os_, N, K, 8, gr, gc)
    xb = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    xt = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV)
    want = o.linear_forward_f64(o.bf16_to_f32(xb), wd, bias, o.OUT_IN, threads=8)
    ql = qb.QuantizedLinear.new(m, t(bias), qb.OUT_IN)
    y = ql.forward(xt, out_dtype=torch.float32)
    assert ql.last_kernel() == "gemm_tcgen05_i8"
    close(y.cpu().numpy(), want, 1e-3)
    yb = ql.forward(xt)
    assert yb.dtype == torch.bfloat16
    close(yb.to(torch.float32).cpu().numpy(), want, 1e-2)
    ks = sorted(set(int(k) for k in rng.integers(0, K, 40)) | {0, 15, 16, 31, 32, 63, K - 1})[:48]
    plain = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
    y1 = plain.forward(_one_hot_rows(ks, K), out_dtype=torch.float32)
    assert plain.last_kernel() == "gemm_tcgen05_i8"
    assert (bits(y1.cpu().numpy()) == bits(wd[:, ks].T.copy())).all()
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0
    assert _lib.load().qb200_qlinear_check(plain._h, None) == 0


def test_int8_prefill_full_size_properties():
    """int8 32x32 prefill at X [2048, 4096], W [11008, 4096]: against an f32 matmul over the bit-exact dequantized
    weight, and linearity in x; the split-K path ([4096, 4096] at 256 rows) against the same."""
    gen = torch.Generator(device=DEV).manual_seed(5)
    for N, M in [(11008, 2048), (4096, 256)]:
        w = torch.randn(N, 4096, device=DEV, generator=gen) * 0.02
        x = torch.randn(M, 4096, device=DEV, generator=gen).to(torch.bfloat16)
        m = qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int8, qb.Block(32, 32))
        ql = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
        y = ql.forward(x, out_dtype=torch.float32)
        assert ql.last_kernel() == "gemm_tcgen05_i8"
        ref = x.to(torch.float32) @ m.dequantize().t()
        assert bool(((y - ref).abs() <= 1e-3 * (1 + ref.abs())).all())
        y2 = ql.forward((x.to(torch.float32) * 2).to(torch.bfloat16), out_dtype=torch.float32)  # exact doubling in bf16
        assert bool(((y2 - 2 * y).abs() <= 1e-5 * (1 + y.abs())).all())
        yb = ql.forward(x)
        assert bool(((yb.to(torch.float32) - ref).abs() <= 1e-2 * (1 + ref.abs())).all())


def test_int8_forward_many_and_graph_replay():
    rng = np.random.default_rng(6)
    qls = []
    for N, gran in [(1024, qb.Block(32, 32)), (3000, qb.Group(1, 128)), (37, qb.PerChannel(0)), (2048, qb.Block(32, 32))]:
        w = torch.from_numpy((rng.standard_normal((N, 1024)) * 0.02).astype(np.float32)).to(DEV)
        b = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(DEV)
        qls.append(qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int8, gran), b, qb.OUT_IN))
    for M in (1, 4, 8):
        x = torch.randn(M, 1024, device=DEV).to(torch.bfloat16)
        x2 = torch.randn(M, 1024, device=DEV).to(torch.bfloat16)
        xs = [x, x, x2, x]
        want = [ql.forward(xi, out_dtype=torch.float32) for ql, xi in zip(qls, xs)]
        got = qb.QuantizedLinear.forward_many(qls, xs, out_dtype=torch.float32)
        assert qls[0].last_kernel() == "gemv_mma_i8_grouped"
        for a, b_ in zip(got, want):
            assert torch.equal(a, b_)   # the same arithmetic per output whatever the launch's item partition
    x = torch.randn(4, 1024, device=DEV).to(torch.bfloat16)
    eager = [ql.forward(x, out_dtype=torch.float32) for ql in qls]
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            cap = [ql.forward(x, out_dtype=torch.float32) for ql in qls]
        for _ in range(3):
            g.replay()
    torch.cuda.synchronize()
    for a, b_ in zip(eager, cap):
        assert torch.equal(a, b_)


def test_config1_int8_block32_bf16_activations_take_the_fast_kernel():
    g = np.random.default_rng(0)
    w = (g.standard_normal((1024, 1024), dtype=np.float32) * np.float32(0.02))
    x = g.standard_normal((8, 1024), dtype=np.float32)
    m, oc, os_ = quantize_both(w, 1024, 1024, qb.QuantDtype.Int8, qb.Block(32, 32))
    wd = o.dequantize_host(oc, os_, 1024, 1024, 8, 32, 32)
    ql = qb.QuantizedLinear.new(m, None, qb.OUT_IN)
    xb = o.f32_to_bf16(x)
    y = ql.forward(torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(DEV), out_dtype=torch.float32)
    assert ql.last_kernel() == "gemv_mma_i8"
    close(y.cpu().numpy(), o.linear_forward(o.bf16_to_f32(xb), wd, None, o.OUT_IN, threads=8), 1e-4)
    assert (bits(ql.forward_host(xb)) == bits(y.cpu().numpy())).all()


@pytest.mark.parametrize("dtype,gran,layout,shape", [
    (qb.QuantDtype.Int4, qb.Group(1, 128), qb.OUT_IN, (4096, 4096)), (qb.QuantDtype.Int4, qb.Group(0, 128), qb.IN_OUT, (4096, 1032)),
    (qb.QuantDtype.Int8, qb.Block(32, 32), qb.OUT_IN, (2048, 4096)), (qb.QuantDtype.Int8, qb.Block(32, 32), qb.IN_OUT, (4096, 1000)),
    (qb.QuantDtype.Int4, qb.Group(1, 128), qb.OUT_IN, (2048, 8192)), (qb.QuantDtype.Int4, qb.Group(1, 128), qb.OUT_IN, (1000, 1024))])
def test_f32_activations_ride_the_bf16_kernels_as_three_exact_parts(dtype, gran, layout, shape):
    """The reference's activations are f32 (Layer::<f32>::apply, crates/ml/quanta-nn/src/quant.rs:903-918).  An f32 is the
    exact sum of three bf16 values; the kernels multiply each part exactly and accumulate in f32, so the folded result
    is the exact-product sum: it meets the f64 checker at 1e-5, tighter than the bf16 tests' bound.  Small layers at small
    batches (fewer than 2^24 multiply-adds) keep the generic kernel's single launch, at its own 1e-4."""
    r, c = shape
    rng = np.random.default_rng(r + c)
    w = (rng.standard_normal((r, c)) * 0.02).astype(np.float32)
    in_dim, out_dim = (r, c) if layout == qb.IN_OUT else (c, r)
    bias = rng.standard_normal(out_dim).astype(np.float32)
    gr, gc = gran.tile(r, c)
    m, oc, os_ = quantize_both(w, r, c, dtype, gran)
    wd = o.dequantize_host(oc, os_, r, c, dtype.bits(), gr, gc)
    ql = qb.QuantizedLinear.new(m, t(bias), layout)
    for M in (1, 2, 5, 7, 40):
        x = (rng.standard_normal((M, in_dim)) * np.exp(rng.uniform(-6, 6, (M, 1)))).astype(np.float32)   # rows of very different size
        want = o.linear_forward_f64(x, wd, bias, layout, threads=8)
        y = ql.forward(t(x), out_dtype=torch.float32).cpu().numpy()
        split = M * in_dim * out_dim >= 2 ** 24
        assert ql.last_kernel().startswith("generic") != split, (ql.last_kernel(), M)
        err = np.abs(y - want) - (1e-5 if split else 1e-4) * (np.abs(x).max(axis=1, keepdims=True) + np.abs(want))
        assert (err <= 0).all(), (M, ql.last_kernel(), float(err.max()))
        yb = ql.forward(t(x), out_dtype=torch.bfloat16).to(torch.float32).cpu().numpy()
        assert (np.abs(yb - want) <= 1e-2 * (np.abs(x).max(axis=1, keepdims=True) + np.abs(want))).all()
        assert (bits(ql.forward_host(x)) == bits(y)).all()    # host buffers in and out: the same kernels
    from quanta_b200 import _lib
    assert _lib.load().qb200_qlinear_check(ql._h, None) == 0


def test_scratch_growth_is_refused_while_a_graph_is_recorded():
    """A forward whose scratch is not allocated yet would free / allocate; on a stream that records a CUDA graph that
    is refused with a message, the recording survives, and after one call outside a capture the same shape records."""
    w = torch.randn(4096, 256, device=DEV) * 0.02   # [in, out] int8, 8 x 8 tiles: the column kernel splits K and needs partial sums
    ql = qb.QuantizedLinear.new(qb.QuantizedMatrix.quantize(w, qb.QuantDtype.Int8, qb.Block(8, 8)), None, qb.IN_OUT)
    x = torch.randn(3, 4096, device=DEV)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    caught = None
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            try:
                ql.forward(x)
            except qb.QuantError as e:
                caught = e
    assert caught is not None and caught.kind == "InvalidParam" and "before the capture" in str(caught)
    want = ql.forward(x)     # allocates
    assert ql.last_kernel() == "generic_cols"
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=s):
            got = ql.forward(x)
        g2.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
