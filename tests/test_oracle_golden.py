"""Pins the CPU oracle against the reference's own literals (no GPU needed)."""
import struct

import numpy as np
import pytest

import oracle as o
from oracle import safetensors_oracle as so
from tests.golden import kats


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_quant_ranges():
    for b, want in kats.QUANT_RANGES.items():
        assert o.quant_range(b) == want


def test_int4_pack_unpack_all_nibbles():
    # dtype.rs:413-434: every value in every slot round-trips; other nibbles untouched
    for i in range(8):
        word = kats.PACK_SWEEP_WORD
        for v in range(-8, 8):
            w = o.int4_pack(word, i, v)
            assert o.int4_unpack(w, i) == v
            for j in range(8):
                if j != i:
                    assert o.int4_unpack(w, j) == o.int4_unpack(word, j)
            word = w


def test_quantize_dequantize_sym_literals():
    for x, s, b, code in kats.QUANTIZE_SYM:
        assert o.quantize_sym(x, s, b) == code, (x, s, b)
    for q, s, v in kats.DEQUANTIZE_SYM:
        assert o.dequantize_sym(q, s) == np.float32(v)


@pytest.mark.parametrize("bits_", [8, 4])
def test_op_matrix_cases(bits_):
    xs = kats.op_matrix_inputs(0.5)
    got = [o.quantize_sym(float(x), 0.5, bits_) for x in xs]
    assert got == kats.op_matrix_expected(bits_)
    lo, hi = kats.QUANT_RANGES[bits_]
    for code in range(lo, hi + 1):
        assert o.dequantize_sym(code, 0.5) == np.float32(0.5) * np.float32(code)


def test_rust_cast_semantics():
    # `as i32` saturates, NaN -> 0; s = inf gives code 0
    assert o.quantize_sym(float("nan"), 1.0, 8) == 0
    assert o.quantize_sym(float("inf"), 1.0, 8) == 127
    assert o.quantize_sym(-3e38, 1e-38, 8) == -128
    assert o.quantize_sym(5.0, float("inf"), 4) == 0
    assert o.quantize_sym(float("inf"), float("inf"), 4) == 0


def test_bf16_conversions():
    assert o.lib().qo_f32_to_bf16(np.float32(3.140625)) == 0x4049
    assert o.lib().qo_bf16_to_f32(0x4049) == 3.140625
    # ties to even on the dropped half: 1 + 2^-8 is a tie between 0x3F80 and 0x3F81
    assert o.lib().qo_f32_to_bf16(np.float32(1.0 + 2.0 ** -8)) == 0x3F80
    assert o.lib().qo_f32_to_bf16(np.float32(1.0 + 3 * 2.0 ** -8)) == 0x3F82
    nan = struct.unpack("<f", struct.pack("<I", 0x7F800001))[0]
    assert o.lib().qo_f32_to_bf16(np.float32(nan)) & 0x7FC0 == 0x7FC0
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    v = o.f32_to_bf16(x)
    assert all(int(v[i]) == o.lib().qo_f32_to_bf16(x[i]) for i in range(0, 4096, 37))
    for h, val in zip(kats.F16_CASE["halves"], kats.F16_CASE["values"]):
        assert abs(o.lib().qo_f16_to_f32(h) - val) < 1e-12


def test_tile_spellings_and_errors():
    assert o.tile(o.PER_TENSOR, 5, 7) == (5, 7)
    assert o.tile(o.PER_CHANNEL, 5, 7, axis=0) == (1, 7)
    assert o.tile(o.PER_CHANNEL, 5, 7, axis=1) == (5, 1)
    assert o.tile(o.GROUP, 5, 7, axis=0, size=3) == (3, 1)
    assert o.tile(o.GROUP, 5, 7, axis=1, size=3) == (1, 3)
    assert o.tile(o.BLOCK, 64, 64, size=32, size2=32) == (32, 32)
    # tests/quant.rs:368-394
    for kind, axis, size in [(o.PER_CHANNEL, 2, 0), (o.GROUP, 3, 2), (o.GROUP, 0, 0), (o.GROUP, 1, 99)]:
        with pytest.raises(o.OracleError) as e:
            o.tile(kind, 4, 4, axis=axis, size=size)
        assert e.value.code == o.ERR_GRANULARITY
    # group of full extent == per-channel twin (tests/quant.rs:306-318)
    assert o.tile(o.GROUP, 6, 4, axis=0, size=6) == o.tile(o.PER_CHANNEL, 6, 4, axis=1)
    w = kats.weights(24)
    ca, sa = o.quantize_host(w, 6, 4, 8, *o.tile(o.GROUP, 6, 4, axis=0, size=6))
    cb, sb = o.quantize_host(w, 6, 4, 8, *o.tile(o.PER_CHANNEL, 6, 4, axis=1))
    assert (ca == cb).all() and (bits(sa) == bits(sb)).all()


@pytest.mark.parametrize("case,b", [(kats.RTE_INT8, 8), (kats.RTE_INT4, 4)])
def test_rte_pins(case, b):
    codes, scales = o.quantize_host(case["w"], 2, 4, b, 2, 4)
    assert scales.tolist() == [[case["scale"]]]
    dq = o.dequantize_host(codes, scales, 2, 4, b, 2, 4)
    assert (bits(dq.reshape(-1)) == bits(case["deq"])).all()


@pytest.mark.parametrize("case", [kats.NIBBLE_ORDER, kats.ROW_PACKING])
def test_int4_packing_pins(case):
    r, c = case["rows"], case["cols"]
    codes, scales = o.quantize_host(case["w"], r, c, 4, r, c)
    assert scales.reshape(-1).tolist() == [case["scale"]]
    assert codes.reshape(-1).tolist() == case["words"]
    dq = o.dequantize_host(codes, scales, r, c, 4, r, c)
    assert (bits(dq.reshape(-1)) == bits(case["w"])).all()


def test_exact_multiples_round_trip():
    for ints, b in [(kats.EXACT_INT8, 8), (kats.EXACT_INT4, 4)]:
        codes, scales = o.quantize_host(ints, 2, 4, b, 2, 4)
        assert scales.reshape(-1).tolist() == [1.0]
        dq = o.dequantize_host(codes, scales, 2, 4, b, 2, 4)
        assert (bits(dq.reshape(-1)) == bits(ints)).all()


def test_from_parts_values():
    c8 = np.array(kats.FROM_PARTS_INT8["codes"], dtype=np.int8).reshape(2, 2)
    s = np.array(kats.FROM_PARTS_INT8["scales"], dtype=np.float32).reshape(2, 1)
    assert o.dequantize_host(c8, s, 2, 2, 8, 1, 2).reshape(-1).tolist() == kats.FROM_PARTS_INT8["deq"]
    c4 = np.array(kats.FROM_PARTS_INT4["words"], dtype=np.uint32).reshape(2, 1)
    assert o.dequantize_host(c4, s, 2, 2, 4, 1, 2).reshape(-1).tolist() == kats.FROM_PARTS_INT4["deq"]


def test_all_zero_tile():
    # tests/quant.rs:286-304 — Group{axis:1,size:2} over [4,4]; tile (2, 0..2) zeroed
    w = kats.weights(16)
    w[8] = 0.0
    w[9] = 0.0
    codes, scales = o.quantize_host(w, 4, 4, 8, 1, 2)
    assert scales.shape == (4, 2) and scales[2, 0] == 0.0
    dq = o.dequantize_host(codes, scales, 4, 4, 8, 1, 2)
    assert bits(dq)[2, 0] == 0 and bits(dq)[2, 1] == 0


@pytest.mark.parametrize("r,c,g", [(4, 8, 2), (5, 7, 3)])
def test_round_trip_within_half_scale(r, c, g):
    # tests/quant.rs:123-150 — the s/2 theorem with its stated 1e-4 slack
    w = kats.weights(r * c)
    for b in (8, 4):
        for kind, axis, size in kats.spellings(g):
            gr, gc = o.tile(kind, r, c, axis=axis, size=size)
            codes, scales = o.quantize_host(w, r, c, b, gr, gc)
            dq = o.dequantize_host(codes, scales, r, c, b, gr, gc).reshape(-1)
            tc = o.div_ceil(c, gc)
            for i in range(r * c):
                s = scales.reshape(-1)[(i // c // gr) * tc + (i % c) // gc]
                assert s > 0
                assert abs(dq[i] - w[i]) <= s * (0.5 + 1e-4)
            # clamp never fires: code lo is never produced (QuantRoundTrip.lean T9235)
            lo = kats.QUANT_RANGES[b][0]
            if b == 8:
                assert codes.min() > lo
            else:
                allq = [o.int4_unpack(int(wd), k) for wd in codes.reshape(-1) for k in range(8)]
                assert min(allq) > lo


def test_length_and_rank_errors():
    w = kats.weights(8)
    with pytest.raises(o.OracleError) as e:
        o.quantize_host(w, 3, 4, 8, 3, 4)
    assert e.value.code == o.ERR_LENGTH
    with pytest.raises(o.OracleError) as e:
        o.quantize_host(np.zeros(0, np.float32), 0, 4, 8, 1, 4)
    assert e.value.code == o.ERR_RANK
    codes, scales = o.quantize_host(w, 2, 4, 8, 2, 4)
    with pytest.raises(o.OracleError):
        o.dequantize_host(codes, scales, 2, 5, 8, 2, 5)
    with pytest.raises(o.OracleError):
        o.dequantize_host(codes, np.array([1.0, 2.0], np.float32), 2, 4, 8, 2, 4)


def test_linear_forward_orders_and_layouts():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 40)).astype(np.float32)
    w = rng.standard_normal((40, 24)).astype(np.float32)
    b = rng.standard_normal(24).astype(np.float32)
    y = o.linear_forward(x, w, b, o.IN_OUT)
    # sequential-k with separate multiply and add, spelled out
    want = np.empty((3, 24), np.float32)
    for i in range(3):
        for j in range(24):
            acc = np.float32(0)
            for p in range(40):
                acc = np.float32(acc + np.float32(x[i, p] * w[p, j]))
            want[i, j] = np.float32(acc + b[j])
    assert (bits(y) == bits(want)).all()
    yt = o.linear_forward(x, np.ascontiguousarray(w.T), b, o.OUT_IN)
    assert (bits(yt) == bits(y)).all()
    ypar = o.linear_forward(x, w, b, o.IN_OUT, threads=4)
    assert (bits(ypar) == bits(y)).all()
    y64 = o.linear_forward_f64(x, w, b, o.IN_OUT)
    assert np.allclose(y64, y, rtol=1e-5, atol=1e-5)


# ---- the quantized-safetensors convention ---------------------------------

def _leaf(kind, shape, vals):
    a = np.array(vals, dtype=np.float32).reshape(shape)
    if kind == "f32":
        return a
    b = 8 if kind == "q8" else 4
    r, c = shape
    codes, scales = o.quantize_host(a, r, c, b, r, c)
    return so.QLeaf(b, r, c, r, c, codes, scales)


def test_save_matches_reference_bytes():
    entries = [(n, _leaf(k, s, v)) for n, k, s, v in kats.REFERENCE_ENTRIES]
    assert so.save_named(entries, None) == kats.reference_quantized_bytes()
    w = np.array([1, 2, 3, 4], np.float32).reshape(2, 2)
    assert so.save_named([("w", w)], None) == kats.reference_plain_bytes()


def test_load_reference_bytes_and_resave():
    leaves, meta = so.load_named(kats.reference_quantized_bytes())
    assert meta == {} and [n for n, _ in leaves] == ["b", "w", "v"]
    assert leaves[1][1].codes.reshape(-1).tolist() == [1, -2, 3, -4, 5, -6, 7, 127]
    assert leaves[2][1].codes.reshape(-1).tolist() == [0xC3E7]
    assert leaves[1][1].gran == ("per_tensor",)
    assert so.save_named(leaves, None) == kats.reference_quantized_bytes()


def test_round_trip_non_divisible_edges():
    # tests/quant.rs:175-237
    w = kats.fill(30, 1).reshape(5, 6)
    u = kats.fill(40, 2).reshape(4, 10)
    gamma = kats.fill(6, 3)
    cw, sw = o.quantize_host(w, 5, 6, 8, 5, 1)
    cu, su = o.quantize_host(u, 4, 10, 4, 2, 1)
    entries = [("blk.w", so.QLeaf(8, 5, 6, 5, 1, cw, sw)), ("blk.u", so.QLeaf(4, 4, 10, 2, 1, cu, su)),
               ("ln.gamma", gamma)]
    meta = {"note": "trained on ramps"}
    b = so.save_named(entries, meta)
    leaves, m2 = so.load_named(b)
    assert m2 == meta and len(leaves) == 3
    assert leaves[0][1].gran == ("per_channel", 1) and leaves[1][1].gran == ("group", 0, 2)
    assert (leaves[0][1].codes == cw).all() and (leaves[1][1].codes == cu).all()
    assert (bits(leaves[1][1].scales) == bits(su)).all()
    assert so.save_named(leaves, m2) == b


def test_loud_errors():
    for label, f, needles in kats.loud_error_files():
        with pytest.raises(so.StError) as e:
            so.load_named(f)
        for n in needles:
            assert n in str(e.value), (label, str(e.value))


def test_meta_grammar_table():
    for s, want in kats.META_ACCEPT:
        m = so.parse_quant_meta("w", s)
        assert (m.bits, m.gr, m.gc, m.rows, m.cols) == want
    for s, needle in kats.META_REJECT:
        with pytest.raises(so.StError) as e:
            so.parse_quant_meta("w", s)
        assert needle in str(e.value), (s, str(e.value))


def test_save_side_collisions():
    q = _leaf("q8", [1, 2], [1.0, 2.0])
    with pytest.raises(so.StError) as e:
        so.save_named([("w", q)], {"quant:w": "spoof"})
    assert "quant:w" in str(e.value) and "collides" in str(e.value)
    with pytest.raises(so.StError) as e:
        so.save_named([("w", q), ("w.q", np.zeros((1, 2), np.float32))], None)
    assert "w.q" in str(e.value) and "collides" in str(e.value)


def test_plain_reader_cases():
    f = so.parse_raw(kats.reference_plain_bytes())
    assert f.entries[0].name == "w" and so.entry_to_f32(f.entries[0], f.data).tolist() == [1, 2, 3, 4]
    h = kats.st_file('{"h":{"dtype":"F16","shape":[3],"data_offsets":[0,6]}}',
                     struct.pack("<HHH", *kats.F16_CASE["halves"]))
    f = so.parse_raw(h)
    v = so.entry_to_f32(f.entries[0], f.data)
    assert v[0] == 1.0 and v[1] == -2.5 and abs(v[2] - 5.9604645e-8) < 1e-12
    bf = kats.st_file('{"b":{"dtype":"BF16","shape":[1],"data_offsets":[0,2]}}', struct.pack("<H", 0x4049))
    f = so.parse_raw(bf)
    assert so.entry_to_f32(f.entries[0], f.data)[0] == 3.140625
    with pytest.raises(so.StError):
        so.parse_raw(bytes([1, 2, 3]))
    with pytest.raises(so.StError):
        so.parse_raw(struct.pack("<Q", 2 ** 64 - 1) + b"{}")
    i64 = kats.st_file('{"q":{"dtype":"I64","shape":[1],"data_offsets":[0,8]}}', bytes(8))
    f = so.parse_raw(i64)
    with pytest.raises(so.StError) as e:
        so.entry_to_f32(f.entries[0], f.data)
    assert "I64" in str(e.value)
