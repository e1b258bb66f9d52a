"""Host-side logic of the product library (no GPU needed): the C ABI loads and exports
every declared symbol, the grid vocabulary and its loud errors, and the quantized-
safetensors writer / validator against the reference's hand-built files and the oracle."""
import ctypes
import os
import re
import struct

import numpy as np
import pytest
import torch

import oracle as o
import quanta_b200 as qb
from oracle import safetensors_oracle as so
from quanta_b200 import _lib
from tests.golden import kats

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "qb200.h")).read()
    declared = set(re.findall(r"QB200_API [\w\* ]+?(qb200_\w+)\(", header))
    assert len(declared) >= 30
    lib = ctypes.CDLL(_lib.lib_path())
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.load().qb200_version().decode().count(".") == 2


def test_tile_spellings():
    assert qb.PerTensor().tile(5, 7) == (5, 7)
    assert qb.PerChannel(0).tile(5, 7) == (1, 7)
    assert qb.PerChannel(1).tile(5, 7) == (5, 1)
    assert qb.Group(0, 3).tile(5, 7) == (3, 1)
    assert qb.Group(1, 3).tile(5, 7) == (1, 3)
    assert qb.Block(32, 32).tile(1024, 1024) == (32, 32)
    assert qb.Group(0, 6).tile(6, 4) == qb.PerChannel(1).tile(6, 4)
    for kind, axis, size in kats.spellings(3):
        g = qb.Granularity(kind, axis, size)
        assert g.tile(5, 7) == o.tile(kind, 5, 7, axis=axis, size=size)


def test_granularity_errors_are_loud():
    # quanta-array/tests/quant.rs:368-394
    for g in [qb.PerChannel(2), qb.Group(3, 2), qb.Group(0, 0), qb.Group(1, 99), qb.Block(0, 4), qb.Block(2, 9)]:
        with pytest.raises(qb.QuantError) as e:
            g.tile(4, 4)
        assert e.value.kind == "Granularity"
    with pytest.raises(qb.QuantError) as e:
        qb.Group(1, 99).tile(4, 4)
    assert "99" in str(e.value) and "4" in str(e.value)


def test_granularity_from_grid_precedence():
    f = qb.granularity_from_grid
    assert f(4, 6, 4, 6) == qb.PerTensor()
    assert f(4, 6, 1, 6) == qb.PerChannel(0)
    assert f(4, 6, 4, 1) == qb.PerChannel(1)
    assert f(4, 6, 2, 1) == qb.Group(0, 2)
    assert f(4, 6, 1, 3) == qb.Group(1, 3)
    with pytest.raises(qb.QuantError) as e:
        f(4, 4, 3, 2)
    assert "not a v1 tile grid" in str(e.value)
    assert f(64, 64, 32, 32, allow_block=True) == qb.Block(32, 32)
    for rows, cols, gr, gc in [(4, 6, 4, 6), (4, 6, 1, 6), (4, 6, 2, 1), (8, 8, 3, 2), (5, 5, 0, 1), (5, 5, 9, 1)]:
        want = so.granularity_from_grid(rows, cols, gr, gc)
        if want is None:
            with pytest.raises(qb.QuantError):
                f(rows, cols, gr, gc)
        else:
            got = f(rows, cols, gr, gc)
            assert {0: "per_tensor", 1: "per_channel", 2: "group"}[got.kind] == want[0]


def test_from_parts_validation():
    # quanta-array/tests/quant.rs:397-435
    codes = torch.tensor([[1, 2], [3, 4]], dtype=torch.int8)
    with pytest.raises(qb.QuantError) as e:
        qb.QuantizedMatrix.from_parts(codes, [4, 2], torch.ones(1, 1), qb.PerTensor())
    assert e.value.kind == "Grid" and "[4, 2]" in str(e.value)
    with pytest.raises(qb.QuantError) as e:
        qb.QuantizedMatrix.from_parts(codes, [2, 2], torch.ones(1, 2), qb.PerChannel(0))
    assert e.value.kind == "Grid"
    words = torch.zeros(2, 2, dtype=torch.int32)
    with pytest.raises(qb.QuantError) as e:
        qb.QuantizedMatrix.from_parts(words, [2, 17], torch.ones(1, 1), qb.PerTensor())
    assert e.value.kind == "Grid"
    with pytest.raises(qb.QuantError) as e:
        qb.QuantizedMatrix.from_parts(codes, [0, 2], torch.ones(1, 1), qb.PerTensor())
    assert e.value.kind == "Rank" and "rank-2" in str(e.value)
    m = qb.QuantizedMatrix.from_parts(codes, [2, 2], torch.ones(2, 1), qb.PerChannel(0))
    assert m.shape() == [2, 2] and m.dtype() is qb.QuantDtype.Int8 and m.tile() == (1, 2)


def test_rank_error_on_quantize():
    for shape in ([6], [2, 2, 2]):
        with pytest.raises(qb.QuantError) as e:
            qb.QuantizedMatrix.quantize(torch.zeros(shape), qb.QuantDtype.Int8, qb.PerTensor())
        assert e.value.kind == "Rank" and "rank-2" in str(e.value)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device refusal")
def test_no_device_is_a_loud_error_not_a_fallback():
    a = torch.zeros(4, 8)
    with pytest.raises(qb.QuantError) as e:
        qb.QuantizedMatrix.quantize(a, qb.QuantDtype.Int8, qb.PerTensor())
    assert e.value.kind == "Cuda"
    m = qb.QuantizedMatrix.from_parts(torch.zeros(4, 8, dtype=torch.int8), [4, 8], torch.ones(1, 1), qb.PerTensor())
    with pytest.raises(qb.QuantError) as e:
        m.dequantize()
    assert e.value.kind == "Cuda"
    with pytest.raises(qb.QuantError) as e:
        qb.QuantizedLinear.new(m)
    assert e.value.kind == "Cuda"


# ---- quantized-safetensors --------------------------------------------------

def _qm(kind, shape, vals, gran=None):
    """Host-resident QuantizedMatrix with oracle-computed codes (the writer only moves bytes)."""
    a = np.array(vals, dtype=np.float32).reshape(shape)
    if kind == "f32":
        return qb.QuantLeaf.F32(torch.from_numpy(a))
    bits = 8 if kind == "q8" else 4
    gran = gran or qb.PerTensor()
    gr, gc = gran.tile(*shape)
    codes, scales = o.quantize_host(a, shape[0], shape[1], bits, gr, gc)
    ct = torch.from_numpy(codes if bits == 8 else codes.view(np.int32))
    return qb.QuantLeaf.Quantized(qb.QuantizedMatrix.from_parts(ct, list(shape), torch.from_numpy(scales), gran))


def test_save_matches_the_reference_bytes():
    entries = [(n, _qm(k, s, v)) for n, k, s, v in kats.REFERENCE_ENTRIES]
    assert qb.save_named(entries, None) == kats.reference_quantized_bytes()
    w = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    assert qb.save_named([("w", qb.QuantLeaf.F32(w))], None) == kats.reference_plain_bytes()


def test_load_reference_bytes_mode_b_on_host():
    loaded = qb.load_named("cpu", kats.reference_quantized_bytes())
    assert loaded.metadata == {} and [n for n, _ in loaded.leaves] == ["b", "w", "v"]
    b, w, v = (leaf.value for _, leaf in loaded.leaves)
    assert b.tolist() == [0.5, -1.5]
    assert w.codes().reshape(-1).tolist() == [1, -2, 3, -4, 5, -6, 7, 127] and w.granularity() == qb.PerTensor()
    assert v.codes().reshape(-1).tolist() == [0xC3E7] and v.shape() == [1, 4] and v.dtype() is qb.QuantDtype.Int4
    assert qb.save_named(loaded.leaves, None) == kats.reference_quantized_bytes()


def test_round_trip_non_divisible_edges_and_resave_identity():
    # quanta-nn/tests/quant.rs:175-237
    entries = [("blk.w", _qm("q8", (5, 6), kats.fill(30, 1), qb.PerChannel(1))),
               ("blk.u", _qm("q4", (4, 10), kats.fill(40, 2), qb.Group(0, 2))),
               ("ln.gamma", qb.QuantLeaf.F32(torch.from_numpy(kats.fill(6, 3))))]
    meta = {"note": "trained on ramps"}
    data = qb.save_named(entries, meta)
    loaded = qb.load_named("cpu", data)
    assert loaded.metadata == meta and len(loaded.leaves) == 3
    for (n0, l0), (n1, l1) in zip(entries, loaded.leaves):
        assert n0 == n1 and l0.is_quantized == l1.is_quantized
        if l0.is_quantized:
            a, b = l0.value, l1.value
            assert a.shape() == b.shape() and a.dtype() == b.dtype() and a.tile() == b.tile()
            assert a.granularity() == b.granularity()
            assert torch.equal(a.codes(), b.codes())
            assert torch.equal(a.scales().view(torch.int32), b.scales().view(torch.int32))
        else:
            assert torch.equal(l0.value.view(torch.int32), l1.value.view(torch.int32))
    assert qb.save_named(loaded.leaves, loaded.metadata) == data
    # and the oracle writer agrees byte for byte
    oe = []
    for n, l in entries:
        if l.is_quantized:
            m = l.value
            c = m.codes().numpy()
            oe.append((n, so.QLeaf(m.dtype().bits(), *m.shape(), *m.tile(), c if c.dtype == np.int8 else c.view(np.uint32),
                                   m.scales().numpy())))
        else:
            oe.append((n, l.value.numpy()))
    assert so.save_named(oe, meta) == data


def test_loud_errors_name_the_problem():
    for label, f, needles in kats.loud_error_files():
        for loader in (qb.load_named, qb.load_named_f32):
            with pytest.raises(qb.QuantError) as e:
                loader("cpu", f)
            for n in needles:
                assert n in str(e.value), (label, str(e.value))
        # same arm as the oracle
        with pytest.raises(so.StError) as oe:
            so.load_named(f)
        want = {"format": "Format", "scale": "Scale", "param": "InvalidParam"}[oe.value.kind]
        assert e.value.kind == want, (label, e.value.kind, want)
        assert str(e.value).split(" (")[0] == str(oe.value).split(" (")[0], label


def test_block_grid_is_refused_by_default_and_admitted_on_request():
    m = _qm("q8", (64, 64), np.linspace(-1, 1, 4096), qb.Block(32, 32))
    data = qb.save_named([("w", m)], None)
    with pytest.raises(qb.QuantError) as e:
        qb.load_named("cpu", data)
    assert "not a v1 tile grid" in str(e.value)
    back = qb.load_named("cpu", data, allow_block=True).leaves[0][1].value
    assert back.granularity() == qb.Block(32, 32) and back.scales().shape == (2, 2)


def test_save_side_collisions():
    q = _qm("q8", (1, 2), [1.0, 2.0])
    with pytest.raises(qb.QuantError) as e:
        qb.save_named([("w", q)], {"quant:w": "spoof"})
    assert "quant:w" in str(e.value) and "collides" in str(e.value)
    with pytest.raises(qb.QuantError) as e:
        qb.save_named([("w", q), ("w.q", qb.QuantLeaf.F32(torch.zeros(1, 2)))], None)
    assert "w.q" in str(e.value) and "collides" in str(e.value)
    with pytest.raises(qb.QuantError) as e:
        qb.save_named([("w", q), ("w", q)], None)
    assert "duplicate leaf name" in str(e.value)


def test_metadata_grammar_table():
    lib = _lib.load()
    for s, want in kats.META_ACCEPT + [("q8s;gr=+1;gc=4;rows=2;cols=4", (8, 1, 4, 2, 4))]:
        bits, gr, gc, rows, cols = _lib.u32(), _lib.u64(), _lib.u64(), _lib.u64(), _lib.u64()
        assert lib.qb200_st_parse_quant_meta(b"w", s.encode(), *(ctypes.byref(v) for v in (bits, gr, gc, rows, cols))) == 0
        assert (bits.value, gr.value, gc.value, rows.value, cols.value) == want
        m = so.parse_quant_meta("w", s)
        assert (m.bits, m.gr, m.gc, m.rows, m.cols) == want
    for s, needle in kats.META_REJECT + [("q8s;gr=-1;gc=1;rows=1;cols=1", "not a positive integer"),
                                          ("q8s;gr=1x;gc=1;rows=1;cols=1", "not a positive integer")]:
        bits, gr, gc, rows, cols = _lib.u32(), _lib.u64(), _lib.u64(), _lib.u64(), _lib.u64()
        rc = lib.qb200_st_parse_quant_meta(b"w", s.encode(), *(ctypes.byref(v) for v in (bits, gr, gc, rows, cols)))
        assert rc == _lib.ERR_FORMAT and needle in _lib.last_error(), (s, _lib.last_error())


def test_plain_container_cases():
    # quanta-nn/tests/safetensors.rs
    t = qb.load_named("cpu", kats.reference_plain_bytes())
    assert t.leaves[0][0] == "w" and t.leaves[0][1].value.tolist() == [[1.0, 2.0], [3.0, 4.0]]
    h = kats.st_file('{"h":{"dtype":"F16","shape":[3],"data_offsets":[0,6]}}', struct.pack("<HHH", *kats.F16_CASE["halves"]))
    v = qb.load_named("cpu", h).leaves[0][1].value
    assert v[0] == 1.0 and v[1] == -2.5 and abs(float(v[2]) - 5.9604645e-8) < 1e-12
    bf = kats.st_file('{"b":{"dtype":"BF16","shape":[1],"data_offsets":[0,2]}}', struct.pack("<H", 0x4049))
    assert qb.load_named("cpu", bf).leaves[0][1].value[0] == 3.140625
    for bad in (bytes([1, 2, 3]), struct.pack("<Q", 2 ** 64 - 1) + b"{}"):
        with pytest.raises(qb.QuantError):
            qb.load_named("cpu", bad)
    i64 = kats.st_file('{"q":{"dtype":"I64","shape":[1],"data_offsets":[0,8]}}', bytes(8))
    with pytest.raises(qb.QuantError) as e:
        qb.load_named("cpu", i64)
    assert "I64" in str(e.value) and "q" in str(e.value)
    meta = {"format": "pt", "note": 'quanta "test"'}
    data = qb.save_named([("w", qb.QuantLeaf.F32(torch.tensor([0.5])))], meta)
    assert qb.load_named("cpu", data).metadata == meta
    assert data == so.save_named([("w", np.array([0.5], np.float32))], meta)


def test_malformed_headers_agree_with_the_oracle():
    cases = [b'{"w":{"dtype":"F32","shape":[1],"data_offsets":[0,4]', b'{"w":{"dtype":"F32","shape":[1.5],"data_offsets":[0,4]}}',
             b'{"w":{"dtype":"F32","shape":[1],"data_offsets":[0,4],"x":1}}', b'{"w":{"dtype":"F32","shape":[1]}}',
             b'{"w":{"dtype":"F32","shape":[1],"data_offsets":[4,0]}}', b'{"w":{"dtype":"F32","shape":[1],"data_offsets":[0,8]}}',
             b'{"__metadata__":{"a":1},"w":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}',
             b'{"w\\q":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}', b'[1]', b'{"w":3}',
             b'{"w":{"dtype":"F32","shape":[99999999999999999999],"data_offsets":[0,4]}}',
             '{"wé\\u00e9":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'.encode("utf-8")]
    for hdr in cases:
        f = kats.st_file(hdr.decode("utf-8"), bytes(4))
        try:
            so.load_named(f)
            want = None
        except so.StError as e:
            want = str(e)
        if want is None:
            qb.load_named("cpu", f)
        else:
            with pytest.raises(qb.QuantError) as e:
                qb.load_named("cpu", f)
            assert str(e.value) == want, hdr


def test_tree_load_errors():
    data = qb.save_named([("not_w", qb.QuantLeaf.F32(torch.zeros(4, 2)))], None)
    with pytest.raises(qb.QuantError) as e:
        qb.load("cpu", {"w": torch.zeros(4, 2)}, data)
    assert "missing tensor" in str(e.value)
    data = qb.save_named([("w", qb.QuantLeaf.F32(torch.zeros(4, 2))), ("extra", qb.QuantLeaf.F32(torch.ones(1)))], None)
    with pytest.raises(qb.QuantError) as e:
        qb.load("cpu", {"w": torch.zeros(4, 2)}, data)
    assert "no home" in str(e.value)
    data = qb.save_named([("w", qb.QuantLeaf.F32(torch.zeros(2, 4)))], None)
    with pytest.raises(qb.QuantError) as e:
        qb.load("cpu", {"w": torch.zeros(4, 2)}, data)
    assert "shape" in str(e.value)


def test_quantized_linear_rejects_a_mismatched_bias():
    m = _qm("q8", (2, 4), kats.fill(8, 4)).value
    with pytest.raises(qb.QuantError) as e:
        qb.QuantizedLinear.new(m, torch.zeros(3))
    assert "bias" in str(e.value)
