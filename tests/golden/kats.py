"""Known-answer data for the quantized-inference path.

Every literal below is a fixture the reference's own test-suites hold for this
path, restated as data (file:line given per block).  The two input generators
are the reference tests' closed-form generators restated in f32 arithmetic.
"""
from __future__ import annotations

import struct

import numpy as np

f32 = np.float32

# crates/gpu/quanta-ir/src/dtype.rs:408-411
QUANT_RANGES = {8: (-128, 127), 4: (-8, 7)}

# crates/gpu/quanta-ir/src/dtype.rs:413-434 — start word of the pack/unpack sweep
PACK_SWEEP_WORD = 0xDEADBEEF

# crates/gpu/quanta-ir/src/dtype.rs:436-451 — (x, scale, bits, code)
QUANTIZE_SYM = [
    (0.0, 0.5, 4, 0), (0.5, 0.5, 4, 1), (-1.0, 0.5, 4, -2), (3.5, 0.5, 4, 7), (3.6, 0.5, 4, 7),
    (-5.0, 0.5, 4, -8), (0.24, 0.5, 4, 0), (0.26, 0.5, 4, 1), (300.0, 1.0, 8, 127),
]
# (code, scale, value)
DEQUANTIZE_SYM = [(7, 0.5, 3.5), (-8, 0.5, -4.0)]


# crates/gpu/quanta-ir/src/op_matrix_cases.rs:1680-1697 — inputs for scale s;
# expected codes (0 ulp) follow from the comments there: ties round to even,
# +-1000 clamp to hi / lo.
def op_matrix_inputs(scale):
    s = f32(scale)
    return [f32(0.0), s, -s, f32(2.0) * s, f32(-3.0) * s, f32(0.5) * s, f32(1.5) * s, f32(2.5) * s,
            f32(1000.0), f32(-1000.0), f32(0.49) * s, f32(0.51) * s]


def op_matrix_expected(bits):
    lo, hi = QUANT_RANGES[bits]
    return [0, 1, -1, 2, -3, 0, 2, 2, hi, lo, 0, 1]


# crates/sci/quanta-array/tests/quant.rs:34-41
def weights(n: int) -> np.ndarray:
    i = np.arange(n, dtype=np.float32)
    x = i * f32(0.7311) - f32(n) * f32(0.317)
    neg = (-x) * f32(0.13)
    pos = x * f32(0.171)
    return np.where(np.arange(n) % 3 == 0, neg, pos).astype(np.float32)


# crates/ml/quanta-nn/tests/quant.rs:60-72 (splitmix64 mixer -> [-1, 1))
def fill(n: int, seed: int) -> np.ndarray:
    M = 0xFFFFFFFFFFFFFFFF
    s = (seed + 0x9E3779B97F4A7C15) & M
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = (s + 0x9E3779B97F4A7C15) & M
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        z ^= z >> 31
        out[i] = f32(f32(f32(z >> 40) / f32(1 << 24)) * f32(2.0)) - f32(1.0)
    return out


# crates/sci/quanta-array/tests/quant.rs:75-115 — (rows, cols, group) shape grid
DEVICE_HOST_SHAPES = [(4, 8, 2), (5, 7, 3), (5, 13, 4), (16, 32, 8)]


def spellings(g):
    """The five granularity spellings as (kind, axis, size) — tests/quant.rs:52-60."""
    return [(0, 0, 0), (1, 0, 0), (1, 1, 0), (2, 0, g), (2, 1, g)]


# crates/sci/quanta-array/tests/quant.rs:177-205 — RTE pins (per-tensor, [2,4])
RTE_INT8 = dict(w=[63.5, -63.5, 0.25, 0.26, 0.75, -0.75, 1.0, 0.0], scale=0.5,
                deq=[63.5, -63.5, 0.0, 0.5, 1.0, -1.0, 1.0, 0.0])
RTE_INT4 = dict(w=[3.5, -3.5, 0.25, 0.26, 0.75, -0.75, 1.0, 0.0], scale=0.5,
                deq=[3.5, -3.5, 0.0, 0.5, 1.0, -1.0, 1.0, 0.0])

# crates/sci/quanta-array/tests/quant.rs:216-225
NIBBLE_ORDER = dict(w=[1.0, 2.0, -1.0, -7.0, 7.0, 0.0, 3.0, -3.0], rows=1, cols=8, scale=1.0,
                    words=[0xD3079F21])
# crates/sci/quanta-array/tests/quant.rs:227-243
ROW_PACKING = dict(w=[1.0, -1.0, 2.0, 3.0, -2.0, 7.0], rows=2, cols=3, scale=1.0, words=[0x2F1, 0x7E3])

# crates/sci/quanta-array/tests/quant.rs:152-169
EXACT_INT8 = [127.0, -127.0, 1.0, -1.0, 64.0, -33.0, 0.0, 100.0]
EXACT_INT4 = [7.0, -7.0, 1.0, -1.0, 3.0, -2.0, 0.0, 5.0]

# crates/sci/quanta-array/tests/quant.rs:247-282 — from_parts, PerChannel{axis:0} over [2,2]
FROM_PARTS_INT8 = dict(codes=[2, -2, 4, -4], scales=[0.5, 0.25], deq=[1.0, -1.0, 1.0, -1.0])
FROM_PARTS_INT4 = dict(words=[0xF1, 0xE2], scales=[0.5, 0.25], deq=[0.5, -0.5, 0.5, -0.5])


# ---- quantized-safetensors fixtures: crates/ml/quanta-nn/tests/quant.rs -----

def st_file(header: str, data: bytes) -> bytes:
    """tests/quant.rs:44-53 — 8-byte LE length, space-padded header, data."""
    hb = header.encode("utf-8")
    while (len(hb) + 8) % 8 != 0:
        hb += b" "
    return struct.pack("<Q", len(hb)) + hb + data


# tests/quant.rs:80-101
def reference_quantized_bytes() -> bytes:
    header = (
        '{"__metadata__":{"quant:v":"q4s;gr=1;gc=4;rows=1;cols=4",'
        '"quant:w":"q8s;gr=2;gc=4;rows=2;cols=4","quanta.quant":"1"},'
        '"b":{"dtype":"F32","shape":[2],"data_offsets":[0,8]},'
        '"w.q":{"dtype":"I8","shape":[2,4],"data_offsets":[8,16]},'
        '"w.qs":{"dtype":"F32","shape":[1,1],"data_offsets":[16,20]},'
        '"v.q":{"dtype":"U32","shape":[1,1],"data_offsets":[20,24]},'
        '"v.qs":{"dtype":"F32","shape":[1,1],"data_offsets":[24,28]}}'
    )
    data = struct.pack("<ff", 0.5, -1.5)
    data += bytes([0x01, 0xFE, 0x03, 0xFC, 0x05, 0xFA, 0x07, 0x7F])
    data += struct.pack("<f", 1.0)
    data += struct.pack("<I", 0x0000C3E7)
    data += struct.pack("<f", 1.0)
    return st_file(header, data)


# tests/quant.rs:103-129 — the leaves whose save must equal the bytes above
REFERENCE_ENTRIES = [
    ("b", "f32", [2], [0.5, -1.5]),
    ("w", "q8", [2, 4], [1.0, -2.0, 3.0, -4.0, 5.0, -6.0, 7.0, 127.0]),  # PerTensor
    ("v", "q4", [1, 4], [7.0, -2.0, 3.0, -4.0]),  # PerTensor
]


# crates/ml/quanta-nn/tests/safetensors.rs:26-38
def reference_plain_bytes() -> bytes:
    return st_file('{"w":{"dtype":"F32","shape":[2,2],"data_offsets":[0,16]}}', struct.pack("<ffff", 1, 2, 3, 4))


# crates/ml/quanta-nn/tests/safetensors.rs:102-131
F16_CASE = dict(halves=[0x3C00, 0xC100, 0x0001], values=[1.0, -2.5, 5.9604645e-8])
BF16_CASE = dict(bits=0x4049, value=3.140625)

_META_W = '"quant:w":"q8s;gr=1;gc=2;rows=1;cols=2"'
_BASE = bytes([0x01, 0xFE, 0x00, 0x00, 0x80, 0x3F])
_WQ = '"w.q":{"dtype":"I8","shape":[1,2],"data_offsets":[0,2]}'
_WQS = '"w.qs":{"dtype":"F32","shape":[1,1],"data_offsets":[2,6]}'


def loud_error_files():
    """tests/quant.rs:280-413 — (label, file bytes, substrings the message must hold)."""
    nan = struct.pack("<f", float("nan"))
    return [
        ("unknown version", st_file('{"__metadata__":{%s,"quanta.quant":"2"},%s,%s}' % (_META_W, _WQ, _WQS), _BASE),
         ["version 2", "reads 1"]),
        ("missing version", st_file('{"__metadata__":{%s},%s,%s}' % (_META_W, _WQ, _WQS), _BASE),
         ["quanta.quant", "missing"]),
        ("orphan metadata", st_file('{"__metadata__":{%s,"quanta.quant":"1"}}' % _META_W, b""), ["w.q", "missing"]),
        ("orphan codes", st_file('{%s}' % _WQ, _BASE[:2]), ["w.q", "no quant:"]),
        ("tensor beside quant", st_file(
            '{"__metadata__":{%s,"quanta.quant":"1"},"w":{"dtype":"F32","shape":[2],"data_offsets":[6,14]},%s,%s}'
            % (_META_W, _WQ, _WQS), _BASE + bytes(8)), ["both a tensor"]),
        ("reserved qz", st_file(
            '{"__metadata__":{%s,"quanta.quant":"1"},%s,%s,"w.qz":{"dtype":"F32","shape":[1,1],"data_offsets":[6,10]}}'
            % (_META_W, _WQ, _WQS), _BASE + bytes(4)), ["w.qz", "reserved affine"]),
        ("unknown tag", st_file(
            '{"__metadata__":{"quant:w":"q5s;gr=1;gc=2;rows=1;cols=2","quanta.quant":"1"},%s,%s}' % (_WQ, _WQS), _BASE),
         ["q5s"]),
        ("affine mode", st_file(
            '{"__metadata__":{"quant:w":"q8s;gr=1;gc=2;rows=1;cols=2;mode=affine","quanta.quant":"1"},%s,%s}'
            % (_WQ, _WQS), _BASE), ["affine"]),
        ("codes dtype", st_file(
            '{"__metadata__":{"quant:w":"q4s;gr=1;gc=2;rows=1;cols=2","quanta.quant":"1"},%s,%s}' % (_WQ, _WQS), _BASE),
         ["U32"]),
        ("scales shape", st_file(
            '{"__metadata__":{%s,"quanta.quant":"1"},%s,"w.qs":{"dtype":"F32","shape":[1,2],"data_offsets":[2,10]}}'
            % (_META_W, _WQ), _BASE[:2] + bytes(8)), ["w.qs", "wants"]),
        ("non-finite scale", st_file('{"__metadata__":{%s,"quanta.quant":"1"},%s,%s}' % (_META_W, _WQ, _WQS),
                                     _BASE[:2] + nan), ["w", "non-finite"]),
        ("not a v1 grid", st_file(
            '{"__metadata__":{"quant:w":"q8s;gr=3;gc=2;rows=4;cols=4","quanta.quant":"1"},'
            '"w.q":{"dtype":"I8","shape":[4,4],"data_offsets":[0,16]},'
            '"w.qs":{"dtype":"F32","shape":[2,2],"data_offsets":[16,32]}}', bytes(32)), ["not a v1 tile grid"]),
    ]


# crates/ml/quanta-nn/src/quant.rs:949-969 — metadata grammar accept / reject table
META_ACCEPT = [("q8s;gr=1;gc=4;rows=2;cols=4", (8, 1, 4, 2, 4)), ("q4s;cols=4;rows=2;gc=4;gr=1", (4, 1, 4, 2, 4))]
META_REJECT = [
    ("q5s;gr=1;gc=1;rows=1;cols=1", "q5s"), ("q8s;gr=1;gc=1;rows=1", "cols"),
    ("q8s;gr=1;gc=1;rows=1;cols=1;mode=affine", "affine"), ("q8s;gr=0;gc=1;rows=1;cols=1", "gr=0"),
    ("q8s;gr=1;gr=2;gc=1;rows=1;cols=1", "duplicate"), ("q8s;gr=1;gc=1;rows=1;cols=1;zp=3", "zp"),
    ("q8s;gr;gc=1;rows=1;cols=1", "key=value"),
]


# crates/sci/quanta-blas/src/reference.rs:1119-1148 — the two literal cases of the quantized-GEMM oracle's own tests
# (gemm_q8_sym_basic, gemm_q4_sym_basic): m, n, k, alpha, a_scale, b_scale, A codes, B codes, beta, expected C.
GEMM_Q8_SYM_BASIC = {"m": 2, "n": 2, "k": 2, "alpha": 1.0, "a_scale": 0.5, "b_scale": 0.25, "a": [2, 4, 6, 8],
                     "b": [1, 0, 0, 1], "beta": 0.0, "c": [0.25, 0.5, 0.75, 1.0]}
# int4 codes, each matrix packed into one u32 word by flat index (nibbles 0..3)
GEMM_Q4_SYM_BASIC = {"m": 2, "n": 2, "k": 2, "alpha": 1.0, "a_scale": 1.0, "b_scale": 2.0, "a": [1, 2, 3, -1],
                     "b": [1, 0, 0, 1], "beta": 0.0, "c": [2.0, 4.0, 6.0, -2.0]}
