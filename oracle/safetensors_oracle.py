"""Pure-Python restatement of the reference's quantized-safetensors convention.

TEST INFRASTRUCTURE ONLY (the checker for the product's C++ reader/writer).
Parity status: PINNED against the hand-built reference files of
crates/ml/quanta-nn/tests/quant.rs:80-101 and tests/safetensors.rs:26-38, the
sixteen loud-error files of tests/quant.rs:280-436 and the metadata grammar
table of crates/ml/quanta-nn/src/quant.rs:949-969.

Follows:
  container writer   crates/ml/quanta-nn/src/safetensors.rs:41-125
  header parser      crates/ml/quanta-nn/src/safetensors.rs:163-348
  parse_raw          crates/ml/quanta-nn/src/safetensors.rs:398-492
  entry_to_f32       crates/ml/quanta-nn/src/safetensors.rs:497-551
  metadata grammar   crates/ml/quanta-nn/src/quant.rs:186-271
  save_named         crates/ml/quanta-nn/src/quant.rs:279-390
  validate           crates/ml/quanta-nn/src/quant.rs:420-635
  granularity_from_grid  crates/ml/quanta-nn/src/quant.rs:119-145
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

FORMAT_VERSION = "1"
VERSION_KEY = "quanta.quant"
META_PREFIX = "quant:"


class StError(Exception):
    """kind: 'format' (QuantError::Format), 'scale' (QuantError::Scale), 'param' (invalid_param)."""

    def __init__(self, kind: str, msg: str):
        super().__init__(msg)
        self.kind = kind


def _format_err(leaf: str, what: str) -> StError:
    return StError("format", f"quantized checkpoint leaf `{leaf}`: {what}")


def _bad(msg: str) -> StError:
    return StError("param", msg)


def _rust_list(v) -> str:
    return "[" + ", ".join(str(int(d)) for d in v) + "]"


# ---- writer (safetensors.rs:41-125) ------------------------------------------

def json_escape(s: str) -> str:
    out = ['"']
    for c in s:
        if c == '"':
            out.append('\\"')
        elif c == "\\":
            out.append("\\\\")
        elif c == "\n":
            out.append("\\n")
        elif c == "\r":
            out.append("\\r")
        elif c == "\t":
            out.append("\\t")
        elif ord(c) < 0x20:
            out.append("\\u%04x" % ord(c))
        else:
            out.append(c)
    out.append('"')
    return "".join(out)


def save_raw(entries, metadata) -> bytes:
    """entries: list of (name, dtype_str, shape, bytes); metadata: dict or None."""
    header = "{"
    data = bytearray()
    first = True
    if metadata is not None:
        keys = sorted(metadata.keys(), key=lambda k: k.encode("utf-8"))
        header += '"__metadata__":{'
        header += ",".join(json_escape(k) + ":" + json_escape(metadata[k]) for k in keys)
        header += "}"
        first = False
    for name, dtype, shape, b in entries:
        if not first:
            header += ","
        first = False
        start = len(data)
        data += b
        header += json_escape(name) + ':{"dtype":"' + dtype + '","shape":['
        header += ",".join(str(int(d)) for d in shape)
        header += '],"data_offsets":[%d,%d]}' % (start, len(data))
    header += "}"
    hb = header.encode("utf-8")
    while (len(hb) + 8) % 8 != 0:
        hb += b" "
    return struct.pack("<Q", len(hb)) + hb + bytes(data)


# ---- header parser (safetensors.rs:163-348) ----------------------------------

class _Parser:
    def __init__(self, b: bytes):
        self.b = b
        self.i = 0

    def err(self, msg):
        return _bad(f"safetensors header: {msg} at byte {self.i}")

    def skip_ws(self):
        while self.i < len(self.b) and self.b[self.i] in b" \t\n\r":
            self.i += 1

    def expect(self, c: int):
        self.skip_ws()
        if self.i < len(self.b) and self.b[self.i] == c:
            self.i += 1
        else:
            raise self.err("expected '%s'" % chr(c))

    def peek(self):
        self.skip_ws()
        return self.b[self.i] if self.i < len(self.b) else None

    def value(self):
        c = self.peek()
        if c == ord('"'):
            return self.string()
        if c == ord("{"):
            return self.object()
        if c == ord("["):
            return self.array()
        if c is not None and ord("0") <= c <= ord("9"):
            return self.number()
        raise self.err("expected a value")

    def string(self):
        self.expect(ord('"'))
        s = []
        while True:
            if self.i >= len(self.b):
                raise self.err("unterminated string")
            c = self.b[self.i]
            self.i += 1
            if c == ord('"'):
                return "".join(s)
            if c == ord("\\"):
                if self.i >= len(self.b):
                    raise self.err("dangling escape")
                e = self.b[self.i]
                self.i += 1
                simple = {ord('"'): '"', ord("\\"): "\\", ord("/"): "/", ord("b"): "\b", ord("f"): "\f",
                          ord("n"): "\n", ord("r"): "\r", ord("t"): "\t"}
                if e in simple:
                    s.append(simple[e])
                elif e == ord("u"):
                    hexs = self.b[self.i:self.i + 4]
                    if len(hexs) < 4:
                        raise self.err("truncated \\u escape")
                    try:
                        txt = hexs.decode("ascii")
                        if not all(ch in "0123456789abcdefABCDEF" for ch in txt):
                            raise ValueError
                        code = int(txt, 16)
                    except (UnicodeDecodeError, ValueError):
                        raise self.err("bad \\u escape")
                    self.i += 4
                    if 0xD800 <= code <= 0xDFFF:
                        raise self.err("surrogate in \\u escape")
                    s.append(chr(code))
                else:
                    raise self.err("unknown escape")
            elif c < 0x80:
                s.append(chr(c))
            else:
                start = self.i - 1
                if 0xC0 <= c <= 0xDF:
                    n = 2
                elif 0xE0 <= c <= 0xEF:
                    n = 3
                elif 0xF0 <= c <= 0xF7:
                    n = 4
                else:
                    raise self.err("invalid utf-8")
                chunk = self.b[start:start + n]
                if len(chunk) < n:
                    raise self.err("truncated utf-8")
                try:
                    s.append(chunk.decode("utf-8"))
                except UnicodeDecodeError:
                    raise self.err("invalid utf-8")
                self.i = start + n

    def number(self):
        self.skip_ws()
        start = self.i
        while self.i < len(self.b) and ord("0") <= self.b[self.i] <= ord("9"):
            self.i += 1
        if start == self.i:
            raise self.err("expected a number")
        v = int(self.b[start:self.i])
        if v > 0xFFFFFFFFFFFFFFFF:
            raise self.err("integer out of range")
        return v

    def array(self):
        self.expect(ord("["))
        items = []
        if self.peek() == ord("]"):
            self.i += 1
            return items
        while True:
            items.append(self.value())
            c = self.peek()
            if c == ord(","):
                self.i += 1
            elif c == ord("]"):
                self.i += 1
                return items
            else:
                raise self.err("expected ',' or ']'")

    def object(self):
        """Objects are lists of (key, value) pairs: duplicate keys survive parsing."""
        self.expect(ord("{"))
        items = _Obj()
        if self.peek() == ord("}"):
            self.i += 1
            return items
        while True:
            key = self.string()
            self.expect(ord(":"))
            items.append((key, self.value()))
            c = self.peek()
            if c == ord(","):
                self.i += 1
            elif c == ord("}"):
                self.i += 1
                return items
            else:
                raise self.err("expected ',' or '}'")


class _Obj(list):
    pass


@dataclass
class RawEntry:
    name: str
    dtype: str
    shape: list
    start: int
    end: int


@dataclass
class RawFile:
    entries: list
    metadata: dict
    data: bytes


def parse_raw(b: bytes) -> RawFile:
    if len(b) < 8:
        raise _bad("safetensors: shorter than the length prefix")
    header_len = struct.unpack("<Q", b[:8])[0]
    if header_len > 100_000_000 or 8 + header_len > len(b):
        raise _bad(f"safetensors: header length {header_len} exceeds the file")
    header = b[8:8 + header_len]
    data = b[8 + header_len:]
    obj = _Parser(header).object()
    entries, metadata = [], {}
    for name, val in obj:
        if name == "__metadata__":
            if not isinstance(val, _Obj):
                raise _bad("safetensors: __metadata__ must be an object")
            for k, v in val:
                if not isinstance(v, str):
                    raise _bad(f"safetensors: __metadata__[{k}] must be a string")
                metadata[k] = v
            continue
        if not isinstance(val, _Obj):
            raise _bad(f"safetensors: entry {name} must be an object")
        dtype = shape = offsets = None
        for k, v in val:
            if k == "dtype" and isinstance(v, str):
                dtype = v
            elif k == "shape" and isinstance(v, list) and not isinstance(v, _Obj):
                for d in v:
                    if not isinstance(d, int):
                        raise _bad(f"safetensors: {name}: non-integer dim")
                shape = list(v)
            elif k == "data_offsets" and isinstance(v, list) and not isinstance(v, _Obj):
                for d in v:
                    if not isinstance(d, int):
                        raise _bad(f"safetensors: {name}: non-integer offset")
                if len(v) != 2:
                    raise _bad(f"safetensors: {name}: offsets must be [s, e]")
                offsets = (v[0], v[1])
            else:
                raise _bad(f'safetensors: {name}: unknown key "{k}"')
        if dtype is None:
            raise _bad(f"safetensors: {name}: missing dtype")
        if shape is None:
            raise _bad(f"safetensors: {name}: missing shape")
        if offsets is None:
            raise _bad(f"safetensors: {name}: missing data_offsets")
        start, end = offsets
        if end < start or end > len(data):
            raise _bad(f"safetensors: {name}: offsets [{start}, {end}] exceed the data section")
        entries.append(RawEntry(name, dtype, shape, start, end))
    return RawFile(entries, metadata, data)


def _f16_to_f32(h: np.ndarray) -> np.ndarray:
    return h.view(np.float16).astype(np.float32)  # IEEE half -> f32 is exact for every class


def entry_to_f32(e: RawEntry, data: bytes) -> np.ndarray:
    count = max(int(np.prod(e.shape, dtype=np.uint64)) if len(e.shape) else 1, 1)
    raw = data[e.start:e.end]
    if e.dtype == "F32":
        if len(raw) != count * 4:
            raise _bad(f"safetensors: {e.name}: F32 needs {count * 4} bytes, offsets give {len(raw)}")
        return np.frombuffer(raw, dtype="<f4").copy()
    if e.dtype == "F16":
        if len(raw) != count * 2:
            raise _bad(f"safetensors: {e.name}: F16 needs {count * 2} bytes, offsets give {len(raw)}")
        return _f16_to_f32(np.frombuffer(raw, dtype="<u2").copy())
    if e.dtype == "BF16":
        if len(raw) != count * 2:
            raise _bad(f"safetensors: {e.name}: BF16 needs {count * 2} bytes, offsets give {len(raw)}")
        return (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << np.uint32(16)).view(np.float32)
    raise _bad(f"safetensors: {e.name}: dtype {e.dtype} not supported (F32/F16/BF16)")


# ---- metadata grammar (quant.rs:186-271) -------------------------------------

@dataclass
class QuantMeta:
    bits: int
    gr: int
    gc: int
    rows: int
    cols: int


def scheme_tag(bits: int) -> str:
    return "q8s" if bits == 8 else "q4s"


def write_quant_meta(bits, gr, gc, rows, cols) -> str:
    return f"{scheme_tag(bits)};gr={gr};gc={gc};rows={rows};cols={cols}"


def _parse_usize(v: str):
    # Rust usize::from_str: optional leading '+', ASCII digits only, no overflow.
    t = v[1:] if v.startswith("+") else v
    if t == "" or not all("0" <= ch <= "9" for ch in t):
        return None
    n = int(t)
    return n if n <= 0xFFFFFFFFFFFFFFFF else None


def parse_quant_meta(leaf: str, s: str) -> QuantMeta:
    parts = s.split(";")
    tag = parts[0]
    if tag == "q8s":
        bits = 8
    elif tag == "q4s":
        bits = 4
    else:
        raise _format_err(leaf, f"unknown scheme tag `{tag}` (this build reads q8s / q4s)")
    names = ["gr", "gc", "rows", "cols"]
    fields = [None] * 4
    for part in parts[1:]:
        if "=" not in part:
            raise _format_err(leaf, f"malformed metadata field `{part}` (want key=value)")
        k, v = part.split("=", 1)
        if k == "mode":
            raise _format_err(leaf, f"mode={v} is the reserved affine extension — this build reads v1 "
                                    "symmetric files only")
        if k not in names:
            raise _format_err(leaf, f"unknown metadata field `{k}`")
        idx = names.index(k)
        if fields[idx] is not None:
            raise _format_err(leaf, f"duplicate metadata field `{k}`")
        n = _parse_usize(v)
        if n is None:
            raise _format_err(leaf, f"field {k}={v} is not a positive integer")
        if n == 0:
            raise _format_err(leaf, f"field {k}=0 (must be positive)")
        fields[idx] = n
    for idx, name in enumerate(names):
        if fields[idx] is None:
            raise _format_err(leaf, f"missing metadata field `{name}`")
    return QuantMeta(bits, *fields)


def granularity_from_grid(rows, cols, gr, gc, allow_block=False):
    """Canonical spelling of a stored grid, None when no v1 writer produces it.

    Returns a tuple ('per_tensor',) / ('per_channel', axis) / ('group', axis, size)
    and, only with allow_block (the additive Block arm), ('block', gr, gc)."""
    if gr == 0 or gc == 0 or gr > rows or gc > cols:
        return None
    if gr == rows and gc == cols:
        return ("per_tensor",)
    if gr == 1 and gc == cols:
        return ("per_channel", 0)
    if gr == rows and gc == 1:
        return ("per_channel", 1)
    if gc == 1:
        return ("group", 0, gr)
    if gr == 1:
        return ("group", 1, gc)
    return ("block", gr, gc) if allow_block else None


# ---- leaves ------------------------------------------------------------------

@dataclass
class QLeaf:
    """A quantized leaf on the host: codes int8 [R,C] or uint32 [R,ceil(C/8)], scales f32 grid."""
    bits: int
    rows: int
    cols: int
    gr: int
    gc: int
    codes: np.ndarray
    scales: np.ndarray
    gran: tuple = field(default=None)


def save_named(entries, metadata=None) -> bytes:
    """entries: list of (name, leaf) with leaf an np.float32 ndarray or a QLeaf."""
    if metadata is not None:
        for k in metadata:
            if k == VERSION_KEY or k.startswith(META_PREFIX):
                raise _format_err(k, f"user metadata key `{k}` collides with the quantized-safetensors "
                                     f"convention (`{VERSION_KEY}` and `{META_PREFIX}*` are synthesized "
                                     "by the writer)")
    tensor_names, leaf_names = set(), set()
    for name, leaf in entries:
        if name in leaf_names:
            raise _format_err(name, "duplicate leaf name")
        leaf_names.add(name)
        slots = [f"{name}.q", f"{name}.qs"] if isinstance(leaf, QLeaf) else [name]
        for slot in slots:
            if slot in tensor_names:
                raise _format_err(name, f"tensor name `{slot}` collides with another leaf's")
            tensor_names.add(slot)
    meta = dict(metadata) if metadata is not None else {}
    raw = []
    any_q = False
    for name, leaf in entries:
        if isinstance(leaf, QLeaf):
            any_q = True
            meta[f"{META_PREFIX}{name}"] = write_quant_meta(leaf.bits, leaf.gr, leaf.gc, leaf.rows, leaf.cols)
            if leaf.bits == 8:
                raw.append((f"{name}.q", "I8", list(leaf.codes.shape), np.ascontiguousarray(leaf.codes, dtype=np.int8).tobytes()))
            else:
                raw.append((f"{name}.q", "U32", list(leaf.codes.shape), np.ascontiguousarray(leaf.codes, dtype="<u4").tobytes()))
            raw.append((f"{name}.qs", "F32", list(leaf.scales.shape), np.ascontiguousarray(leaf.scales, dtype="<f4").tobytes()))
        else:
            a = np.ascontiguousarray(leaf, dtype="<f4")
            raw.append((name, "F32", list(a.shape), a.tobytes()))
    if any_q:
        meta[VERSION_KEY] = FORMAT_VERSION
    meta_opt = None if (not meta and metadata is None) else meta
    return save_raw(raw, meta_opt)


@dataclass
class Validated:
    file: RawFile
    items: list  # ('plain', entry_index) | ('quant', name, QuantMeta, gran, q_index, scales)
    metadata: dict


def validate(b: bytes, allow_block: bool = False) -> Validated:
    f = parse_raw(b)
    quant_keys = sorted((k[len(META_PREFIX):] for k in f.metadata if k.startswith(META_PREFIX)),
                        key=lambda k: k.encode("utf-8"))
    v = f.metadata.get(VERSION_KEY)
    if v is not None and v != FORMAT_VERSION:
        raise _format_err(VERSION_KEY, f"format version {v} (this build reads {FORMAT_VERSION})")
    if quant_keys and VERSION_KEY not in f.metadata:
        raise _format_err(VERSION_KEY, "missing — a file with quant:* metadata must carry "
                                       f'{VERSION_KEY} = "{FORMAT_VERSION}"')
    by_name = {}
    for i, e in enumerate(f.entries):
        if e.name in by_name:
            raise _format_err(e.name, "duplicate tensor name")
        by_name[e.name] = i
    claimed, quantized = {}, []
    for leaf in quant_keys:
        if leaf == "":
            raise _format_err(META_PREFIX, "empty leaf name in quant:* metadata")
        meta = parse_quant_meta(leaf, f.metadata[f"{META_PREFIX}{leaf}"])
        if leaf in by_name:
            raise _format_err(leaf, f"both a tensor `{leaf}` and quant:{leaf} metadata are present (a "
                                    "quantized leaf stores NO tensor under its own name)")
        if f"{leaf}.qz" in by_name:
            raise _format_err(leaf, f"`{leaf}.qz` zero-points are the reserved affine extension — this "
                                    "build reads v1 symmetric files only")
        qn, sn = f"{leaf}.q", f"{leaf}.qs"
        if qn not in by_name:
            raise _format_err(leaf, f"quant:{leaf} present but tensor `{qn}` is missing")
        if sn not in by_name:
            raise _format_err(leaf, f"quant:{leaf} present but tensor `{sn}` is missing")
        qi, si = by_name[qn], by_name[sn]
        rows, cols, gr, gc = meta.rows, meta.cols, meta.gr, meta.gc
        gran = granularity_from_grid(rows, cols, gr, gc, allow_block)
        if gran is None:
            raise _format_err(leaf, f"grid (gr={gr}, gc={gc}) over [{rows}, {cols}] is not a v1 tile grid")
        qe = f.entries[qi]
        if meta.bits == 8:
            want_dtype, want_shape, want_bytes = "I8", [rows, cols], rows * cols
        else:
            wpr = -(-cols // 8)
            want_dtype, want_shape, want_bytes = "U32", [rows, wpr], rows * wpr * 4
        if qe.dtype != want_dtype:
            raise _format_err(leaf, f"`{qn}` has dtype {qe.dtype}, scheme {scheme_tag(meta.bits)} wants {want_dtype}")
        if qe.shape != want_shape:
            raise _format_err(leaf, f"`{qn}` has shape {_rust_list(qe.shape)}, metadata [rows={rows}, cols={cols}] wants "
                                    f"{_rust_list(want_shape)}")
        if qe.end - qe.start != want_bytes:
            raise _format_err(leaf, f"`{qn}` holds {qe.end - qe.start} data bytes, shape {_rust_list(want_shape)} wants {want_bytes}")
        se = f.entries[si]
        want_scales = [-(-rows // gr), -(-cols // gc)]
        if se.dtype != "F32":
            raise _format_err(leaf, f"`{sn}` has dtype {se.dtype}, scales are F32")
        if se.shape != want_scales:
            raise _format_err(leaf, f"`{sn}` has shape {_rust_list(se.shape)}, grid (gr={gr}, gc={gc}) wants {_rust_list(want_scales)}")
        scales = entry_to_f32(se, f.data)
        bad_tiles = np.nonzero(~np.isfinite(scales))[0]
        if bad_tiles.size:
            t = int(bad_tiles[0])
            raise StError("scale", f"leaf `{leaf}`: scale at tile {t} is {_rust_f32(scales[t])} (non-finite or zero) — "
                                   "the checkpoint is corrupt or hostile")
        claimed[qi] = ("codes", len(quantized))
        claimed[si] = ("scales",)
        quantized.append((leaf, meta, gran, qi, scales.reshape(want_scales)))
    items = []
    for i, e in enumerate(f.entries):
        c = claimed.get(i)
        if c is None:
            if e.dtype in ("I8", "U32"):
                raise _format_err(e.name, f"dtype {e.dtype} tensor carries no quant:<leaf> metadata — not a v1 "
                                          "quantized leaf, and not a plain F32/F16/BF16 tensor")
            items.append(("plain", i))
        elif c[0] == "codes":
            items.append(("quant",) + quantized[c[1]])
    metadata = {k: v for k, v in f.metadata.items() if k != VERSION_KEY and not k.startswith(META_PREFIX)}
    return Validated(f, items, metadata)


def _rust_f32(x) -> str:
    x = float(x)
    if x != x:
        return "NaN"
    if x == float("inf"):
        return "inf"
    if x == float("-inf"):
        return "-inf"
    return repr(x)


def load_named(b: bytes, allow_block: bool = False):
    """Mode B on the host: returns (leaves, metadata); leaves hold np.float32 arrays or QLeaf."""
    v = validate(b, allow_block)
    leaves = []
    for item in v.items:
        if item[0] == "plain":
            e = v.file.entries[item[1]]
            leaves.append((e.name, entry_to_f32(e, v.file.data).reshape(e.shape)))
        else:
            _, name, meta, gran, qi, scales = item
            qe = v.file.entries[qi]
            raw = v.file.data[qe.start:qe.end]
            if meta.bits == 8:
                codes = np.frombuffer(raw, dtype=np.int8).reshape(qe.shape).copy()
            else:
                codes = np.frombuffer(raw, dtype="<u4").reshape(qe.shape).copy()
            leaves.append((name, QLeaf(meta.bits, meta.rows, meta.cols, meta.gr, meta.gc, codes, scales, gran)))
    return leaves, v.metadata
