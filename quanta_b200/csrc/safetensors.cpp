// Quantized-safetensors: container scanner, total validation and the
// deterministic writer (host bytes only — no device work here).
//
// Format (crates/ml/quanta-nn/src/quant.rs:12-46 of the reference): a valid
// safetensors file — u64 LE header length, JSON header, data section — where a
// quantized leaf `x` is the pair `x.q` (I8 [R,C] or U32 [R,ceil(C/8)]) and
// `x.qs` (F32 scale grid) plus `__metadata__["quant:x"]`, and
// `__metadata__["quanta.quant"] = "1"` marks the format version.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.hpp"

using qb::fail;

namespace {

const char* kVersionKey = "quanta.quant";
const char* kMetaPrefix = "quant:";
const char* kFormatVersion = "1";

bool starts_with(const std::string& s, const char* p) { return s.rfind(p, 0) == 0; }

std::string format_msg(const std::string& leaf, const std::string& what) {
    return "quantized checkpoint leaf `" + leaf + "`: " + what;
}

// ---- header JSON ----------------------------------------------------------
// The header grammar is a strict subset of JSON: objects, arrays, strings and
// unsigned integers.  Objects keep their pairs in file order (duplicate keys
// survive so the validator can refuse them).

struct Json {
    enum Kind { STR, NUM, ARR, OBJ } kind = NUM;
    std::string str;
    uint64_t num = 0;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
};

struct Scanner {
    const uint8_t* p;
    size_t n;
    size_t at = 0;
    std::string error;

    bool bad(const std::string& what) {
        if (error.empty()) error = "safetensors header: " + what + " at byte " + std::to_string(at);
        return false;
    }
    void blanks() {
        while (at < n && (p[at] == ' ' || p[at] == '\t' || p[at] == '\n' || p[at] == '\r')) at++;
    }
    int look() {
        blanks();
        return at < n ? p[at] : -1;
    }
    bool take(char c) {
        blanks();
        if (at < n && p[at] == (uint8_t)c) {
            at++;
            return true;
        }
        return bad(std::string("expected '") + c + "'");
    }
    static void put_utf8(std::string& s, uint32_t cp) {
        if (cp < 0x80) {
            s += (char)cp;
        } else if (cp < 0x800) {
            s += (char)(0xC0 | (cp >> 6));
            s += (char)(0x80 | (cp & 0x3F));
        } else {
            s += (char)(0xE0 | (cp >> 12));
            s += (char)(0x80 | ((cp >> 6) & 0x3F));
            s += (char)(0x80 | (cp & 0x3F));
        }
    }
    static bool valid_utf8(const uint8_t* b, int len) {
        // Strict UTF-8: continuation bytes, no overlongs, no surrogates, <= U+10FFFF.
        for (int i = 1; i < len; i++)
            if ((b[i] & 0xC0) != 0x80) return false;
        uint32_t cp;
        if (len == 2) {
            cp = ((b[0] & 0x1Fu) << 6) | (b[1] & 0x3Fu);
            return cp >= 0x80;
        }
        if (len == 3) {
            cp = ((b[0] & 0x0Fu) << 12) | ((b[1] & 0x3Fu) << 6) | (b[2] & 0x3Fu);
            return cp >= 0x800 && !(cp >= 0xD800 && cp <= 0xDFFF);
        }
        cp = ((b[0] & 0x07u) << 18) | ((b[1] & 0x3Fu) << 12) | ((b[2] & 0x3Fu) << 6) | (b[3] & 0x3Fu);
        return cp >= 0x10000 && cp <= 0x10FFFF;
    }
    bool string(std::string& out) {
        if (!take('"')) return false;
        out.clear();
        for (;;) {
            if (at >= n) return bad("unterminated string");
            uint8_t c = p[at++];
            if (c == '"') return true;
            if (c == '\\') {
                if (at >= n) return bad("dangling escape");
                uint8_t e = p[at++];
                switch (e) {
                    case '"': out += '"'; break;
                    case '\\': out += '\\'; break;
                    case '/': out += '/'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'n': out += '\n'; break;
                    case 'r': out += '\r'; break;
                    case 't': out += '\t'; break;
                    case 'u': {
                        if (at + 4 > n) return bad("truncated \\u escape");
                        uint32_t cp = 0;
                        for (int i = 0; i < 4; i++) {
                            uint8_t h = p[at + i];
                            uint32_t d;
                            if (h >= '0' && h <= '9') d = h - '0';
                            else if (h >= 'a' && h <= 'f') d = h - 'a' + 10;
                            else if (h >= 'A' && h <= 'F') d = h - 'A' + 10;
                            else return bad("bad \\u escape");
                            cp = cp * 16 + d;
                        }
                        at += 4;
                        if (cp >= 0xD800 && cp <= 0xDFFF) return bad("surrogate in \\u escape");
                        put_utf8(out, cp);
                        break;
                    }
                    default: return bad("unknown escape");
                }
            } else if (c < 0x80) {
                out += (char)c;
            } else {
                size_t start = at - 1;
                int len = (c >= 0xC0 && c <= 0xDF) ? 2 : (c >= 0xE0 && c <= 0xEF) ? 3 : (c >= 0xF0 && c <= 0xF7) ? 4 : 0;
                if (!len) return bad("invalid utf-8");
                if (start + len > n) return bad("truncated utf-8");
                if (!valid_utf8(p + start, len)) return bad("invalid utf-8");
                out.append((const char*)p + start, len);
                at = start + len;
            }
        }
    }
    bool number(Json& v) {
        blanks();
        size_t start = at;
        uint64_t acc = 0;
        bool overflow = false;
        while (at < n && p[at] >= '0' && p[at] <= '9') {
            uint64_t d = p[at] - '0';
            if (acc > (UINT64_MAX - d) / 10) overflow = true;
            acc = acc * 10 + d;
            at++;
        }
        if (start == at) return bad("expected a number");
        if (overflow) return bad("integer out of range");
        v.kind = Json::NUM;
        v.num = acc;
        return true;
    }
    bool value(Json& v, int depth = 0) {
        if (depth > 64) return bad("nesting too deep");
        int c = look();
        if (c == '"') {
            v.kind = Json::STR;
            return string(v.str);
        }
        if (c == '{') return object(v, depth);
        if (c == '[') return array(v, depth);
        if (c >= '0' && c <= '9') return number(v);
        return bad("expected a value");
    }
    bool array(Json& v, int depth) {
        if (!take('[')) return false;
        v.kind = Json::ARR;
        if (look() == ']') {
            at++;
            return true;
        }
        for (;;) {
            v.arr.emplace_back();
            if (!value(v.arr.back(), depth + 1)) return false;
            int c = look();
            if (c == ',') {
                at++;
            } else if (c == ']') {
                at++;
                return true;
            } else {
                return bad("expected ',' or ']'");
            }
        }
    }
    bool object(Json& v, int depth = 0) {
        if (!take('{')) return false;
        v.kind = Json::OBJ;
        if (look() == '}') {
            at++;
            return true;
        }
        for (;;) {
            std::string key;
            if (!string(key)) return false;
            if (!take(':')) return false;
            v.obj.emplace_back(std::move(key), Json());
            if (!value(v.obj.back().second, depth + 1)) return false;
            int c = look();
            if (c == ',') {
                at++;
            } else if (c == '}') {
                at++;
                return true;
            } else {
                return bad("expected ',' or '}'");
            }
        }
    }
};

// ---- container ------------------------------------------------------------

struct Entry {
    std::string name, dtype;
    std::vector<uint64_t> shape;
    uint64_t start = 0, end = 0;  // offsets within the data section
};

struct Container {
    std::vector<Entry> entries;
    std::vector<std::pair<std::string, std::string>> metadata;  // file order; later keys win
    uint64_t data_base = 0;                                     // offset of the data section
    uint64_t data_len = 0;
};

qb200_status parse_container(const uint8_t* b, uint64_t len, Container& out) {
    if (!b || len < 8) return fail(QB200_ERR_INVALID_PARAM, "safetensors: shorter than the length prefix");
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | b[i];
    if (hlen > 100000000ull || hlen > len - 8)
        return fail(QB200_ERR_INVALID_PARAM,
                    "safetensors: header length " + std::to_string(hlen) + " exceeds the file");
    out.data_base = 8 + hlen;
    out.data_len = len - out.data_base;
    Scanner sc{b + 8, (size_t)hlen};
    Json root;
    if (!sc.object(root)) return fail(QB200_ERR_INVALID_PARAM, sc.error);
    for (auto& kv : root.obj) {
        const std::string& name = kv.first;
        Json& val = kv.second;
        if (name == "__metadata__") {
            if (val.kind != Json::OBJ)
                return fail(QB200_ERR_INVALID_PARAM, "safetensors: __metadata__ must be an object");
            for (auto& m : val.obj) {
                if (m.second.kind != Json::STR)
                    return fail(QB200_ERR_INVALID_PARAM,
                                "safetensors: __metadata__[" + m.first + "] must be a string");
                out.metadata.emplace_back(m.first, m.second.str);
            }
            continue;
        }
        if (val.kind != Json::OBJ)
            return fail(QB200_ERR_INVALID_PARAM, "safetensors: entry " + name + " must be an object");
        Entry e;
        e.name = name;
        bool has_dtype = false, has_shape = false, has_off = false;
        for (auto& f : val.obj) {
            if (f.first == "dtype" && f.second.kind == Json::STR) {
                e.dtype = f.second.str;
                has_dtype = true;
            } else if (f.first == "shape" && f.second.kind == Json::ARR) {
                e.shape.clear();
                for (auto& d : f.second.arr) {
                    if (d.kind != Json::NUM)
                        return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": non-integer dim");
                    e.shape.push_back(d.num);
                }
                has_shape = true;
            } else if (f.first == "data_offsets" && f.second.kind == Json::ARR) {
                for (auto& d : f.second.arr)
                    if (d.kind != Json::NUM)
                        return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": non-integer offset");
                if (f.second.arr.size() != 2)
                    return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": offsets must be [s, e]");
                e.start = f.second.arr[0].num;
                e.end = f.second.arr[1].num;
                has_off = true;
            } else {
                return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": unknown key \"" + f.first + "\"");
            }
        }
        if (!has_dtype) return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": missing dtype");
        if (!has_shape) return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": missing shape");
        if (!has_off) return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": missing data_offsets");
        if (e.end < e.start || e.end > out.data_len)
            return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + name + ": offsets [" + std::to_string(e.start) +
                                                     ", " + std::to_string(e.end) + "] exceed the data section");
        out.entries.push_back(std::move(e));
    }
    return QB200_OK;
}

// ---- the quant:<leaf> grammar ----------------------------------------------

struct QuantMeta {
    uint32_t bits = 0;
    uint64_t gr = 0, gc = 0, rows = 0, cols = 0;
};

const char* scheme_tag(uint32_t bits) { return bits == 8 ? "q8s" : "q4s"; }

// Unsigned decimal, optional leading '+', digits only, no overflow.
bool parse_uint(const std::string& v, uint64_t& out) {
    size_t i = (!v.empty() && v[0] == '+') ? 1 : 0;
    if (i >= v.size()) return false;
    uint64_t acc = 0;
    for (; i < v.size(); i++) {
        if (v[i] < '0' || v[i] > '9') return false;
        uint64_t d = v[i] - '0';
        if (acc > (UINT64_MAX - d) / 10) return false;
        acc = acc * 10 + d;
    }
    out = acc;
    return true;
}

qb200_status parse_meta(const std::string& leaf, const std::string& s, QuantMeta& m) {
    std::vector<std::string> parts;
    size_t pos = 0;
    for (;;) {
        size_t semi = s.find(';', pos);
        parts.push_back(s.substr(pos, semi == std::string::npos ? std::string::npos : semi - pos));
        if (semi == std::string::npos) break;
        pos = semi + 1;
    }
    const std::string& tag = parts[0];
    if (tag == "q8s") m.bits = 8;
    else if (tag == "q4s") m.bits = 4;
    else
        return fail(QB200_ERR_FORMAT,
                    format_msg(leaf, "unknown scheme tag `" + tag + "` (this build reads q8s / q4s)"));
    static const char* names[4] = {"gr", "gc", "rows", "cols"};
    uint64_t vals[4] = {0, 0, 0, 0};
    bool seen[4] = {false, false, false, false};
    for (size_t i = 1; i < parts.size(); i++) {
        const std::string& part = parts[i];
        size_t eq = part.find('=');
        if (eq == std::string::npos)
            return fail(QB200_ERR_FORMAT, format_msg(leaf, "malformed metadata field `" + part + "` (want key=value)"));
        std::string k = part.substr(0, eq), v = part.substr(eq + 1);
        if (k == "mode")
            return fail(QB200_ERR_FORMAT,
                        format_msg(leaf, "mode=" + v + " is the reserved affine extension — this build reads v1 "
                                                        "symmetric files only"));
        int idx = -1;
        for (int j = 0; j < 4; j++)
            if (k == names[j]) idx = j;
        if (idx < 0) return fail(QB200_ERR_FORMAT, format_msg(leaf, "unknown metadata field `" + k + "`"));
        if (seen[idx]) return fail(QB200_ERR_FORMAT, format_msg(leaf, "duplicate metadata field `" + k + "`"));
        uint64_t nval;
        if (!parse_uint(v, nval))
            return fail(QB200_ERR_FORMAT, format_msg(leaf, "field " + k + "=" + v + " is not a positive integer"));
        if (nval == 0) return fail(QB200_ERR_FORMAT, format_msg(leaf, "field " + k + "=0 (must be positive)"));
        seen[idx] = true;
        vals[idx] = nval;
    }
    for (int j = 0; j < 4; j++)
        if (!seen[j])
            return fail(QB200_ERR_FORMAT, format_msg(leaf, std::string("missing metadata field `") + names[j] + "`"));
    m.gr = vals[0];
    m.gc = vals[1];
    m.rows = vals[2];
    m.cols = vals[3];
    return QB200_OK;
}

std::string f32_text(float v) {
    if (std::isnan(v)) return "NaN";
    if (std::isinf(v)) return v > 0 ? "inf" : "-inf";
    return std::to_string(v);
}

// ---- validated file ---------------------------------------------------------

struct Item {
    std::string name;
    bool quantized = false;
    std::string dtype;
    std::vector<uint64_t> shape;
    uint64_t data_offset = 0, data_len = 0;
    QuantMeta meta;
    uint64_t scales_offset = 0, scales_len = 0;
    int32_t gran_kind = 0;
    uint64_t gran_axis = 0, gran_size = 0, gran_size2 = 0;
};

}  // namespace

struct qb200_st_file {
    const uint8_t* bytes = nullptr;
    uint64_t len = 0;
    std::vector<Item> items;
    std::vector<std::pair<std::string, std::string>> metadata;
};

namespace {

bool mul_overflow(uint64_t a, uint64_t b, uint64_t& out) { return __builtin_mul_overflow(a, b, &out); }

qb200_status validate(const uint8_t* b, uint64_t len, bool allow_block, qb200_st_file& out) {
    Container c;
    if (qb200_status s = parse_container(b, len, c)) return s;

    // Later duplicate metadata keys win (a map insert overwrites).
    std::map<std::string, std::string> meta;
    for (auto& kv : c.metadata) meta[kv.first] = kv.second;

    // The version gate comes before any structural interpretation.
    std::vector<std::string> leaves;  // sorted by the map's byte order
    for (auto& kv : meta)
        if (starts_with(kv.first, kMetaPrefix)) leaves.push_back(kv.first.substr(std::strlen(kMetaPrefix)));
    auto ver = meta.find(kVersionKey);
    if (ver != meta.end() && ver->second != kFormatVersion)
        return fail(QB200_ERR_FORMAT, format_msg(kVersionKey, "format version " + ver->second +
                                                                  " (this build reads " + kFormatVersion + ")"));
    if (!leaves.empty() && ver == meta.end())
        return fail(QB200_ERR_FORMAT,
                    format_msg(kVersionKey, std::string("missing — a file with quant:* metadata must carry ") +
                                                kVersionKey + " = \"" + kFormatVersion + "\""));

    std::unordered_map<std::string, size_t> by_name;
    for (size_t i = 0; i < c.entries.size(); i++)
        if (!by_name.emplace(c.entries[i].name, i).second)
            return fail(QB200_ERR_FORMAT, format_msg(c.entries[i].name, "duplicate tensor name"));

    // role[i]: -1 unclaimed, -2 a scales tensor, >= 0 index into `quant`
    std::vector<long> role(c.entries.size(), -1);
    std::vector<Item> quant;
    for (const std::string& leaf : leaves) {
        if (leaf.empty()) return fail(QB200_ERR_FORMAT, format_msg(kMetaPrefix, "empty leaf name in quant:* metadata"));
        QuantMeta m;
        if (qb200_status s = parse_meta(leaf, meta[std::string(kMetaPrefix) + leaf], m)) return s;
        if (by_name.count(leaf))
            return fail(QB200_ERR_FORMAT,
                        format_msg(leaf, "both a tensor `" + leaf + "` and quant:" + leaf +
                                             " metadata are present (a quantized leaf stores NO tensor under its own name)"));
        if (by_name.count(leaf + ".qz"))
            return fail(QB200_ERR_FORMAT,
                        format_msg(leaf, "`" + leaf + ".qz` zero-points are the reserved affine extension — this "
                                                      "build reads v1 symmetric files only"));
        const std::string qn = leaf + ".q", sn = leaf + ".qs";
        auto qi = by_name.find(qn), si = by_name.find(sn);
        if (qi == by_name.end())
            return fail(QB200_ERR_FORMAT, format_msg(leaf, "quant:" + leaf + " present but tensor `" + qn + "` is missing"));
        if (si == by_name.end())
            return fail(QB200_ERR_FORMAT, format_msg(leaf, "quant:" + leaf + " present but tensor `" + sn + "` is missing"));

        Item it;
        it.name = leaf;
        it.quantized = true;
        it.meta = m;
        {
            qb200_status s = qb200_granularity_from_grid(m.rows, m.cols, m.gr, m.gc, allow_block ? 1 : 0,
                                                         &it.gran_kind, &it.gran_axis, &it.gran_size, &it.gran_size2);
            if (s) {
                char buf[256];
                qb200_last_error(buf, sizeof buf);
                return fail(QB200_ERR_FORMAT, format_msg(leaf, buf));
            }
        }
        const Entry& qe = c.entries[qi->second];
        const uint64_t wpr = qb::div_ceil(m.cols, 8);
        const char* want_dtype = m.bits == 8 ? "I8" : "U32";
        std::vector<uint64_t> want_shape = {m.rows, m.bits == 8 ? m.cols : wpr};
        uint64_t want_bytes = 0;
        bool ovf = mul_overflow(want_shape[0], want_shape[1], want_bytes);
        if (m.bits == 4) ovf = ovf || mul_overflow(want_bytes, 4, want_bytes);
        if (qe.dtype != want_dtype)
            return fail(QB200_ERR_FORMAT, format_msg(leaf, "`" + qn + "` has dtype " + qe.dtype + ", scheme " +
                                                               scheme_tag(m.bits) + " wants " + want_dtype));
        if (qe.shape != want_shape)
            return fail(QB200_ERR_FORMAT,
                        format_msg(leaf, "`" + qn + "` has shape " + qb::fmt_shape(qe.shape.data(), qe.shape.size()) +
                                             ", metadata [rows=" + std::to_string(m.rows) + ", cols=" +
                                             std::to_string(m.cols) + "] wants " + qb::fmt_shape(want_shape.data(), 2)));
        if (ovf || qe.end - qe.start != want_bytes)
            return fail(QB200_ERR_FORMAT,
                        format_msg(leaf, "`" + qn + "` holds " + std::to_string(qe.end - qe.start) + " data bytes, shape " +
                                             qb::fmt_shape(want_shape.data(), 2) + " wants " + std::to_string(want_bytes)));

        const Entry& se = c.entries[si->second];
        std::vector<uint64_t> want_scales = {qb::div_ceil(m.rows, m.gr), qb::div_ceil(m.cols, m.gc)};
        if (se.dtype != "F32")
            return fail(QB200_ERR_FORMAT, format_msg(leaf, "`" + sn + "` has dtype " + se.dtype + ", scales are F32"));
        if (se.shape != want_scales)
            return fail(QB200_ERR_FORMAT,
                        format_msg(leaf, "`" + sn + "` has shape " + qb::fmt_shape(se.shape.data(), se.shape.size()) +
                                             ", grid (gr=" + std::to_string(m.gr) + ", gc=" + std::to_string(m.gc) +
                                             ") wants " + qb::fmt_shape(want_scales.data(), 2)));
        uint64_t ns = 0, sb = 0;
        if (mul_overflow(want_scales[0], want_scales[1], ns) || mul_overflow(ns, 4, sb) || se.end - se.start != sb)
            return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + sn + ": F32 needs " + std::to_string(ns * 4) +
                                                     " bytes, offsets give " + std::to_string(se.end - se.start));
        // Zero is legal (an all-zero tile stores s = 0); non-finite is a corrupt file.
        const uint8_t* sp = b + c.data_base + se.start;
        for (uint64_t t = 0; t < ns; t++) {
            float v;
            std::memcpy(&v, sp + 4 * t, 4);
            if (!std::isfinite(v))
                return fail(QB200_ERR_SCALE, "leaf `" + leaf + "`: scale at tile " + std::to_string(t) + " is " +
                                                 f32_text(v) + " (non-finite or zero) — the checkpoint is corrupt or hostile");
        }
        it.dtype = want_dtype;
        it.shape = {m.rows, m.cols};
        it.data_offset = c.data_base + qe.start;
        it.data_len = qe.end - qe.start;
        it.scales_offset = c.data_base + se.start;
        it.scales_len = sb;
        role[qi->second] = (long)quant.size();
        role[si->second] = -2;
        quant.push_back(std::move(it));
    }

    // Items in header order; a quantized leaf sits where its `.q` tensor does.
    for (size_t i = 0; i < c.entries.size(); i++) {
        const Entry& e = c.entries[i];
        if (role[i] == -2) continue;
        if (role[i] >= 0) {
            out.items.push_back(quant[(size_t)role[i]]);
            continue;
        }
        if (e.dtype == "I8" || e.dtype == "U32")
            return fail(QB200_ERR_FORMAT,
                        format_msg(e.name, "dtype " + e.dtype + " tensor carries no quant:<leaf> metadata — not a v1 "
                                                                 "quantized leaf, and not a plain F32/F16/BF16 tensor"));
        Item it;
        it.name = e.name;
        it.dtype = e.dtype;
        it.shape = e.shape;
        it.data_offset = c.data_base + e.start;
        it.data_len = e.end - e.start;
        out.items.push_back(std::move(it));
    }
    for (auto& kv : meta)
        if (kv.first != kVersionKey && !starts_with(kv.first, kMetaPrefix)) out.metadata.emplace_back(kv.first, kv.second);
    out.bytes = b;
    out.len = len;
    return QB200_OK;
}

float half_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1F, m = h & 0x3FF, bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {  // subnormal half = m * 2^-24: renormalise
            int top = 31 - __builtin_clz(m);
            bits = sign | ((uint32_t)(127 + top - 24) << 23) | ((m << (23 - top)) & 0x7FFFFF);
        }
    } else if (e == 0x1F) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((e + 112) << 23) | (m << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

void json_quote(const std::string& s, std::string& out) {
    out += '"';
    for (unsigned char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    std::snprintf(buf, sizeof buf, "\\u%04x", c);
                    out += buf;
                } else {
                    out += (char)c;
                }
        }
    }
    out += '"';
}

struct WEntry {
    std::string name, dtype;
    std::vector<uint64_t> shape;
    std::vector<uint8_t> bytes;
};

}  // namespace

struct qb200_st_writer {
    bool has_metadata = false;
    std::map<std::string, std::string> metadata;
    std::vector<WEntry> entries;
    std::set<std::string> leaf_names, tensor_names;
    bool any_quantized = false;
    std::vector<uint8_t> out;
};

extern "C" {

qb200_status qb200_st_validate(const uint8_t* bytes, uint64_t len, int32_t allow_block, qb200_st_file** out) {
    if (!out) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_validate: null output pointer");
    *out = nullptr;
    auto f = std::make_unique<qb200_st_file>();
    if (qb200_status s = validate(bytes, len, allow_block != 0, *f)) return s;
    *out = f.release();
    return QB200_OK;
}

void qb200_st_free(qb200_st_file* f) { delete f; }

uint64_t qb200_st_num_items(const qb200_st_file* f) { return f ? f->items.size() : 0; }

qb200_status qb200_st_item_at(const qb200_st_file* f, uint64_t i, qb200_st_item* out) {
    if (!f || !out || i >= f->items.size()) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_item_at: index out of range");
    const Item& it = f->items[i];
    out->name = it.name.c_str();
    out->quantized = it.quantized ? 1 : 0;
    out->dtype = it.dtype.c_str();
    out->ndim = (uint32_t)it.shape.size();
    out->shape = it.shape.data();
    out->data_offset = it.data_offset;
    out->data_len = it.data_len;
    out->bits = it.meta.bits;
    out->gr = it.meta.gr;
    out->gc = it.meta.gc;
    out->scales_offset = it.scales_offset;
    out->scales_len = it.scales_len;
    out->gran_kind = it.gran_kind;
    out->gran_axis = it.gran_axis;
    out->gran_size = it.gran_size;
    out->gran_size2 = it.gran_size2;
    return QB200_OK;
}

uint64_t qb200_st_num_metadata(const qb200_st_file* f) { return f ? f->metadata.size() : 0; }

qb200_status qb200_st_metadata_at(const qb200_st_file* f, uint64_t i, const char** key, const char** value) {
    if (!f || !key || !value || i >= f->metadata.size())
        return fail(QB200_ERR_INVALID_PARAM, "qb200_st_metadata_at: index out of range");
    *key = f->metadata[i].first.c_str();
    *value = f->metadata[i].second.c_str();
    return QB200_OK;
}

qb200_status qb200_st_plain_to_f32(const qb200_st_file* f, uint64_t i, float* out, uint64_t count) {
    if (!f || i >= f->items.size() || f->items[i].quantized)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_st_plain_to_f32: not a plain tensor");
    const Item& it = f->items[i];
    uint64_t n = 1;
    for (uint64_t d : it.shape)
        if (mul_overflow(n, d, n)) return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + it.name + ": shape overflows");
    if (n < 1) n = 1;  // a zero extent still counts one element, as the reference's product().max(1)
    const uint8_t* p = f->bytes + it.data_offset;
    auto need = [&](const char* dt, uint64_t width) {
        return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + it.name + ": " + dt + " needs " + std::to_string(n * width) +
                                                 " bytes, offsets give " + std::to_string(it.data_len));
    };
    if (it.dtype == "F32") {
        if (it.data_len != n * 4) return need("F32", 4);
    } else if (it.dtype == "F16" || it.dtype == "BF16") {
        if (it.data_len != n * 2) return need(it.dtype.c_str(), 2);
    } else {
        return fail(QB200_ERR_INVALID_PARAM, "safetensors: " + it.name + ": dtype " + it.dtype + " not supported (F32/F16/BF16)");
    }
    if (!out || count != n)
        return fail(QB200_ERR_LENGTH, "length mismatch: expected " + std::to_string(n) + ", got " + std::to_string(count));
    if (it.dtype == "F32") {
        std::memcpy(out, p, n * 4);
    } else if (it.dtype == "F16") {
        for (uint64_t k = 0; k < n; k++) out[k] = half_to_f32((uint16_t)(p[2 * k] | (p[2 * k + 1] << 8)));
    } else {
        for (uint64_t k = 0; k < n; k++) {
            uint32_t bits = (uint32_t)(p[2 * k] | (p[2 * k + 1] << 8)) << 16;
            std::memcpy(&out[k], &bits, 4);
        }
    }
    return QB200_OK;
}

qb200_status qb200_st_writer_create(qb200_st_writer** out) {
    if (!out) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_writer_create: null output pointer");
    *out = new qb200_st_writer();
    return QB200_OK;
}

void qb200_st_writer_free(qb200_st_writer* w) { delete w; }

qb200_status qb200_st_writer_set_has_metadata(qb200_st_writer* w, int32_t has) {
    if (!w) return fail(QB200_ERR_INVALID_PARAM, "null writer");
    w->has_metadata = has != 0;
    return QB200_OK;
}

qb200_status qb200_st_writer_add_metadata(qb200_st_writer* w, const char* key, const char* value) {
    if (!w || !key || !value) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_writer_add_metadata: null argument");
    std::string k = key;
    if (k == kVersionKey || starts_with(k, kMetaPrefix))
        return fail(QB200_ERR_FORMAT,
                    format_msg(k, "user metadata key `" + k + "` collides with the quantized-safetensors convention (`" +
                                      kVersionKey + "` and `" + kMetaPrefix + "*` are synthesized by the writer)"));
    w->has_metadata = true;
    w->metadata[k] = value;
    return QB200_OK;
}

static qb200_status claim(qb200_st_writer* w, const std::string& leaf, std::initializer_list<std::string> slots) {
    if (!w->leaf_names.insert(leaf).second) return fail(QB200_ERR_FORMAT, format_msg(leaf, "duplicate leaf name"));
    for (const std::string& s : slots)
        if (!w->tensor_names.insert(s).second)
            return fail(QB200_ERR_FORMAT, format_msg(leaf, "tensor name `" + s + "` collides with another leaf's"));
    return QB200_OK;
}

qb200_status qb200_st_writer_add_f32(qb200_st_writer* w, const char* name, const uint64_t* shape, uint32_t ndim,
                                     const float* data) {
    if (!w || !name || (ndim && !shape)) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_writer_add_f32: null argument");
    if (qb200_status s = claim(w, name, {name})) return s;
    WEntry e;
    e.name = name;
    e.dtype = "F32";
    uint64_t n = 1;
    for (uint32_t i = 0; i < ndim; i++) {
        e.shape.push_back(shape[i]);
        n *= shape[i];
    }
    if (n && !data) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_writer_add_f32: null data");
    e.bytes.resize(n * 4);
    if (n) std::memcpy(e.bytes.data(), data, n * 4);  // little-endian host
    w->entries.push_back(std::move(e));
    return QB200_OK;
}

qb200_status qb200_st_writer_add_quantized(qb200_st_writer* w, const char* name, uint32_t bits, uint64_t rows,
                                           uint64_t cols, uint64_t gr, uint64_t gc, const void* codes,
                                           const float* scales) {
    if (!w || !name || !codes || !scales) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_writer_add_quantized: null argument");
    uint64_t cbytes, tr, tc;
    if (qb200_status s = qb200_codes_bytes(rows, cols, bits, &cbytes)) return s;
    if (qb200_status s = qb200_scales_count(rows, cols, gr, gc, &tr, &tc)) return s;
    std::string leaf = name;
    if (qb200_status s = claim(w, leaf, {leaf + ".q", leaf + ".qs"})) return s;
    w->any_quantized = true;
    w->metadata[std::string(kMetaPrefix) + leaf] = std::string(scheme_tag(bits)) + ";gr=" + std::to_string(gr) +
                                                   ";gc=" + std::to_string(gc) + ";rows=" + std::to_string(rows) +
                                                   ";cols=" + std::to_string(cols);
    WEntry q;
    q.name = leaf + ".q";
    q.dtype = bits == 8 ? "I8" : "U32";
    q.shape = {rows, bits == 8 ? cols : qb::div_ceil(cols, 8)};
    q.bytes.assign((const uint8_t*)codes, (const uint8_t*)codes + cbytes);
    w->entries.push_back(std::move(q));
    WEntry s;
    s.name = leaf + ".qs";
    s.dtype = "F32";
    s.shape = {tr, tc};
    s.bytes.assign((const uint8_t*)scales, (const uint8_t*)scales + tr * tc * 4);
    w->entries.push_back(std::move(s));
    return QB200_OK;
}

qb200_status qb200_st_writer_finish(qb200_st_writer* w, const uint8_t** bytes, uint64_t* len) {
    if (!w || !bytes || !len) return fail(QB200_ERR_INVALID_PARAM, "qb200_st_writer_finish: null argument");
    if (w->any_quantized) w->metadata[kVersionKey] = kFormatVersion;
    std::string header = "{";
    bool first = true;
    if (!w->metadata.empty() || w->has_metadata) {
        header += "\"__metadata__\":{";
        bool f2 = true;
        for (auto& kv : w->metadata) {  // std::map: keys in byte order
            if (!f2) header += ',';
            f2 = false;
            json_quote(kv.first, header);
            header += ':';
            json_quote(kv.second, header);
        }
        header += '}';
        first = false;
    }
    uint64_t off = 0;
    for (const WEntry& e : w->entries) {
        if (!first) header += ',';
        first = false;
        json_quote(e.name, header);
        header += ":{\"dtype\":\"" + e.dtype + "\",\"shape\":[";
        for (size_t i = 0; i < e.shape.size(); i++) {
            if (i) header += ',';
            header += std::to_string(e.shape[i]);
        }
        header += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + e.bytes.size()) + "]}";
        off += e.bytes.size();
    }
    header += '}';
    while ((header.size() + 8) % 8 != 0) header += ' ';
    w->out.clear();
    w->out.reserve(8 + header.size() + off);
    uint64_t hl = header.size();
    for (int i = 0; i < 8; i++) w->out.push_back((uint8_t)(hl >> (8 * i)));
    w->out.insert(w->out.end(), header.begin(), header.end());
    for (const WEntry& e : w->entries) w->out.insert(w->out.end(), e.bytes.begin(), e.bytes.end());
    *bytes = w->out.data();
    *len = w->out.size();
    return QB200_OK;
}

qb200_status qb200_st_parse_quant_meta(const char* leaf, const char* value, uint32_t* bits, uint64_t* gr,
                                       uint64_t* gc, uint64_t* rows, uint64_t* cols) {
    if (!leaf || !value || !bits || !gr || !gc || !rows || !cols)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_st_parse_quant_meta: null argument");
    QuantMeta m;
    if (qb200_status s = parse_meta(leaf, value, m)) return s;
    *bits = m.bits;
    *gr = m.gr;
    *gc = m.gc;
    *rows = m.rows;
    *cols = m.cols;
    return QB200_OK;
}

}  // extern "C"
