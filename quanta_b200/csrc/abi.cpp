// Library-level entry points and the grid vocabulary (host only).
#include <cstring>
#include <string>

#include "common.hpp"

namespace qb {

static thread_local std::string g_last_error;

qb200_status fail(qb200_status code, const std::string& msg) {
    g_last_error = msg;
    return code;
}
void clear_error() { g_last_error.clear(); }

std::string fmt_shape(const uint64_t* dims, size_t n) {
    std::string s = "[";
    for (size_t i = 0; i < n; i++) {
        if (i) s += ", ";
        s += std::to_string(dims[i]);
    }
    return s + "]";
}

}  // namespace qb

using qb::fail;

extern "C" {

const char* qb200_version(void) { return "0.1.0"; }

size_t qb200_last_error(char* buf, size_t cap) {
    const std::string& e = qb::g_last_error;
    if (buf && cap) {
        size_t n = e.size() < cap - 1 ? e.size() : cap - 1;
        std::memcpy(buf, e.data(), n);
        buf[n] = 0;
    }
    return e.size();
}

// Granularity::tile, quanta-array/src/quant.rs:109-144 (+ the Block arm).
qb200_status qb200_tile(int32_t kind, uint64_t axis, uint64_t size, uint64_t size2, uint64_t rows,
                        uint64_t cols, uint64_t* gr, uint64_t* gc) {
    if (!gr || !gc) return fail(QB200_ERR_INVALID_PARAM, "qb200_tile: null output pointer");
    const std::string pre = "invalid quantization granularity: ";
    switch (kind) {
        case QB200_PER_TENSOR:
            *gr = rows;
            *gc = cols;
            return QB200_OK;
        case QB200_PER_CHANNEL:
            if (axis == 0) {
                *gr = 1;
                *gc = cols;
                return QB200_OK;
            }
            if (axis == 1) {
                *gr = rows;
                *gc = 1;
                return QB200_OK;
            }
            return fail(QB200_ERR_GRANULARITY, pre + "PerChannel { axis: " + std::to_string(axis) +
                                                   " } — axis must be 0 (rows) or 1 (cols)");
        case QB200_GROUP: {
            const std::string sp =
                "Group { axis: " + std::to_string(axis) + ", size: " + std::to_string(size) + " }";
            if (axis > 1)
                return fail(QB200_ERR_GRANULARITY, pre + sp + " — axis must be 0 (rows) or 1 (cols)");
            uint64_t extent = axis == 0 ? rows : cols;
            if (size == 0 || size > extent)
                return fail(QB200_ERR_GRANULARITY, pre + sp + " — size must be in 1..=" +
                                                       std::to_string(extent) + " (the axis extent)");
            *gr = axis == 0 ? size : 1;
            *gc = axis == 0 ? 1 : size;
            return QB200_OK;
        }
        case QB200_BLOCK: {
            const std::string sp =
                "Block { rows: " + std::to_string(size) + ", cols: " + std::to_string(size2) + " }";
            if (size == 0 || size > rows || size2 == 0 || size2 > cols)
                return fail(QB200_ERR_GRANULARITY, pre + sp + " — block extents must be in 1..=[" +
                                                       std::to_string(rows) + ", " +
                                                       std::to_string(cols) + "] (the matrix extents)");
            *gr = size;
            *gc = size2;
            return QB200_OK;
        }
        default:
            return fail(QB200_ERR_GRANULARITY, pre + "unknown granularity kind " + std::to_string(kind));
    }
}

// granularity_from_grid, quanta-nn/src/quant.rs:119-145.
qb200_status qb200_granularity_from_grid(uint64_t rows, uint64_t cols, uint64_t gr, uint64_t gc,
                                         int32_t allow_block, int32_t* kind, uint64_t* axis,
                                         uint64_t* size, uint64_t* size2) {
    if (!kind || !axis || !size || !size2)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_granularity_from_grid: null output pointer");
    *axis = *size = *size2 = 0;
    auto none = [&]() {
        return fail(QB200_ERR_FORMAT, "grid (gr=" + std::to_string(gr) + ", gc=" + std::to_string(gc) +
                                          ") over [" + std::to_string(rows) + ", " +
                                          std::to_string(cols) + "] is not a v1 tile grid");
    };
    if (gr == 0 || gc == 0 || gr > rows || gc > cols) return none();
    if (gr == rows && gc == cols) {
        *kind = QB200_PER_TENSOR;
    } else if (gr == 1 && gc == cols) {
        *kind = QB200_PER_CHANNEL;
        *axis = 0;
    } else if (gr == rows && gc == 1) {
        *kind = QB200_PER_CHANNEL;
        *axis = 1;
    } else if (gc == 1) {
        *kind = QB200_GROUP;
        *axis = 0;
        *size = gr;
    } else if (gr == 1) {
        *kind = QB200_GROUP;
        *axis = 1;
        *size = gc;
    } else if (allow_block) {
        *kind = QB200_BLOCK;
        *size = gr;
        *size2 = gc;
    } else {
        return none();
    }
    return QB200_OK;
}

static qb200_status check_dims(uint64_t rows, uint64_t cols) {
    if (rows == 0 || cols == 0) {
        uint64_t d[2] = {rows, cols};
        return fail(QB200_ERR_RANK,
                    "quantized leaves must be rank-2 with nonzero extents, got shape " +
                        qb::fmt_shape(d, 2) + " (reshape rank-2 views before quantizing)");
    }
    return QB200_OK;
}

qb200_status qb200_codes_bytes(uint64_t rows, uint64_t cols, uint32_t bits, uint64_t* bytes) {
    if (!bytes) return fail(QB200_ERR_INVALID_PARAM, "qb200_codes_bytes: null output pointer");
    if (qb200_status s = check_dims(rows, cols)) return s;
    if (bits == 8)
        *bytes = rows * cols;
    else if (bits == 4)
        *bytes = rows * qb::div_ceil(cols, 8) * 4;
    else
        return fail(QB200_ERR_INVALID_PARAM, "code width must be 8 or 4 bits, got " + std::to_string(bits));
    return QB200_OK;
}

qb200_status qb200_scales_count(uint64_t rows, uint64_t cols, uint64_t gr, uint64_t gc,
                                uint64_t* tile_rows, uint64_t* tile_cols) {
    if (!tile_rows || !tile_cols)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_scales_count: null output pointer");
    if (qb200_status s = check_dims(rows, cols)) return s;
    if (gr == 0 || gc == 0 || gr > rows || gc > cols)
        return fail(QB200_ERR_GRANULARITY,
                    "invalid quantization granularity: tile (" + std::to_string(gr) + ", " +
                        std::to_string(gc) + ") must lie in 1..=[" + std::to_string(rows) + ", " +
                        std::to_string(cols) + "]");
    *tile_rows = qb::div_ceil(rows, gr);
    *tile_cols = qb::div_ceil(cols, gc);
    return QB200_OK;
}

// QuantizedMatrix::from_parts, quanta-array/src/quant.rs:521-568.
qb200_status qb200_check_parts(uint64_t codes_rows, uint64_t codes_cols, uint64_t scales_rows,
                               uint64_t scales_cols, uint64_t rows, uint64_t cols, uint32_t bits,
                               uint64_t gr, uint64_t gc) {
    if (qb200_status s = check_dims(rows, cols)) return s;
    if (bits != 8 && bits != 4)
        return fail(QB200_ERR_INVALID_PARAM, "code width must be 8 or 4 bits, got " + std::to_string(bits));
    uint64_t tr, tc;
    if (qb200_status s = qb200_scales_count(rows, cols, gr, gc, &tr, &tc)) return s;
    uint64_t want[2] = {rows, bits == 8 ? cols : qb::div_ceil(cols, 8)};
    uint64_t got[2] = {codes_rows, codes_cols};
    if (got[0] != want[0] || got[1] != want[1])
        return fail(QB200_ERR_GRID, "quantized matrix parts disagree: codes shape " +
                                        qb::fmt_shape(got, 2) + " does not match " +
                                        qb::fmt_shape(want, 2) + " for a [" + std::to_string(rows) +
                                        ", " + std::to_string(cols) + "] " +
                                        (bits == 8 ? "Int8" : "Int4") + " matrix");
    uint64_t sgot[2] = {scales_rows, scales_cols};
    if (scales_rows != tr || scales_cols != tc)
        return fail(QB200_ERR_GRID, "quantized matrix parts disagree: scales shape " +
                                        qb::fmt_shape(sgot, 2) + " does not match the [" +
                                        std::to_string(tr) + ", " + std::to_string(tc) +
                                        "] grid of tile (" + std::to_string(gr) + ", " +
                                        std::to_string(gc) + ") over a [" + std::to_string(rows) +
                                        ", " + std::to_string(cols) + "] matrix");
    return QB200_OK;
}

}  // extern "C"
