// Quantize-on-load and dequantize: the two bandwidth kernels of the path.
//
// quantize  : per-tile max-abs -> s = m / hi -> clamp(rte(w / s)) -> pack
//             (reference: crates/sci/quanta-array/src/quant.rs:293-367, a
//             single-threaded host loop over a device read-back).
// dequantize: out[r, c] = s * f32(q)
//             (reference: crates/sci/quanta-array/src/quant.rs:373-413, 639-752).
//
// Data layout in HBM: W `[rows, cols]` row-major (f32 / bf16 / f16); codes int8
// `[rows, cols]` or packed int4 `[rows, ceil(cols/8)]` u32 words; scales f32
// `[ceil(rows/gr), ceil(cols/gc)]`.
//
// The tile kernel reads every weight exactly once: a sub-warp group of G lanes
// owns one tile, keeps its 8-element chunks in registers, reduces the max with
// shuffles and writes codes as whole words.  Tiles that do not fit the register
// budget, or matrices whose rows are not 8-element aligned, take the three-pass
// generic path (bit-pattern atomicMax into the scale grid, finalize, encode).
#include <cstdint>
#include <cstdlib>
#include <string>

#include "common.hpp"
#include "quant_math.cuh"

namespace qb {

enum SrcType { SRC_F32 = 0, SRC_BF16 = 1, SRC_F16 = 2 };

// ---- 8-element chunk loads --------------------------------------------------

// KEEP: the caller reads the chunk again soon, so it is loaded with the default policy instead of as a stream.
template <int SRC, bool KEEP = false>
__device__ __forceinline__ void load_chunk8(const void* base, uint64_t elem, float (&v)[8]) {
    if constexpr (SRC == SRC_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem);
        float4 a = KEEP ? __ldg(p) : __ldcs(p), b = KEEP ? __ldg(p + 1) : __ldcs(p + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem);
        uint4 a = KEEP ? __ldg(p) : __ldcs(p);
        uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if constexpr (SRC == SRC_BF16) {
                v[2 * i] = bf16_bits_to_f32(w[i] & 0xFFFFu);
                v[2 * i + 1] = bf16_bits_to_f32(w[i] >> 16);
            } else {
                v[2 * i] = half_bits_to_f32((uint16_t)(w[i] & 0xFFFFu));
                v[2 * i + 1] = half_bits_to_f32((uint16_t)(w[i] >> 16));
            }
        }
    }
}

template <int SRC>
__device__ __forceinline__ float load_elem(const void* base, uint64_t i) {
    if constexpr (SRC == SRC_F32) return static_cast<const float*>(base)[i];
    uint16_t h = static_cast<const uint16_t*>(base)[i];
    if constexpr (SRC == SRC_BF16) return bf16_bits_to_f32(h);
    return half_bits_to_f32(h);
}

// ---- the single-pass tile kernel ------------------------------------------

struct TileGeom {
    uint64_t rows, cols;      // matrix
    uint32_t gr, gc;          // tile
    uint64_t tr, tc;          // scale grid
    uint32_t chunks_per_row;  // gc / 8
    uint32_t chunks;          // gr * gc / 8 chunks per tile
    uint32_t lanes;           // G: lanes per tile (power of two <= 32)
    uint32_t lane_shift;      // log2(lanes)
};

// CPL: chunks per lane (ceil(chunks / lanes)).  One group of `lanes` lanes quantizes one tile;
// a warp holds 32 / lanes groups.  A group walks tiles with a grid stride and keeps the next
// tile's chunks in flight while it works on the current one (PF).  All index arithmetic is
// 32-bit and incremental: with 64-bit divisions per thread the kernel was bound by its own
// address computation, not by memory.
template <int SRC, int BITS, int CPL, bool PF>
__global__ void __launch_bounds__(256) k_quantize_tiles(const void* __restrict__ w, TileGeom g,
                                                        void* __restrict__ codes,
                                                        float* __restrict__ scales) {
    constexpr int HI = BITS == 8 ? 127 : 7;
    constexpr int LO = -HI - 1;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t sub = lane & (g.lanes - 1u);
    const uint32_t groups_per_block = blockDim.x >> g.lane_shift;
    // the launcher keeps tiles below 2^31 and rows, cols below 2^32
    const uint32_t tiles = (uint32_t)(g.tr * g.tc), tc = (uint32_t)g.tc, rows = (uint32_t)g.rows, cols = (uint32_t)g.cols;
    const uint32_t stride = gridDim.x * groups_per_block;
    uint32_t tile = blockIdx.x * groups_per_block + (threadIdx.x >> g.lane_shift);
    // this lane's chunks inside a tile: the same for every tile
    uint32_t rr[CPL], cc[CPL];
    bool chunk_ok[CPL];
#pragma unroll
    for (int i = 0; i < CPL; i++) {
        const uint32_t ch = sub + (uint32_t)i * g.lanes;
        rr[i] = ch / g.chunks_per_row;
        cc[i] = (ch - rr[i] * g.chunks_per_row) * 8u;
        chunk_ok[i] = ch < g.chunks;
    }
    // tile coordinates advance by (stride / tc, stride % tc) with a carry
    uint32_t t_r = tile / tc, t_c = tile - t_r * tc;
    const uint32_t step_r = stride / tc, step_c = stride - step_r * tc;

    struct Buf {
        float v[CPL][8];
        bool ok[CPL];
        uint64_t pos[CPL];
    };
    auto fetch = [&](uint32_t t, uint32_t tr_, uint32_t tc_, Buf& b) {
        const uint32_t r0 = tr_ * g.gr, c0 = tc_ * g.gc;  // below 2^32: the tile starts inside the matrix
#pragma unroll
        for (int i = 0; i < CPL; i++) {
            const uint32_t r = r0 + rr[i], c = c0 + cc[i];
            b.ok[i] = t < tiles && chunk_ok[i] && r < rows && c < cols;
            b.pos[i] = (uint64_t)r * cols + c;
            if (b.ok[i]) {
                load_chunk8<SRC>(w, b.pos[i], b.v[i]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) b.v[i][j] = 0.0f;
            }
        }
    };
    auto advance = [&]() {
        tile += stride;
        t_r += step_r;
        t_c += step_c;
        if (t_c >= tc) {
            t_c -= tc;
            t_r++;
        }
    };
    auto process = [&](uint32_t t, const Buf& b) {
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < CPL; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) m = max_abs_ignoring_nan(m, b.v[i][j]);
        for (uint32_t o = g.lanes >> 1; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        const float s = scale_from_maxabs(m, HI);
        if (sub == 0 && t < tiles) scales[t] = s;
        const bool fast = s >= 7.888609052210118e-31f && s <= 1.2676506002282294e30f;  // [2^-100, 2^100]
        const float rinv = __frcp_rn(s);
#pragma unroll
        for (int i = 0; i < CPL; i++) {
            if (!b.ok[i]) continue;
            float n[8];
            quantize_chunk8(b.v[i], s, rinv, fast, LO, HI, n);
            if constexpr (BITS == 4) static_cast<uint32_t*>(codes)[b.pos[i] >> 3] = pack_int4x8(n);  // cols % 8 == 0
            else *reinterpret_cast<uint2*>(static_cast<int8_t*>(codes) + b.pos[i]) = pack_int8x8(n);
        }
    };
    // The trip count is the warp's, not the group's (the shuffles need every lane): the warp's first group
    // holds its lowest tile, and a group past the end only skips its loads and stores.  With PF the loop is
    // unrolled by two over a pair of buffers, so the tile in flight is never copied.
    uint32_t tile_w = tile - (lane >> g.lane_shift);
    if constexpr (PF) {
        Buf b0, b1;
        fetch(tile, t_r, t_c, b0);
        while (tile_w < tiles) {
            const uint32_t t0 = tile;
            advance();
            fetch(tile, t_r, t_c, b1);
            process(t0, b0);
            tile_w += stride;
            if (tile_w >= tiles) break;
            const uint32_t t1 = tile;
            advance();
            fetch(tile, t_r, t_c, b0);
            process(t1, b1);
            tile_w += stride;
        }
    } else {
        Buf b0;
        for (; tile_w < tiles; tile_w += stride) {
            fetch(tile, t_r, t_c, b0);
            process(tile, b0);
            advance();
        }
    }
}

// ---- the generic three-pass path ------------------------------------------

// Pass 1: scales[tile] holds the bit pattern of max|w| (non-negative floats
// order like unsigned integers; NaN is mapped to 0 first).
template <int SRC>
__global__ void k_absmax_generic(const void* __restrict__ w, uint64_t rows, uint64_t cols, uint64_t gr,
                                 uint64_t gc, uint64_t tc, uint32_t* __restrict__ maxbits) {
    const uint64_t n = rows * cols;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t r = i / cols, c = i % cols;
        float a = abs_or_zero(load_elem<SRC>(w, i));
        if (a != 0.0f) atomicMax(&maxbits[(r / gr) * tc + c / gc], __float_as_uint(a));
    }
}

__global__ void k_scales_finalize(float* scales, uint64_t n, int hi) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) scales[i] = scale_from_maxabs(scales[i], hi);
}

// Pass 3: one thread per output word (int4: 8 codes) or per 4 codes (int8).
template <int SRC, int BITS>
__global__ void k_encode_generic(const void* __restrict__ w, uint64_t rows, uint64_t cols, uint64_t gr,
                                 uint64_t gc, uint64_t tc, const float* __restrict__ scales,
                                 void* __restrict__ codes) {
    constexpr int HI = BITS == 8 ? 127 : 7;
    constexpr int LO = -HI - 1;
    constexpr uint64_t PER = BITS == 4 ? 8 : 1;
    const uint64_t upr = (cols + PER - 1) / PER;  // units per row
    const uint64_t n = rows * upr;
    for (uint64_t u = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; u < n; u += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t r = u / upr, c0 = (u % upr) * PER;
        if constexpr (BITS == 4) {
            uint32_t word = 0;
            for (uint64_t j = 0; j < 8 && c0 + j < cols; j++) {
                uint64_t c = c0 + j;
                float s = scales[(r / gr) * tc + c / gc];
                int q = quantize_code(load_elem<SRC>(w, r * cols + c), s, LO, HI);
                word |= ((uint32_t)q & 0xFu) << (4 * j);
            }
            static_cast<uint32_t*>(codes)[u] = word;
        } else {
            float s = scales[(r / gr) * tc + c0 / gc];
            static_cast<int8_t*>(codes)[u] = (int8_t)quantize_code(load_elem<SRC>(w, u), s, LO, HI);
        }
    }
}

// ---- large tiles (more than 2048 elements: per-channel rows, per-tensor, big blocks) ----
// Two passes over 8-element chunks with 32-bit index arithmetic; the arithmetic per chunk is the tile kernel's.

// Pass 1: maxbits[tile] = bit pattern of max|w| over the tile.  A warp covers 256 consecutive elements, which
// mostly lie in one tile: one atomic per warp then, not per thread.
template <int SRC>
__global__ void __launch_bounds__(256) k_absmax_chunks(const void* __restrict__ w, uint32_t rows, uint32_t cols, uint32_t gr,
                                                        uint32_t gc, uint32_t tc, uint32_t* __restrict__ maxbits) {
    const uint32_t cpr = cols >> 3, n = rows * cpr, lane = threadIdx.x & 31, stride = gridDim.x * 256;
    for (uint32_t base = blockIdx.x * 256 + (threadIdx.x & ~31u); base < n; base += stride) {  // warp-uniform: n, stride < 2^31
        const uint32_t ch = base + lane;
        const bool valid = ch < n;
        uint32_t tile = 0;
        float m = 0.0f;
        if (valid) {
            const uint32_t r = ch / cpr, c = (ch - r * cpr) * 8u;
            tile = (r / gr) * tc + c / gc;
            float v[8];
            load_chunk8<SRC>(w, (uint64_t)r * cols + c, v);
#pragma unroll
            for (int j = 0; j < 8; j++) m = max_abs_ignoring_nan(m, v[j]);
        }
        const uint32_t tile0 = __shfl_sync(0xFFFFFFFFu, tile, 0);  // lane 0 is valid whenever any lane is
        if (__all_sync(0xFFFFFFFFu, !valid || tile == tile0)) {
#pragma unroll
            for (uint32_t o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            if (lane == 0 && m != 0.0f) atomicMax(&maxbits[tile0], __float_as_uint(m));
        } else if (valid && m != 0.0f) {
            atomicMax(&maxbits[tile], __float_as_uint(m));
        }
    }
}

// Pass 3: one thread per chunk, the tile kernel's quantize_chunk8 and packing.
template <int SRC, int BITS>
__global__ void __launch_bounds__(256) k_encode_chunks(const void* __restrict__ w, uint32_t rows, uint32_t cols, uint32_t gr,
                                                        uint32_t gc, uint32_t tc, const float* __restrict__ scales,
                                                        void* __restrict__ codes) {
    constexpr int HI = BITS == 8 ? 127 : 7;
    constexpr int LO = -HI - 1;
    const uint32_t cpr = cols >> 3, n = rows * cpr, stride = gridDim.x * 256;
    for (uint32_t ch = blockIdx.x * 256 + threadIdx.x; ch < n; ch += stride) {
        const uint32_t r = ch / cpr, c = (ch - r * cpr) * 8u;
        const float s = __ldg(&scales[(r / gr) * tc + c / gc]);
        const bool fast = s >= 7.888609052210118e-31f && s <= 1.2676506002282294e30f;  // [2^-100, 2^100]
        const float rinv = __frcp_rn(s);
        const uint64_t pos = (uint64_t)r * cols + c;
        float v[8], q[8];
        load_chunk8<SRC>(w, pos, v);
        quantize_chunk8(v, s, rinv, fast, LO, HI, q);
        if constexpr (BITS == 4) static_cast<uint32_t*>(codes)[pos >> 3] = pack_int4x8(q);  // cols % 8 == 0
        else *reinterpret_cast<uint2*>(static_cast<int8_t*>(codes) + pos) = pack_int8x8(q);
    }
}

// Whole-row tiles (per-channel scales along the rows, gr == 1 and gc == cols, rows longer than 2048 elements): one
// warp per row reads the row twice, first for its max |w|, then to encode it.  The second read comes back from L2
// (a row is a few KB and was just read), so W crosses HBM once.
template <int SRC, int BITS>
__global__ void __launch_bounds__(256) k_quantize_rows(const void* __restrict__ w, uint32_t rows, uint32_t cols,
                                                        void* __restrict__ codes, float* __restrict__ scales) {
    constexpr int HI = BITS == 8 ? 127 : 7;
    constexpr int LO = -HI - 1;
    const uint32_t lane = threadIdx.x & 31, row = blockIdx.x * 8 + (threadIdx.x >> 5), cpr = cols >> 3;
    if (row >= rows) return;
    const uint64_t base = (uint64_t)row * cols;
    float m = 0.0f;
    uint32_t ch = lane;
    for (; ch + 96 < cpr; ch += 128) {  // four chunks (128 B of f32) in flight per lane
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; u++) load_chunk8<SRC, true>(w, base + (uint64_t)(ch + 32 * u) * 8, v[u]);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int j = 0; j < 8; j++) m = max_abs_ignoring_nan(m, v[u][j]);
    }
    for (; ch < cpr; ch += 32) {
        float v[8];
        load_chunk8<SRC, true>(w, base + (uint64_t)ch * 8, v);
#pragma unroll
        for (int j = 0; j < 8; j++) m = max_abs_ignoring_nan(m, v[j]);
    }
#pragma unroll
    for (uint32_t o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    const float s = scale_from_maxabs(m, HI);
    if (lane == 0) scales[row] = s;
    const bool fast = s >= 7.888609052210118e-31f && s <= 1.2676506002282294e30f;  // [2^-100, 2^100]
    const float rinv = __frcp_rn(s);
    auto encode = [&](uint32_t c, const float (&v)[8]) {
        float q[8];
        quantize_chunk8(v, s, rinv, fast, LO, HI, q);
        const uint64_t pos = base + (uint64_t)c * 8;
        if constexpr (BITS == 4) static_cast<uint32_t*>(codes)[pos >> 3] = pack_int4x8(q);  // cols % 8 == 0
        else *reinterpret_cast<uint2*>(static_cast<int8_t*>(codes) + pos) = pack_int8x8(q);
    };
    ch = lane;
    for (; ch + 96 < cpr; ch += 128) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; u++) load_chunk8<SRC>(w, base + (uint64_t)(ch + 32 * u) * 8, v[u]);
#pragma unroll
        for (int u = 0; u < 4; u++) encode(ch + 32 * u, v[u]);
    }
    for (; ch < cpr; ch += 32) {
        float v[8];
        load_chunk8<SRC>(w, base + (uint64_t)ch * 8, v);
        encode(ch, v);
    }
}

// ---- dequantize -------------------------------------------------------------

// Fast path: cols % 8 == 0 and gc % 8 == 0, so one scale covers a chunk of 8.
template <int BITS>
__global__ void __launch_bounds__(256) k_dequant_chunks(const void* __restrict__ codes,
                                                        const float* __restrict__ scales, uint64_t rows,
                                                        uint64_t cols, uint64_t gr, uint64_t gc, uint64_t tc,
                                                        float* __restrict__ out) {
    const uint64_t cpr = cols >> 3;
    const uint64_t n = rows * cpr;
    uint64_t ch = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= n) return;
    uint64_t r = ch / cpr, c = (ch % cpr) << 3;
    float s = __ldg(&scales[(r / gr) * tc + c / gc]);
    int q[8];
    if constexpr (BITS == 4) {
        uint32_t word = __ldcs(static_cast<const uint32_t*>(codes) + ch);
#pragma unroll
        for (int j = 0; j < 8; j++) q[j] = int4_unpack(word, j);
    } else {
        uint2 b = __ldcs(reinterpret_cast<const uint2*>(static_cast<const int8_t*>(codes) + (ch << 3)));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            q[j] = (int)(int8_t)((b.x >> (8 * j)) & 0xFFu);
            q[4 + j] = (int)(int8_t)((b.y >> (8 * j)) & 0xFFu);
        }
    }
    float4 a = make_float4(dequantize_code(q[0], s), dequantize_code(q[1], s), dequantize_code(q[2], s),
                           dequantize_code(q[3], s));
    float4 b4 = make_float4(dequantize_code(q[4], s), dequantize_code(q[5], s), dequantize_code(q[6], s),
                            dequantize_code(q[7], s));
    float4* o = reinterpret_cast<float4*>(out + (ch << 3));
    __stcs(o, a);
    __stcs(o + 1, b4);
}

// Fastest path: cols % 256 == 0 (and what the chunk path needs), sizes that fit 32 bits.  A warp takes 256
// consecutive elements of a row as one item: every store instruction writes 512 contiguous bytes (lane i the i-th
// 16 bytes).  The kernel is bound by instruction issue, not by HBM, so the item loop is kept lean: the (row, segment)
// pair advances incrementally (two divisions per warp, not per item), tile indices are shifts when the tile sizes
// are powers of two, a lane's four int4 codes come out of its half-word with constant-position sign-extending bit
// field extracts, and a warp issues the loads of four items before it converts and stores any of them.
template <int BITS>
__global__ void __launch_bounds__(256) k_dequant_rows256(const void* __restrict__ codes, const float* __restrict__ scales,
                                                          uint32_t rows, uint32_t cols, uint32_t gr, uint32_t gc, int gr_shift,
                                                          int gc_shift, uint32_t tc, float* __restrict__ out) {
    constexpr uint32_t U = 4;
    const uint32_t lane = threadIdx.x & 31, segs = cols >> 8, items = rows * segs, warps = gridDim.x * 8;
    const uint32_t step_r = warps / segs, step_s = warps - step_r * segs;  // how (row, segment) moves from item to item + warps
    uint32_t item = blockIdx.x * 8 + (threadIdx.x >> 5);  // items < 2^31: item + U * warps cannot wrap
    uint32_t r = item / segs, seg = item - r * segs;
    const uint32_t lane_c = lane * 4u, lane_w = lane >> 1, half = (lane & 1u) * 16u;
    while (item < items) {
        uint32_t word[U][2];
        float sc[U][2];
        uint64_t e0[U];
        bool ok[U];
#pragma unroll
        for (uint32_t u = 0; u < U; u++) {
            ok[u] = item < items;
            if (ok[u]) {
                const float* srow = scales + (uint64_t)(gr_shift >= 0 ? r >> gr_shift : r / gr) * tc;
                e0[u] = (uint64_t)r * cols + seg * 256u;  // first element of the segment
#pragma unroll
                for (uint32_t k = 0; k < 2; k++) {
                    const uint32_t c = seg * 256u + k * 128u + lane_c;
                    sc[u][k] = __ldg(srow + (gc_shift >= 0 ? c >> gc_shift : c / gc));
                    if constexpr (BITS == 4)
                        word[u][k] = __ldcs(static_cast<const uint32_t*>(codes) + ((e0[u] >> 3) + k * 16u + lane_w));
                    else
                        word[u][k] = __ldcs(reinterpret_cast<const uint32_t*>(static_cast<const int8_t*>(codes) + e0[u] + k * 128u + lane_c));
                }
            }
            item += warps;
            seg += step_s;
            r += step_r;
            if (seg >= segs) {
                seg -= segs;
                r++;
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < U; u++) {
            if (ok[u]) {
#pragma unroll
                for (uint32_t k = 0; k < 2; k++) {
                    int q0, q1, q2, q3;
                    if constexpr (BITS == 4) {
                        const uint32_t h = word[u][k] >> half;  // this lane's four nibbles in bits 0..15
                        asm("bfe.s32 %0, %1, 0, 4;" : "=r"(q0) : "r"(h));
                        asm("bfe.s32 %0, %1, 4, 4;" : "=r"(q1) : "r"(h));
                        asm("bfe.s32 %0, %1, 8, 4;" : "=r"(q2) : "r"(h));
                        asm("bfe.s32 %0, %1, 12, 4;" : "=r"(q3) : "r"(h));
                    } else {
                        const uint32_t w = word[u][k];
                        asm("bfe.s32 %0, %1, 0, 8;" : "=r"(q0) : "r"(w));
                        asm("bfe.s32 %0, %1, 8, 8;" : "=r"(q1) : "r"(w));
                        asm("bfe.s32 %0, %1, 16, 8;" : "=r"(q2) : "r"(w));
                        asm("bfe.s32 %0, %1, 24, 8;" : "=r"(q3) : "r"(w));
                    }
                    const float s = sc[u][k];
                    __stcs(reinterpret_cast<float4*>(out + e0[u] + k * 128u + lane_c),
                           make_float4(dequantize_code(q0, s), dequantize_code(q1, s), dequantize_code(q2, s), dequantize_code(q3, s)));
                }
            }
        }
    }
}

template <int BITS>
__global__ void k_dequant_generic(const void* __restrict__ codes, const float* __restrict__ scales,
                                  uint64_t rows, uint64_t cols, uint64_t gr, uint64_t gc, uint64_t tc,
                                  float* __restrict__ out) {
    const uint64_t n = rows * cols, wpr = (cols + 7) / 8;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t r = i / cols, c = i % cols;
        float s = scales[(r / gr) * tc + c / gc];
        int q;
        if constexpr (BITS == 4)
            q = int4_unpack(static_cast<const uint32_t*>(codes)[r * wpr + c / 8], (uint32_t)(c % 8));
        else
            q = (int)static_cast<const int8_t*>(codes)[i];
        out[i] = dequantize_code(q, s);
    }
}

// ---- dispatch -----------------------------------------------------------------

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static qb200_status check_grid(uint64_t rows, uint64_t cols, uint32_t bits, uint64_t gr, uint64_t gc) {
    uint64_t tr, tc;
    if (qb200_status s = qb200_scales_count(rows, cols, gr, gc, &tr, &tc)) return s;
    if (bits != 8 && bits != 4)
        return fail(QB200_ERR_INVALID_PARAM, "code width must be 8 or 4 bits, got " + std::to_string(bits));
    return QB200_OK;
}

static uint32_t grid_for(uint64_t n, uint32_t block, uint64_t cap) {
    uint64_t b = (n + block - 1) / block;
    if (b < 1) b = 1;
    return (uint32_t)(b > cap ? cap : b);
}

template <int SRC, int BITS>
static qb200_status launch_tiles(const void* w, const TileGeom& g, void* codes, float* scales, cudaStream_t st) {
    const uint32_t cpl = (g.chunks + g.lanes - 1) / g.lanes;
    const uint32_t block = 256;
    const uint64_t tiles = g.tr * g.tc, per_block = block / g.lanes;
    uint64_t blocks = (tiles + per_block - 1) / per_block;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // Exactly the blocks that are resident at once (every group then walks many tiles with the grid stride): a
    // partial extra wave leaves SMs idle at the end.  Measured on [11008, 4096]: int8 32x32 39.3 -> 36.6 us.
    static int resident[3][2][4] = {};
    const int ci = cpl <= 1 ? 0 : cpl == 2 ? 1 : cpl <= 4 ? 2 : 3;
    int& per_sm = resident[SRC][BITS == 4 ? 0 : 1][ci];
    if (!per_sm) {
        switch (ci) {
            case 0: QB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_quantize_tiles<SRC, BITS, 1, true>, 256, 0)); break;
            case 1: QB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_quantize_tiles<SRC, BITS, 2, true>, 256, 0)); break;
            case 2: QB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_quantize_tiles<SRC, BITS, 4, false>, 256, 0)); break;
            default: QB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_quantize_tiles<SRC, BITS, 8, false>, 256, 0)); break;
        }
        if (per_sm < 1) per_sm = 1;
    }
    const uint64_t cap = (uint64_t)sms * per_sm;
    if (blocks > cap) blocks = cap;
    dim3 grid((uint32_t)blocks);
    switch (cpl) {
        case 1: k_quantize_tiles<SRC, BITS, 1, true><<<grid, block, 0, st>>>(w, g, codes, scales); break;
        case 2: k_quantize_tiles<SRC, BITS, 2, true><<<grid, block, 0, st>>>(w, g, codes, scales); break;
        case 3:
        case 4: k_quantize_tiles<SRC, BITS, 4, false><<<grid, block, 0, st>>>(w, g, codes, scales); break;
        default: k_quantize_tiles<SRC, BITS, 8, false><<<grid, block, 0, st>>>(w, g, codes, scales); break;
    }
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

template <int SRC, int BITS>
static qb200_status quantize_typed(const void* w, uint64_t rows, uint64_t cols, uint64_t gr, uint64_t gc,
                                   void* codes, float* scales, cudaStream_t st) {
    const uint64_t tr = div_ceil(rows, gr), tc = div_ceil(cols, gc);
    const uint64_t chunks = (gr * gc) / 8;
    const bool src_ok = aligned16(w) && (SRC == SRC_F32 || cols % 8 == 0);
    const bool dst_ok = BITS == 4 ? (reinterpret_cast<uintptr_t>(codes) & 3u) == 0
                                  : (reinterpret_cast<uintptr_t>(codes) & 7u) == 0;
    if (cols % 8 == 0 && gc % 8 == 0 && chunks <= 256 && gr <= 0xFFFFFFFFull && src_ok && dst_ok && tr * tc < (1ull << 31) && rows < (1ull << 32) &&
        cols < (1ull << 32)) {
        TileGeom g;
        g.rows = rows; g.cols = cols; g.gr = (uint32_t)gr; g.gc = (uint32_t)gc; g.tr = tr; g.tc = tc;
        g.chunks_per_row = (uint32_t)(gc / 8);
        g.chunks = (uint32_t)chunks;
        uint32_t lanes = 1;
        // four chunks (128 B of f32) per lane where the tile has them: with one chunk per lane too few bytes are in
        // flight per SM (int4 1x128 on [11008, 4096]: 39.5 us with 16 lanes per tile, 32.3 us with 4)
        while (lanes < 32 && lanes * 4 < g.chunks) lanes <<= 1;
        g.lanes = lanes;
        g.lane_shift = 0;
        while ((1u << g.lane_shift) < lanes) g.lane_shift++;
        return launch_tiles<SRC, BITS>(w, g, codes, scales, st);
    }
    const int hi = BITS == 8 ? 127 : 7;
    if (gr == 1 && gc == cols && cols % 8 == 0 && src_ok && dst_ok && rows < (1ull << 31) && cols < (1ull << 32)) {
        k_quantize_rows<SRC, BITS><<<(uint32_t)((rows + 7) / 8), 256, 0, st>>>(w, (uint32_t)rows, (uint32_t)cols, codes, scales);
        QB_CUDA_TRY(cudaGetLastError());
        return QB200_OK;
    }
    if (cols % 8 == 0 && gc % 8 == 0 && src_ok && dst_ok && rows * (cols / 8) < (1ull << 31) && tr * tc < (1ull << 32) &&
        gr < (1ull << 32) && gc < (1ull << 32)) {
        // large tiles: absmax, scales, encode over 8-element chunks
        const uint32_t grid = grid_for(rows * (cols / 8), 256, 148 * 8);
        QB_CUDA_TRY(cudaMemsetAsync(scales, 0, tr * tc * sizeof(float), st));
        k_absmax_chunks<SRC><<<grid, 256, 0, st>>>(w, (uint32_t)rows, (uint32_t)cols, (uint32_t)gr, (uint32_t)gc, (uint32_t)tc,
                                                  reinterpret_cast<uint32_t*>(scales));
        QB_CUDA_TRY(cudaGetLastError());
        k_scales_finalize<<<grid_for(tr * tc, 256, 0x7FFFFFFF), 256, 0, st>>>(scales, tr * tc, hi);
        QB_CUDA_TRY(cudaGetLastError());
        k_encode_chunks<SRC, BITS><<<grid, 256, 0, st>>>(w, (uint32_t)rows, (uint32_t)cols, (uint32_t)gr, (uint32_t)gc, (uint32_t)tc,
                                                        scales, codes);
        QB_CUDA_TRY(cudaGetLastError());
        return QB200_OK;
    }
    // generic: any grid, any alignment
    QB_CUDA_TRY(cudaMemsetAsync(scales, 0, tr * tc * sizeof(float), st));
    k_absmax_generic<SRC><<<grid_for(rows * cols, 256, 148 * 32), 256, 0, st>>>(
        w, rows, cols, gr, gc, tc, reinterpret_cast<uint32_t*>(scales));
    QB_CUDA_TRY(cudaGetLastError());
    k_scales_finalize<<<grid_for(tr * tc, 256, 0x7FFFFFFF), 256, 0, st>>>(scales, tr * tc, hi);
    QB_CUDA_TRY(cudaGetLastError());
    const uint64_t units = BITS == 4 ? rows * div_ceil(cols, 8) : rows * cols;
    k_encode_generic<SRC, BITS><<<grid_for(units, 256, 148 * 32), 256, 0, st>>>(w, rows, cols, gr, gc, tc, scales, codes);
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

}  // namespace qb

using qb::fail;

extern "C" {

int32_t qb200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

qb200_status qb200_quantize(const void* w_dev, int32_t src_dtype, uint64_t rows, uint64_t cols, uint32_t bits,
                            uint64_t gr, uint64_t gc, void* codes_dev, float* scales_dev, void* stream) {
    if (qb200_status s = qb::check_grid(rows, cols, bits, gr, gc)) return s;
    if (!w_dev || !codes_dev || !scales_dev) return fail(QB200_ERR_INVALID_PARAM, "qb200_quantize: null device pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define QB_Q(SRC)                                                                                              \
    (bits == 8 ? qb::quantize_typed<SRC, 8>(w_dev, rows, cols, gr, gc, codes_dev, scales_dev, st)              \
               : qb::quantize_typed<SRC, 4>(w_dev, rows, cols, gr, gc, codes_dev, scales_dev, st))
    switch (src_dtype) {
        case QB200_F32: return QB_Q(qb::SRC_F32);
        case QB200_BF16: return QB_Q(qb::SRC_BF16);
        case QB200_F16: return QB_Q(qb::SRC_F16);
        default: return fail(QB200_ERR_INVALID_PARAM, "qb200_quantize: unknown source dtype " + std::to_string(src_dtype));
    }
#undef QB_Q
}

qb200_status qb200_dequantize(const void* codes_dev, const float* scales_dev, uint64_t rows, uint64_t cols,
                              uint32_t bits, uint64_t gr, uint64_t gc, float* out_dev, void* stream) {
    if (qb200_status s = qb::check_grid(rows, cols, bits, gr, gc)) return s;
    if (!codes_dev || !scales_dev || !out_dev) return fail(QB200_ERR_INVALID_PARAM, "qb200_dequantize: null device pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint64_t tc = qb::div_ceil(cols, gc);
    const bool fast = cols % 8 == 0 && gc % 8 == 0 && qb::aligned16(out_dev) &&
                      (reinterpret_cast<uintptr_t>(codes_dev) & (bits == 4 ? 3u : 7u)) == 0;
    const bool fast256 = fast && cols % 256 == 0 && gc % 4 == 0 && rows * (cols / 256) < (1ull << 31) && cols < (1ull << 32) &&
                         gr < (1ull << 32) && gc < (1ull << 32) && tc < (1ull << 32);
    if (fast256) {
        // One round of four items per warp: blocks that retire make room for fresh ones, so the loads of some warps
        // always overlap the stores of others (measured on [11008, 4096] int4: 33.7 us; one resident wave of
        // persistent blocks walking the items: 38.2 us).
        const uint64_t items = rows * (cols / 256);
        const uint32_t grid = (uint32_t)((items + 31) / 32 ? (items + 31) / 32 : 1);
        int shift = -1, rshift = -1;  // tile sizes that are powers of two are indexed by shifts
        if ((gc & (gc - 1)) == 0)
            for (shift = 0; (1ull << shift) < gc; shift++) {}
        if ((gr & (gr - 1)) == 0)
            for (rshift = 0; (1ull << rshift) < gr; rshift++) {}
        if (bits == 4)
            qb::k_dequant_rows256<4><<<grid, 256, 0, st>>>(codes_dev, scales_dev, (uint32_t)rows, (uint32_t)cols, (uint32_t)gr, (uint32_t)gc,
                                                           rshift, shift, (uint32_t)tc, out_dev);
        else
            qb::k_dequant_rows256<8><<<grid, 256, 0, st>>>(codes_dev, scales_dev, (uint32_t)rows, (uint32_t)cols, (uint32_t)gr, (uint32_t)gc,
                                                           rshift, shift, (uint32_t)tc, out_dev);
    } else if (fast) {
        const uint64_t n = rows * (cols / 8), blocks = (n + 255) / 256;
        if (blocks > 0x7FFFFFFFull) return fail(QB200_ERR_INVALID_PARAM, "dequantize: matrix too large for one launch");
        if (bits == 4)
            qb::k_dequant_chunks<4><<<(uint32_t)blocks, 256, 0, st>>>(codes_dev, scales_dev, rows, cols, gr, gc, tc, out_dev);
        else
            qb::k_dequant_chunks<8><<<(uint32_t)blocks, 256, 0, st>>>(codes_dev, scales_dev, rows, cols, gr, gc, tc, out_dev);
    } else {
        uint32_t grid = qb::grid_for(rows * cols, 256, 148 * 32);
        if (bits == 4)
            qb::k_dequant_generic<4><<<grid, 256, 0, st>>>(codes_dev, scales_dev, rows, cols, gr, gc, tc, out_dev);
        else
            qb::k_dequant_generic<8><<<grid, 256, 0, st>>>(codes_dev, scales_dev, rows, cols, gr, gc, tc, out_dev);
    }
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

}  // extern "C"
