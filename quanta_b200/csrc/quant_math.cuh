// Device twins of the reference's quantization arithmetic
// (crates/gpu/quanta-ir/src/dtype.rs:8-21, 232-268).  Every function here is
// bit-exact against the host definition: IEEE f32 divide, round-to-nearest-even,
// saturating conversion, one f32 multiply for dequantize.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace qb {

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

// Round-to-nearest-even; a NaN keeps its top half and is quieted (dtype.rs:14-21).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    uint32_t bits = __float_as_uint(v);
    if (v != v) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t bias = 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}

// |w| for the tile max: Rust's f32::max ignores a NaN operand, so a NaN weight
// contributes nothing (quanta-array/src/quant.rs:302-306).
__device__ __forceinline__ float abs_or_zero(float w) { return (w != w) ? 0.0f : fabsf(w); }
// max(m, |w|) with the same rule in one instruction: fmaxf returns its other operand when one is NaN
// (m itself is never NaN: it starts at 0).
__device__ __forceinline__ float max_abs_ignoring_nan(float m, float w) { return fmaxf(m, fabsf(w)); }

// s = max|w| / hi as one IEEE divide (quanta-array/src/quant.rs:308).
__device__ __forceinline__ float scale_from_maxabs(float m, int hi) { return __fdiv_rn(m, (float)hi); }

// clamp(round_ties_even(x / s) as i32, lo, hi) with s == 0 -> 0
// (dtype.rs:238-242, quanta-array/src/quant.rs:336-343).  __float2int_rn rounds
// to nearest even, saturates and maps NaN to 0 — Rust's `as i32`.
__device__ __forceinline__ int quantize_code(float x, float s, int lo, int hi) {
    if (s == 0.0f) return 0;
    int r = __float2int_rn(__fdiv_rn(x, s));
    return min(max(r, lo), hi);
}

// The same eight codes at a fraction of the instructions: d' = x * (1 / s) differs from the
// IEEE quotient d = x / s by at most 1.5 * 2^-23 * |x / s| <= 2.4e-5 (|x / s| <= 128 by
// construction of s), so whenever d' is further than 2^-14 from every half-integer, d lies in
// the same rounding interval and rte(d') == rte(d).  Otherwise — and for scales outside
// [2^-100, 2^100], zero, infinite or NaN, where 1 / s is not trustworthy — the chunk is redone
// with the exact divide.  A NaN weight fails the distance test (comparison with NaN is false)
// and takes the exact path too.  On the fast path no clamp is needed: |x| <= max|w| = m and
// s = fl(m / hi) >= (m / hi)(1 - 2^-24) give |x / s| < hi + 0.5.  The codes come back as
// integral floats (the packers below work in floating point).  Result: bit-identical to
// quantize_code for every input.
__device__ __forceinline__ void quantize_chunk8(const float (&x)[8], float s, float rinv, bool fast, int lo, int hi,
                                                float (&n)[8]) {
    bool redo = !fast;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float d = __fmul_rn(x[j], rinv);
        n[j] = rintf(d);
        redo |= !(fabsf(__fsub_rn(d, n[j])) < 0.49993896484375f);  // 0.5 - 2^-14
    }
    if (redo) {
#pragma unroll
        for (int j = 0; j < 8; j++) n[j] = (float)quantize_code(x[j], s, lo, hi);
    }
}

// Eight int4 codes (integral floats in [-8, 7]) -> one packed word, low nibble first.  Each
// half is built by Horner in f32 (16 bits: exact) from q + 8, which is the nibble with its top
// bit flipped; one XOR restores the two's-complement nibbles.
__device__ __forceinline__ uint32_t pack_int4x8(const float (&n)[8]) {
    float lo = fmaf(n[3], 16.0f, n[2]), hi = fmaf(n[7], 16.0f, n[6]);
    lo = fmaf(lo, 16.0f, n[1]);
    hi = fmaf(hi, 16.0f, n[5]);
    lo = fmaf(lo, 16.0f, n[0] + 34952.0f);  // + 8 * (1 + 16 + 256 + 4096)
    hi = fmaf(hi, 16.0f, n[4] + 34952.0f);
    const uint32_t l = (uint32_t)__float2int_rn(lo), h = (uint32_t)__float2int_rn(hi);
    return (l | (h << 16)) ^ 0x88888888u;
}

// Eight int8 codes (integral floats in [-128, 127]) -> two words of four bytes, low byte first.
__device__ __forceinline__ uint2 pack_int8x8(const float (&n)[8]) {
    uint32_t h[4];
#pragma unroll
    for (int i = 0; i < 4; i++)  // (q1 + 128) * 256 + (q0 + 128): 16 bits, exact in f32
        h[i] = (uint32_t)__float2int_rn(fmaf(n[2 * i + 1], 256.0f, n[2 * i] + 32896.0f));
    uint2 out;
    out.x = (h[0] | (h[1] << 16)) ^ 0x80808080u;
    out.y = (h[2] | (h[3] << 16)) ^ 0x80808080u;
    return out;
}

// scale * f32(q): one multiply, never fused with anything (dtype.rs:245-247).
__device__ __forceinline__ float dequantize_code(int q, float s) { return __fmul_rn(s, (float)q); }

// Nibble i (0..8) of a packed word, sign-extended (dtype.rs:256-260).
__device__ __forceinline__ int int4_unpack(uint32_t word, uint32_t i) {
    uint32_t n = (word >> (i * 4u)) & 0xFu;
    return (int)((n ^ 0x8u) - 0x8u);
}

__device__ __forceinline__ float load_as_f32(const float* p, uint64_t i) { return p[i]; }

// IEEE half -> f32 is exact for every class (safetensors.rs:354-373).
__device__ __forceinline__ float half_bits_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)(h >> 15)) << 31, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {
            int top = 31 - __clz((int)m);
            bits = sign | ((uint32_t)(127 + top - 24) << 23) | ((m << (23 - top)) & 0x7FFFFFu);
        }
    } else if (e == 0x1F) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    }
    return __uint_as_float(bits);
}

}  // namespace qb
