// Register-resident variant of the persistent decode GEMV for K <= 4096 (at most two scale
// groups per warp with 16 warps).  Each warp keeps the activation fragments of its two groups
// in registers for the whole launch, so an item costs only: two 16-byte code loads per group,
// five integer instructions per packed word, the MMAs and a short f32 epilogue.
// Included by gemv_decode.cu (shares its helpers); see that file for the arithmetic.
#pragma once

namespace qb {

constexpr int REG_WARPS = 16;
constexpr uint32_t REG_THREADS = REG_WARPS * 32;

// One work item of a CTA: where its codes and scales start and where its outputs go.
struct RegItem {
    const uint16_t* x;
    void* y;
    const float* bias;
    const uint8_t* codes;
    const float* scales;
    uint32_t row0, nrows, N, layer;  // layer: index of the launch's layer descriptor (input row stride, valid columns)
};
constexpr uint32_t REG_MAX_ITEMS = 120;  // items per CTA and launch (descriptors: 6.6 KB of shared memory)

struct RegSmem {
    uint32_t desc, red, scales, codes, total, stage_scales, stage_codes;
};
// `red_cols`: batch columns kept per row of partial sums (0: all of the MMA tile's nt * 8)
__host__ __device__ inline RegSmem reg_smem_layout(uint32_t K, uint32_t nt, uint32_t rb, uint32_t stages, uint32_t red_cols = 0) {
    RegSmem L;
    const uint32_t groups = K / 128, batch = red_cols ? red_cols : nt * 8;
    auto up = [](uint32_t v) { return (v + 127u) & ~127u; };
    L.desc = 128;  // barriers at 0
    L.red = L.desc + up(REG_MAX_ITEMS * (uint32_t)sizeof(RegItem));
    L.scales = L.red + up(2 * REG_WARPS * rb * 16 * batch * 4);
    L.stage_scales = up(rb * 16 * groups * 4);
    L.codes = L.scales + stages * L.stage_scales;
    L.stage_codes = up(rb * 16 * (K / 2));
    L.total = L.codes + stages * L.stage_codes;
    return L;
}

// Activation fragment of one scale group for batch row b: the thread's 32 consecutive bf16,
// permuted to the nibble order and scaled; returns their plain sum (for the "+ 8" correction).
// ldx: elements between the rows of x.  out_of_domain is set when an activation cannot take the 2^40 pre-scale.
__device__ __forceinline__ float load_fragment(const uint16_t* __restrict__ x, uint32_t ldx, uint32_t b, uint32_t G,
                                               uint32_t t, bool valid, uint4 (&frag)[4], bool& out_of_domain) {
    uint32_t klo = X_SCALE_LO, khi = X_SCALE_HI;
    const __nv_bfloat162 slo = *reinterpret_cast<const __nv_bfloat162*>(&klo);
    const __nv_bfloat162 shi = *reinterpret_cast<const __nv_bfloat162*>(&khi);
    uint32_t xr[16];
    if (valid) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + (uint64_t)b * ldx + G * 128 + t * 32);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint4 v = __ldg(xp + i);
            xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) xr[i] = 0;
    }
    float sum = 0.0f;
    uint32_t top = 0;  // the largest exponent field among the 32 activations
#pragma unroll
    for (int i = 0; i < 16; i++) {
        sum += bf16_bits_to_f32(xr[i] & 0xFFFFu) + bf16_bits_to_f32(xr[i] >> 16);
        top = max(top, max(xr[i] & 0x7F80u, (xr[i] >> 16) & 0x7F80u));
    }
    if (top >= ((127u + 87u) << 7)) out_of_domain = true;  // |x| >= 2^87, infinite or NaN: the 2^40 pre-scale would overflow
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t o[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t lo = __byte_perm(xr[4 * j + h], xr[4 * j + h + 2], 0x5410);
            uint32_t hi = __byte_perm(xr[4 * j + h], xr[4 * j + h + 2], 0x7632);
            __nv_bfloat162 l2 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&lo), slo);
            __nv_bfloat162 h2 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&hi), shi);
            o[2 * h] = *reinterpret_cast<uint32_t*>(&l2);
            o[2 * h + 1] = *reinterpret_cast<uint32_t*>(&h2);
        }
        frag[j] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    return sum;
}

// One packed word pair (rows g and g + 8) -> the A operands of two MMAs.
#define QB_UNPACK(w0, w1)                                                                                    \
    const uint32_t a0 = lop3_and_xor(w0, NIB_LO, EIGHT_LO), a2 = lop3_and_xor(w0, NIB_HI, EIGHT_HI);         \
    const uint32_t a1 = lop3_and_xor(w1, NIB_LO, EIGHT_LO), a3 = lop3_and_xor(w1, NIB_HI, EIGHT_HI);         \
    const uint32_t d0 = lop3_and_xor((w0) >> 8, NIB_LO, EIGHT_LO), d2 = lop3_and_xor((w0) >> 8, NIB_HI, EIGHT_HI); \
    const uint32_t d1 = lop3_and_xor((w1) >> 8, NIB_LO, EIGHT_LO), d3 = lop3_and_xor((w1) >> 8, NIB_HI, EIGHT_HI);

}  // namespace qb
