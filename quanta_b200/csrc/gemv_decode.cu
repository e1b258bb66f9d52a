// Decode GEMV (M <= 16): y[m, n] = sum_k x[m, k] * s[n, k/128] * q[n, k] over resident
// packed-int4 codes `[N, K/8]` (u32, low nibble first) with a 1x128 f32 scale grid and bf16
// activations.  HBM-bound: the kernel's job is to keep the codes streaming and to spend as
// few issue slots per weight as possible.
//
// Layout and flow, one CTA per contiguous slab of output rows:
//   1. one warp issues bulk async copies (cp.async.bulk, completion on an mbarrier per
//      16-row block) for the slab's codes — every row a contiguous K/2-byte burst — and all
//      threads fetch its scales; nothing here depends on the previous kernel, so with
//      programmatic dependent launch this prefetch overlaps the previous layer's tail;
//   2. griddepcontrol.wait, then each warp takes a slice of the scale groups, loads its x
//      fragment from L2 and multiplies on the tensor pipe (mma.sync m16n8k16, f32
//      accumulate; W rows are the M side, the batch is the N side);
//   3. warps fold their K slices through shared memory and write y (+ bias).
//
// Unpacking costs five integer instructions per packed word.  A bf16 whose exponent field is
// 0 or 1 is linear in its bit pattern (value = bits * 2^-133), and the tensor pipe honours
// such inputs exactly, so a masked nibble IS a bf16 operand: `(w & 0x000F000F) ^ 0x00080008`
// holds (q + 8) for nibbles 0 and 4, `(w & 0x00F000F0) ^ 0x00800080` holds 16 (q + 8) for
// nibbles 1 and 5, and one shift by 8 exposes nibbles 2, 3, 6, 7 the same way.  x is scaled by
// 2^40 (2^36 against the 16x positions) so products stay normal f32; the "+ 8" is removed by
// subtracting 8 * sum_k x_k per group (summed once per CTA), and the group's f32 scale and
// 2^93 are applied once per 128-k group.  Every product (integer code times bf16 activation)
// is exact in f32; the only rounding is f32 accumulation.  Activations must satisfy
// |x| < 2^87.
//
// The kernel is persistent: a CTA walks work items (a slab of <= 16*RB rows of one layer)
// through a ring of shared-memory stages, so the copies of later items are in flight while
// the current one is multiplied.  One launch can serve several layers (grouped forward);
// a single layer is the same kernel with one descriptor.
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdlib>

#include "forward.hpp"
#include "quant_math.cuh"

namespace qb {

constexpr uint32_t GEMV_SPIN_LIMIT = 1u << 22;  // mbarrier polls before giving up (~ seconds)
constexpr int GEMV_MAX_LAYERS = 48;             // descriptors travel by value in the kernel parameters

struct GemvLayer {
    const uint32_t* codes;  // [N, K/8]
    const float* scales;    // [N, K/128]
    const float* bias;      // [N] or null
    const uint16_t* x;      // bf16 [M, K]
    void* y;                // [M, N] f32 or bf16
    uint32_t N, rows_per_item, item0;  // this layer owns items [item0, item0 + ceil(N / rows_per_item))
};

struct GemvBatch {
    GemvLayer layer[GEMV_MAX_LAYERS];
    int32_t* status;  // device status word (0 = ok, QB200_ERR_TIMEOUT on a wait that ran out)
    uint32_t count, total_items, M, K, stages;
    uint32_t async_scales;  // scales are not 16-byte aligned slabs: copy them element-wise
    uint32_t red_cols;      // batch columns kept per row of partial sums (kernels with a service warp)
    uint32_t red_stride;    // floats between rows of a slot of partial sums (>= red_cols)
    uint32_t peer_spin_limit;  // polls of a peer's arrival flag before the barrier gives up
    uint32_t n_peers;       // fused all-gather: every output is stored at y + peer_delta[p], p < n_peers (0: plain store)
    int64_t peer_delta[8];
    uint64_t* peer_flags[8];  // every rank's barrier state as mapped here (null: the caller runs the barrier itself)
    uint32_t rank;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false when the limit ran out (the caller records it and bails out).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < GEMV_SPIN_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy; bytes and both addresses are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) ^ c
    return d;
}

// d = a * b (+ 0): the first MMA of a chain takes a zero accumulator without spending moves.
__device__ __forceinline__ void mma_bf16_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename YT>
__device__ __forceinline__ void store_y(YT* p, float v);
template <>
__device__ __forceinline__ void store_y<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_y<uint16_t>(uint16_t* p, float v) { *p = f32_to_bf16_bits(v); }

// Masks and xor constants of the four nibble pairs of a word (see the header comment).
constexpr uint32_t NIB_LO = 0x000F000Fu, NIB_HI = 0x00F000F0u, EIGHT_LO = 0x00080008u, EIGHT_HI = 0x00800080u;
constexpr uint32_t X_SCALE_LO = 0x53805380u;  // bf16x2 2^40
constexpr uint32_t X_SCALE_HI = 0x51805180u;  // bf16x2 2^36: pairs with the 16x nibble positions
#define GEMV_UNSCALE 9903520314283042199192993792.0f  // 2^93 = 2^133 / 2^40
#define GEMV_EIGHT_X 8.077935669463161e-28f           // 8 * 2^-93: the "+ 8" in units of the MMA partial sums

// Shared-memory carve-up, identical on host and device.
struct GemvSmem {
    uint32_t corr, xtab, red, scales, codes, total;  // byte offsets; barriers sit at 0
    uint32_t stride, stage_scales, stage_codes;
};
__host__ __device__ inline GemvSmem gemv_smem_layout(uint32_t K, uint32_t M, uint32_t rb, uint32_t nt, uint32_t warps,
                                                     uint32_t stages) {
    GemvSmem L;
    const uint32_t groups = K / 128, rows = rb * 16, batch = nt * 8;
    auto up = [](uint32_t v) { return (v + 127u) & ~127u; };
    L.stride = K / 2;  // rows stay contiguous so an item is ONE bulk copy (small copies cap the copy engine)
    L.corr = 128;
    L.xtab = L.corr + up(groups * batch * 4);
    L.red = L.xtab + up(M * K * 2);
    L.scales = L.red + up(2 * warps * rows * batch * 4);
    L.stage_scales = up(rows * groups * 4);
    L.codes = L.scales + stages * L.stage_scales;
    L.stage_codes = up(rows * L.stride);
    L.total = L.codes + stages * L.stage_codes;
    return L;
}

// Offset (bytes) of the 16-byte piece i of the x fragment of (batch row b, group G, lane t).
// Pieces of odd batch rows are swapped in pairs so the two rows served in one shared-memory
// phase fall in different banks.
__device__ __forceinline__ uint32_t xtab_offset(uint32_t b, uint32_t G, uint32_t groups, uint32_t i, uint32_t t) {
    return ((b * groups + G) * 4 + (i ^ (b & 1))) * 64 + t * 16;
}

// Builds the activation table of one layer: per (batch row, group, lane) the 32 activations a
// thread feeds to its eight MMAs, permuted to the nibble order and scaled (2^40 against nibble
// pairs (2h, 2h+4), 2^36 against the 16x pairs (2h+1, 2h+5)), plus corr[G][b] = 8 * 2^-93 * sum, the value the "+ 8" adds to an MMA partial sum.
template <int NT>
__device__ __forceinline__ void build_xtab(const uint16_t* __restrict__ x, uint32_t M, uint32_t K, uint8_t* xtab,
                                           float* corr, uint32_t tid, uint32_t threads) {
    const uint32_t groups = K >> 7, chunks = M * groups * 4;
    uint32_t klo = X_SCALE_LO, khi = X_SCALE_HI;
    const __nv_bfloat162 slo = *reinterpret_cast<const __nv_bfloat162*>(&klo);
    const __nv_bfloat162 shi = *reinterpret_cast<const __nv_bfloat162*>(&khi);
    for (uint32_t c0 = 0; c0 < chunks; c0 += threads) {
        const uint32_t c = c0 + tid;  // chunk = 32 consecutive activations; 4 chunks per (b, G)
        const bool ok = c < chunks;
        const uint32_t t = c & 3, G = (c >> 2) % groups, b = (c >> 2) / groups;
        float sum = 0.0f;
        if (ok) {
            const uint4* xp = reinterpret_cast<const uint4*>(x + (uint64_t)b * K + G * 128 + t * 32);
            uint32_t xr[16];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint4 v = __ldg(xp + i);
                xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < 16; i++) sum += bf16_bits_to_f32(xr[i] & 0xFFFFu) + bf16_bits_to_f32(xr[i] >> 16);
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
                *reinterpret_cast<uint4*>(xtab + xtab_offset(b, G, groups, j, t)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if (ok && t == 0) corr[G * (NT * 8) + b] = sum * GEMV_EIGHT_X;
    }
}

// RB: 16-row blocks per work item; NT: 8-wide batch tiles (M <= 8 * NT); WARPS: warps per CTA.
template <int RB, int NT, int WARPS, typename YT>
__global__ void __launch_bounds__(WARPS * 32) k_gemv_i4(const __grid_constant__ GemvBatch a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t THREADS = WARPS * 32, ROWS = RB * 16, BATCH = NT * 8;
    const uint32_t groups = a.K >> 7, row_bytes = a.K >> 1, S = a.stages;
    const GemvSmem L = gemv_smem_layout(a.K, a.M, RB, NT, WARPS, S);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    float* s_corr = reinterpret_cast<float*>(smem + L.corr);
    uint8_t* s_xtab = smem + L.xtab;
    float* s_red = reinterpret_cast<float*>(smem + L.red);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t n_my = blockIdx.x < a.total_items ? (a.total_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    // which layer an item belongs to (items are numbered layer by layer)
    auto layer_of = [&](uint32_t item, uint32_t from) {
        uint32_t l = from;
        while (l + 1 < a.count && item >= a.layer[l + 1].item0) l++;
        return l;
    };
    // One thread arms the stage barrier and issues ONE bulk copy for the item's codes (its rows are
    // contiguous in HBM) and, when 16-byte aligned, one for its scales; unaligned scales travel as
    // 4-byte async copies.  Every thread's copies are counted on the same barrier.
    auto issue = [&](uint32_t j, uint32_t l) {
        const GemvLayer& ly = a.layer[l];
        const uint32_t item = blockIdx.x + j * gridDim.x, st = j % S;
        const uint32_t row0 = (item - ly.item0) * ly.rows_per_item, nrows = min(ly.rows_per_item, ly.N - row0);
        const float* src = ly.scales + (uint64_t)row0 * groups;
        const uint32_t sbytes = nrows * groups * 4;
        const bool bulk_scales = ((reinterpret_cast<uintptr_t>(src) | sbytes) & 15u) == 0;
        if (tid == 0) {
            mbar_expect_tx(&bars[st], nrows * row_bytes + (bulk_scales ? sbytes : 0));
            bulk_g2s(smem + L.codes + st * L.stage_codes,
                     reinterpret_cast<const uint8_t*>(ly.codes) + (uint64_t)row0 * row_bytes, nrows * row_bytes, &bars[st]);
            if (bulk_scales) bulk_g2s(smem + L.scales + st * L.stage_scales, src, sbytes, &bars[st]);
        }
        if (!bulk_scales) {
            const uint32_t sc = smem_u32(smem + L.scales + st * L.stage_scales);
            for (uint32_t i = tid; i < nrows * groups; i += THREADS)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sc + i * 4), "l"(src + i) : "memory");
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars[st])) : "memory");
    };

    if (tid == 0) {
        for (uint32_t s = 0; s < S; s++) mbar_init(&bars[s], 1 + THREADS);  // the expect_tx arrival + one per thread
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t l_issue = 0;
    for (uint32_t j = 0; j < n_my && j < S; j++) {
        l_issue = layer_of(blockIdx.x + j * gridDim.x, l_issue);
        issue(j, l_issue);
    }
    // The codes and scales do not depend on the previous kernel; everything below may.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const uint16_t* cur_x = nullptr;
    uint32_t l_cur = 0;
    bool failed = false;
    for (uint32_t j = 0; j < n_my; j++) {
        const uint32_t item = blockIdx.x + j * gridDim.x, st = j % S;
        l_cur = layer_of(item, l_cur);
        const GemvLayer& ly = a.layer[l_cur];
        if (ly.x != cur_x) {  // uniform: rebuild the activation table (the barrier below also orders the reuse)
            cur_x = ly.x;
            build_xtab<NT>(cur_x, a.M, a.K, s_xtab, s_corr, tid, THREADS);
            __syncthreads();
        } else if (j == 0) {
            __syncthreads();
        }
        const uint32_t row0 = (item - ly.item0) * ly.rows_per_item, nrows = min(ly.rows_per_item, ly.N - row0);
        if (!mbar_wait_bounded(&bars[st], (j / S) & 1)) failed = true;

        const uint8_t* s_codes = smem + L.codes + st * L.stage_codes;
        const float* s_scales = reinterpret_cast<const float*>(smem + L.scales + st * L.stage_scales);
        float acc[RB][NT][4];
#pragma unroll
        for (int rb = 0; rb < RB; rb++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[rb][nt][i] = 0.0f;

        for (uint32_t G = warp; G < groups && !failed; G += WARPS) {
            // codes of this group: rows g and g + 8 of every row block
            uint4 c0[RB], c1[RB];
#pragma unroll
            for (int rb = 0; rb < RB; rb++) {
                c0[rb] = *reinterpret_cast<const uint4*>(s_codes + (rb * 16 + g) * L.stride + G * 64 + t * 16);
                c1[rb] = *reinterpret_cast<const uint4*>(s_codes + (rb * 16 + g + 8) * L.stride + G * 64 + t * 16);
            }
            float p[RB][NT][2][4];
#pragma unroll
            for (int j4 = 0; j4 < 4; j4++) {
                uint4 bx[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint32_t b = g + 8 * nt;
                    bx[nt] = b < a.M ? *reinterpret_cast<const uint4*>(s_xtab + xtab_offset(b, G, groups, j4, t))
                                     : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int rb = 0; rb < RB; rb++) {
                    const uint32_t w0 = j4 == 0 ? c0[rb].x : j4 == 1 ? c0[rb].y : j4 == 2 ? c0[rb].z : c0[rb].w;
                    const uint32_t w1 = j4 == 0 ? c1[rb].x : j4 == 1 ? c1[rb].y : j4 == 2 ? c1[rb].z : c1[rb].w;
                    const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
                    const uint32_t a0 = lop3_and_xor(w0, NIB_LO, EIGHT_LO), a2 = lop3_and_xor(w0, NIB_HI, EIGHT_HI);
                    const uint32_t a1 = lop3_and_xor(w1, NIB_LO, EIGHT_LO), a3 = lop3_and_xor(w1, NIB_HI, EIGHT_HI);
                    const uint32_t d0 = lop3_and_xor(w0s, NIB_LO, EIGHT_LO), d2 = lop3_and_xor(w0s, NIB_HI, EIGHT_HI);
                    const uint32_t d1 = lop3_and_xor(w1s, NIB_LO, EIGHT_LO), d3 = lop3_and_xor(w1s, NIB_HI, EIGHT_HI);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        if (j4 == 0) {
                            mma_bf16_first(p[rb][nt][0], a0, a1, a2, a3, bx[nt].x, bx[nt].y);
                            mma_bf16_first(p[rb][nt][1], d0, d1, d2, d3, bx[nt].z, bx[nt].w);
                        } else {
                            mma_bf16(p[rb][nt][0], a0, a1, a2, a3, bx[nt].x, bx[nt].y);
                            mma_bf16(p[rb][nt][1], d0, d1, d2, d3, bx[nt].z, bx[nt].w);
                        }
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const float2 kc = *reinterpret_cast<const float2*>(s_corr + G * BATCH + nt * 8 + 2 * t);
#pragma unroll
                for (int rb = 0; rb < RB; rb++) {
                    const float s0 = s_scales[(rb * 16 + g) * groups + G] * GEMV_UNSCALE;
                    const float s1 = s_scales[(rb * 16 + g + 8) * groups + G] * GEMV_UNSCALE;
                    acc[rb][nt][0] = fmaf(s0, (p[rb][nt][0][0] + p[rb][nt][1][0]) - kc.x, acc[rb][nt][0]);
                    acc[rb][nt][1] = fmaf(s0, (p[rb][nt][0][1] + p[rb][nt][1][1]) - kc.y, acc[rb][nt][1]);
                    acc[rb][nt][2] = fmaf(s1, (p[rb][nt][0][2] + p[rb][nt][1][2]) - kc.x, acc[rb][nt][2]);
                    acc[rb][nt][3] = fmaf(s1, (p[rb][nt][0][3] + p[rb][nt][1][3]) - kc.y, acc[rb][nt][3]);
                }
            }
        }

        // fold the K slices of the warps through red[j & 1][warp][row][batch]
        float* red = s_red + (j & 1) * (WARPS * ROWS * BATCH);
#pragma unroll
        for (int rb = 0; rb < RB; rb++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float* base = red + (warp * ROWS + rb * 16) * BATCH + nt * 8;
                *reinterpret_cast<float2*>(base + g * BATCH + 2 * t) = make_float2(acc[rb][nt][0], acc[rb][nt][1]);
                *reinterpret_cast<float2*>(base + (g + 8) * BATCH + 2 * t) = make_float2(acc[rb][nt][2], acc[rb][nt][3]);
            }
        if (__syncthreads_or(failed ? 1 : 0)) {
            failed = true;
            break;
        }
        // the stage is free: refill it with the item S steps ahead
        if (j + S < n_my) {
            l_issue = layer_of(blockIdx.x + (j + S) * gridDim.x, l_issue);
            issue(j + S, l_issue);
        }
        for (uint32_t e = tid; e < nrows * a.M; e += THREADS) {
            const uint32_t r = e % nrows, b = e / nrows;
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) v += red[(w * ROWS + r) * BATCH + b];
            const uint32_t n = row0 + r;
            if (ly.bias) v += ly.bias[n];
            store_y<YT>(static_cast<YT*>(ly.y) + (uint64_t)b * ly.N + n, v);
        }
    }
    if (failed) {
        // A copy never completed: record it, give copies still in flight a bounded chance to land, leave.
        if (tid == 0) atomicExch(a.status, QB200_ERR_TIMEOUT);
        for (uint32_t s = 0; s < S; s++) mbar_wait_bounded(&bars[s], 0);
    }
}

}  // namespace qb

#include "gemv_reg.cuh"
#include "gemv_reg_kernel.cuh"
#include "gemv_reg_async.cuh"

namespace qb {

// ---- host side ------------------------------------------------------------------

template <int NT, int RB, typename YT>
static qb200_status launch_gemv_async(const GemvBatch& b, uint32_t smem, uint32_t ctas, cudaStream_t st) {
    auto kern = k_gemv_i4_async<NT, RB, YT>;
    static bool attr_set[64] = {};  // per instantiation and device
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        QB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(async_threads(NT));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, b));
    return QB200_OK;
}

template <int NT, int RB, int OCC, typename YT>
static qb200_status launch_gemv_reg(const GemvBatch& b, uint32_t smem, uint32_t ctas, cudaStream_t st) {
    auto kern = k_gemv_i4_reg<NT, RB, OCC, YT>;
    static bool attr_set[64] = {};  // per instantiation and device
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        QB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(REG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, b));
    return QB200_OK;
}

struct GemvShape {
    uint32_t rb, nt, warps, stages, smem, rows_per_item;
};

bool gemv_i4_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* scales, const void* x) {
    if (bits != 4 || gr != 1 || gc != 128 || layout != QB200_OUT_IN || x_dtype != QB200_BF16) return false;
    if (m == 0 || m > 16 || in_dim % 128 != 0 || in_dim > 32768 || out_dim > 0x7FFFFFFF) return false;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return al(codes) && al(scales) && al(x);
}

// Rows per work item.  A launch with few items per CTA cuts the layer into a multiple of 148
// items of at most 16 * rb rows, so the last wave of items is as full as the others; a launch
// with many items per CTA (`full_tiles`) takes whole 16 * rb-row items instead — the MMA and the
// unpack cost the same for a 28-row item as for a 32-row one, and the waves even out by number.
static uint32_t gemv_rows_per_item(uint32_t N, uint32_t rb, bool full_tiles) {
    if (full_tiles) return 16 * rb;
    const uint32_t tiles = (N + 16 * rb - 1) / (16 * rb), k = (tiles + 147) / 148;
    uint32_t rows = (N + 148 * k - 1) / (148 * k);
    return rows < 1 ? 1 : rows;
}

// Picks the stage count that fits shared memory; false when the activation table does not fit.
static bool gemv_shape(uint32_t K, uint32_t M, uint32_t max_items_per_cta, bool chained, GemvShape& s) {
    s.nt = M <= 8 ? 1 : 2;
    s.rb = 1;
    s.warps = s.nt == 1 ? 16 : 8;
    const uint32_t cap = 227 * 1024, want = max_items_per_cta < 2 ? 2 : (max_items_per_cta > 4 ? 4 : max_items_per_cta);
    for (uint32_t st = want; st >= 2; st--) {
        GemvSmem L = gemv_smem_layout(K, M, s.rb, s.nt, s.warps, st);
        if (L.total <= cap) {
            s.stages = st;
            s.smem = L.total;
            (void)chained;
            return true;
        }
    }
    return false;
}

template <int NT, typename YT>
static qb200_status launch_gemv(const GemvBatch& b, const GemvShape& s, uint32_t ctas, cudaStream_t st) {
    auto kern = k_gemv_i4<1, NT, (NT == 1 ? 16 : 8), YT>;
    static bool attr_set[64] = {};  // per instantiation and device
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        QB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(s.warps * 32);
    cfg.dynamicSmemBytes = s.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, b));
    return QB200_OK;
}

// Grouped forward over `count` layers that share K and M.  Returns QB200_ERR_NOT_SUPPORTED
// (without setting an error) when the shape does not fit the kernel.
qb200_status gemv_i4_forward_many(const FwdArgs* f, uint32_t count, int y_dtype, int32_t* status, cudaStream_t st,
                                  const PeerSpec* peers) {
    if (count == 0) return QB200_OK;
    const uint32_t K = (uint32_t)f[0].in_dim, M = (uint32_t)f[0].m;
    const bool reg_path = K / 128 <= 2 * REG_WARPS;
    // Row blocks per item: a lone small layer keeps 16-row items (more items to pipeline and to
    // overlap with the neighbouring launches); grouped launches take 32-row items.
    uint32_t rb = (count > 1 || peers) ? 2 : 1;
    if (!reg_path) rb = 1;
    uint64_t all_tiles = 0;
    for (uint32_t i = 0; i < count; i++) all_tiles += (f[i].out_dim + 16 * rb - 1) / (16 * rb);
    const bool full_tiles = all_tiles >= 8 * 148;  // eight or more items per CTA
    for (uint32_t base = 0, n = 0; base < count; base += n) {
        // as many layers as fit the descriptor table and, on the register path, the per-CTA item table
        n = 0;
        for (uint32_t items = 0; base + n < count && n < (uint32_t)GEMV_MAX_LAYERS; n++) {
            const uint32_t N = (uint32_t)f[base + n].out_dim, rpi = gemv_rows_per_item(N, rb, full_tiles);
            items += (N + rpi - 1) / rpi;
            if (reg_path && n > 0 && items > REG_MAX_ITEMS * 148) break;
        }
        GemvBatch b = {};
        uint32_t items = 0;
        for (uint32_t i = 0; i < n; i++) {
            const FwdArgs& a = f[base + i];
            GemvLayer& ly = b.layer[i];
            ly.codes = static_cast<const uint32_t*>(a.codes);
            ly.scales = a.scales;
            ly.bias = a.bias;
            ly.x = static_cast<const uint16_t*>(a.x);
            ly.y = a.y;
            ly.N = (uint32_t)a.out_dim;
            ly.rows_per_item = gemv_rows_per_item(ly.N, rb, full_tiles);
            ly.item0 = items;
            items += (ly.N + ly.rows_per_item - 1) / ly.rows_per_item;
        }
        b.async_scales = (K % 512 != 0) ? 1 : 0;  // a row of scales is K / 32 bytes
        for (uint32_t i = 0; i < n; i++)
            if (reinterpret_cast<uintptr_t>(b.layer[i].scales) & 15u) b.async_scales = 1;
        b.status = status;
        b.n_peers = peers ? peers->world : 0;
        for (uint32_t p = 0; p < 8; p++) {
            b.peer_delta[p] = peers ? peers->delta[p] : 0;
            b.peer_flags[p] = peers ? peers->flags[p] : nullptr;
        }
        b.rank = peers ? peers->rank : 0;
        b.peer_spin_limit = peer_spin_limit();
        b.count = n;
        b.total_items = items;
        b.M = M;
        b.K = K;
        uint32_t ctas = items < 148 ? items : 148;
        if (reg_path && (items + 147) / 148 <= REG_MAX_ITEMS) {  // activation fragments stay in registers
            const uint32_t nt = M <= 8 ? 1 : 2;
            // The kernel with a service warp serves 32-row items and every batch above 8; a lone layer with a
            // small batch keeps 16-row items on the kernel whose warps fold together (two CTAs per SM).
            static const bool exp_async11 = getenv("QB200_EXP_ASYNC11") != nullptr;  // EXPERIMENT
            const bool service = nt == 2 || rb == 2 || exp_async11;
            if (peers && !service) return QB200_ERR_NOT_SUPPORTED;  // only the service warp stores to peers
            qb200_status r;
            if (service) {
                // slots of partial sums keep only the batch's columns, which for a single row frees the room of
                // one more 68 KB stage; 16-row sub-items (nt == 2) pad their rows against bank conflicts
                b.red_cols = M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : (M + 1) & ~1u;
                b.red_stride = nt == 2 ? async_red_stride(b.red_cols) : b.red_cols;
                const uint32_t sub_rows = nt == 2 ? 16 : rb * 16;
                ctas = items < 148 ? items : 148;
                const uint32_t per_cta = (items + ctas - 1) / ctas;
                uint32_t stages = per_cta < 2 ? 2 : (per_cta > 5 ? 5 : per_cta);
                while (stages > 2 && async_smem_layout(K, rb, sub_rows, b.red_stride, stages).total > 227u * 1024) stages--;
                b.stages = stages;
                const uint32_t smem = async_smem_layout(K, rb, sub_rows, b.red_stride, stages).total;
                if (smem > 227u * 1024) return QB200_ERR_NOT_SUPPORTED;
#define QB_LAUNCH(YT)                                                                                        \
    (nt == 2 ? (rb == 2 ? launch_gemv_async<2, 2, YT>(b, smem, ctas, st) : launch_gemv_async<2, 1, YT>(b, smem, ctas, st)) \
             : (rb == 2 ? launch_gemv_async<1, 2, YT>(b, smem, ctas, st) : launch_gemv_async<1, 1, YT>(b, smem, ctas, st)))
                r = y_dtype == QB200_F32 ? QB_LAUNCH(float) : QB_LAUNCH(uint16_t);
#undef QB_LAUNCH
            } else {
                const uint32_t occ = 2;
                ctas = items < 148 * occ ? items : 148 * occ;
                const uint32_t per_cta = (items + ctas - 1) / ctas, budget = 113u * 1024;
                uint32_t stages = per_cta < 2 ? 2 : (per_cta > 5 ? 5 : per_cta);
                while (stages > 2 && reg_smem_layout(K, 1, 1, stages).total > budget) stages--;
                b.stages = stages;
                r = y_dtype == QB200_F32 ? launch_gemv_reg<1, 1, 2, float>(b, reg_smem_layout(K, 1, 1, stages).total, ctas, st)
                                         : launch_gemv_reg<1, 1, 2, uint16_t>(b, reg_smem_layout(K, 1, 1, stages).total, ctas, st);
            }
            if (r) return r;
            continue;
        }
        if (peers) return QB200_ERR_NOT_SUPPORTED;
        GemvShape s;
        if (!gemv_shape(K, M, (items + ctas - 1) / ctas, n == 1, s)) return QB200_ERR_NOT_SUPPORTED;
        b.stages = s.stages;
        qb200_status r;
        if (y_dtype == QB200_F32)
            r = s.nt == 1 ? launch_gemv<1, float>(b, s, ctas, st) : launch_gemv<2, float>(b, s, ctas, st);
        else
            r = s.nt == 1 ? launch_gemv<1, uint16_t>(b, s, ctas, st) : launch_gemv<2, uint16_t>(b, s, ctas, st);
        if (r) return r;
    }
    return QB200_OK;
}

qb200_status gemv_i4_forward(const FwdArgs& f, int y_dtype, int32_t* status, cudaStream_t st) {
    return gemv_i4_forward_many(&f, 1, y_dtype, status, st, nullptr);
}

}  // namespace qb
