// Prefill GEMM (M >= 64): Y[m, n] = sum_k X[m, k] * s[n, k/128] * q[n, k] over resident
// packed-int4 codes `[N, K/8]` with a 1x128 f32 scale grid, bf16 activations, f32 accumulation.
// Tensor-core bound: tcgen05.mma with the accumulator in TMEM.
//
// Staging (stated, and mirrored by the checker): the codes enter the tensor core as EXACT
// integers and the activations as exact bf16, so every product is exact in f32; a group's
// f32 scale is applied to the group's partial sum, never to a weight.  Concretely
//   * a pre-pass writes X' = X * 2^40 (exact in bf16) and corr[m, g] = 8 * sum_{k in g} X[m, k];
//   * the B operand holds (q + 8) as a bf16 whose exponent field is zero — such a value is
//     its bit pattern times 2^-133, and the tensor core honours it exactly — so unpacking a
//     word costs one shift, two LOP3 and four PRMT and no floating-point work;
//   * per 128-k group the MMA leaves D_g = 2^-93 * sum (q + 8) x in TMEM; the epilogue warps
//     fold total += s[n, g] * (D_g * 2^93 - corr[m, g]) in registers (f32).
// X' and corr live in a scratch buffer owned by the QuantizedLinear handle.
//
// A persistent kernel, one CTA per SM, walks 128 (m) x 256 (n) output tiles (m fastest, so the
// CTAs that run together share code rows in L2).  The tile is wide in n because the int4 side
// is the cheap one to fetch: per 64-k step a CTA pulls 16 KB of activations and 8 KB of codes
// for 512 tensor-core cycles of work.  Roles, by warp:
//   warp 0        TMA producer: X' tiles (128B-swizzled) and packed-code tiles (64B-swizzled)
//   warp 1        MMA issuer (128 x 256 x 16, two 256-column TMEM accumulators)
//   warps 2-3     stage the tile's scales and corrections, four groups at a time, transposed
//   warps 4-7     unpack the packed codes from shared memory into the swizzled B ring
//   warps 8-15    TMEM epilogue: per-group promotion into 128 f32 totals per thread, final store
// Registers are re-balanced between the roles with setmaxnreg (the epilogue keeps a 128 x 256
// f32 tile).  All rings run across tile boundaries, so one tile's store overlaps the next
// tile's K loop.  Every wait is bounded and reports through the handle's status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <string>

#include "forward.hpp"
#include "quant_math.cuh"

namespace qb {

constexpr uint32_t PF_BM = 128, PF_BN = 256, PF_BK = 64;  // tile; BK bf16 = one 128-byte swizzle row
constexpr uint32_t PF_SA = 4, PF_SB = 3;                  // ring depths: X' stages (16 KB), B stages (32 KB)
constexpr uint32_t PF_SQ = 3;                             // ring of packed-code slots: 256 rows x 64 B = one k-group each
constexpr uint32_t PF_SC = 2, PF_CG = 4;                  // scale ring: slots, groups per slot
constexpr uint32_t PF_SLOT_FLOATS = PF_CG * (PF_BN + PF_BM);
constexpr uint32_t PF_THREADS = 512;
constexpr uint32_t PF_A_BYTES = PF_BM * 128, PF_B_BYTES = PF_BN * 128, PF_Q_BYTES = PF_BN * 64;
constexpr uint32_t PF_SMEM =
    1024 + PF_SA * PF_A_BYTES + PF_SB * PF_B_BYTES + PF_SQ * PF_Q_BYTES + PF_SC * PF_SLOT_FLOATS * 4 + 256;
constexpr uint32_t PF_SPIN = 1u << 22;
#define PF_UNSCALE 9903520314283042199192993792.0f  // 2^93
#define PF_RESCALE 1.0097419586828951e-28f             // 2^-93

// ---- pre-pass: X' = X * 2^40, corr[g, m] = 8 * sum_{k in g} X[m, k] (group-major) -----------
// One warp per (row, group of 128): lanes read 8 bytes each.
__global__ void __launch_bounds__(256) k_prefill_prep(const uint16_t* __restrict__ x, uint32_t M, uint32_t K,
                                                      uint16_t* __restrict__ xs, float* __restrict__ corr) {
    const uint32_t groups = K >> 7, lane = threadIdx.x & 31;
    const uint64_t unit = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (uint64_t)M * groups) return;
    const uint32_t m = (uint32_t)(unit / groups), g = (uint32_t)(unit % groups);
    const uint64_t off = (uint64_t)m * K + g * 128 + lane * 4;
    const uint2 v = *reinterpret_cast<const uint2*>(x + off);
    const uint32_t k40 = 0x53805380u;  // bf16x2 2^40
    const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162*>(&k40);
    uint32_t w[2] = {v.x, v.y};
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        sum += bf16_bits_to_f32(w[i] & 0xFFFFu) + bf16_bits_to_f32(w[i] >> 16);
        __nv_bfloat162 p = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&w[i]), sc);
        w[i] = *reinterpret_cast<uint32_t*>(&p);
    }
    *reinterpret_cast<uint2*>(xs + off) = make_uint2(w[0], w[1]);
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane == 0) corr[(uint64_t)g * M + m] = 8.0f * sum;
}

// ---- PTX helpers ------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t pf_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pf_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_smem(bar)), "r"(count));
}
__device__ __forceinline__ void pf_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pf_smem(bar)) : "memory");
}
__device__ __forceinline__ void pf_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pf_smem(bar)), "r"(bytes) : "memory");
}
// Bounded wait: false when the poll limit ran out.
__device__ __forceinline__ bool pf_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < PF_SPIN; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(pf_smem(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void pf_tma_load_2d(void* dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            pf_smem(dst)),
        "l"(map), "r"(x), "r"(y), "r"(pf_smem(bar))
        : "memory");
}
// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t pf_desc(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;               // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;     // stride byte offset
    d |= (uint64_t)1 << 46;               // descriptor version
    d |= (uint64_t)2 << 61;               // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void pf_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pf_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pf_smem(bar)) : "memory");
}
__device__ __forceinline__ void pf_tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}


__device__ __forceinline__ uint64_t pf_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
// (t0, t1) += (s0, s1) * ((v0, v1) + (c, c)) with the packed f32x2 add / fma of sm_100
__device__ __forceinline__ void pf_fold2(float& t0, float& t1, float s0, float s1, float v0, float v1, uint64_t c2) {
    asm("{\n\t.reg .b64 t, s, v, d;\n\t"
        "mov.b64 t, {%0, %1};\n\tmov.b64 s, {%2, %3};\n\tmov.b64 v, {%4, %5};\n\t"
        "add.rn.f32x2 d, v, %6;\n\tfma.rn.f32x2 t, s, d, t;\n\t"
        "mov.b64 {%0, %1}, t;\n\t}"
        : "+f"(t0), "+f"(t1)
        : "f"(s0), "f"(s1), "f"(v0), "f"(v1), "l"(c2));
}

struct PrefillArgs {
    const uint32_t* codes;  // [N, K/8]
    const float* scales;    // [N, K/128]
    const float* bias;      // [N] or null
    const float* corr;      // [K/128, M]: 8 * group sums of X
    void* y;                // [M, N] bf16 or f32
    int32_t* status;
    uint32_t M, N, K;
    uint32_t vec_store;     // 1 when every row of y and the bias take 16-byte accesses
};

// One packed word -> eight bf16 values (q + 8) * 2^-133 in natural k order (four registers).
__device__ __forceinline__ void pf_unpack(uint32_t w, uint32_t (&r)[4]) {
    uint32_t t0, t1;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(t0) : "r"(w), "r"(0x0F0F0F0Fu), "r"(0x08080808u));       // nibbles 0,2,4,6
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(t1) : "r"(w >> 4), "r"(0x0F0F0F0Fu), "r"(0x08080808u));  // nibbles 1,3,5,7
    // selector 8 replicates the (clear) sign bit of a byte: a zero byte for the bf16 high halves
    // (prmt.b32 in PTX: the __byte_perm intrinsic ignores the replicate bit)
    asm("prmt.b32 %0, %1, %2, 0x8480;" : "=r"(r[0]) : "r"(t0), "r"(t1));
    asm("prmt.b32 %0, %1, %2, 0x8581;" : "=r"(r[1]) : "r"(t0), "r"(t1));
    asm("prmt.b32 %0, %1, %2, 0x8682;" : "=r"(r[2]) : "r"(t0), "r"(t1));
    asm("prmt.b32 %0, %1, %2, 0x8783;" : "=r"(r[3]) : "r"(t0), "r"(t1));
}

// Unpacks the 64 codes of one row and k-step (two 16-byte loads) into the row's 128-byte line of a
// swizzled B stage: chunk c lands at (row_off ^ (c << 4)).
__device__ __forceinline__ void pf_unpack_row(uint8_t* dst, uint32_t row_off, const uint4& lo, const uint4& hi) {
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (uint32_t c = 0; c < 8; c++) {
        uint32_t o[4];
        pf_unpack(w[c], o);
        *reinterpret_cast<uint4*>(dst + (row_off ^ (c << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

template <typename YT>
__global__ void __launch_bounds__(PF_THREADS, 1) k_gemm_i4_tc(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap qmap,
                                                                 PrefillArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t groups = a.K >> 7, num_k = a.K / PF_BK;
    uint8_t* sA = smem;                                      // [SA][128 rows][128 B]
    uint8_t* sB = sA + PF_SA * PF_A_BYTES;                   // [SB][256 rows][128 B]
    uint8_t* sQ = sB + PF_SB * PF_B_BYTES;                   // [SQ][256 rows][64 B] packed codes
    float* sS = reinterpret_cast<float*>(sQ + PF_SQ * PF_Q_BYTES);  // [SC]{ scales [CG][256], corr [CG][128] }
    uint64_t* bars = reinterpret_cast<uint64_t*>(sS + PF_SC * PF_SLOT_FLOATS);
    uint64_t* full_a = bars;
    uint64_t* empty_a = full_a + PF_SA;
    uint64_t* full_b = empty_a + PF_SA;
    uint64_t* empty_b = full_b + PF_SB;
    uint64_t* full_q = empty_b + PF_SB;
    uint64_t* empty_q = full_q + PF_SQ;
    uint64_t* sfull = empty_q + PF_SQ;
    uint64_t* sempty = sfull + PF_SC;
    uint64_t* dfull = sempty + PF_SC;
    uint64_t* dempty = dfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dempty + 2);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t m_tiles = (a.M + PF_BM - 1) / PF_BM, n_tiles = (a.N + PF_BN - 1) / PF_BN;
    const uint32_t tiles = m_tiles * n_tiles;  // numbered m-fastest; this CTA takes blockIdx.x, + gridDim.x, ...

    if (tid == 0) {
        for (uint32_t s = 0; s < PF_SA; s++) {
            pf_mbar_init(&full_a[s], 1);
            pf_mbar_init(&empty_a[s], 1);
        }
        for (uint32_t s = 0; s < PF_SB; s++) {
            pf_mbar_init(&full_b[s], 4);
            pf_mbar_init(&empty_b[s], 1);
        }
        for (uint32_t s = 0; s < PF_SQ; s++) {
            pf_mbar_init(&full_q[s], 1);
            pf_mbar_init(&empty_q[s], 4);
        }
        for (uint32_t s = 0; s < PF_SC; s++) {
            pf_mbar_init(&sfull[s], 64);
            pf_mbar_init(&sempty[s], 8);
        }
        for (uint32_t b = 0; b < 2; b++) {
            pf_mbar_init(&dfull[b], 1);
            pf_mbar_init(&dempty[b], 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // all 512 TMEM columns: two 256-column f32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(pf_smem(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 0) {
            // ---- TMA producer: per k-group one packed-code tile, per k-step one X' tile ----
            if (lane == 0) {
                uint32_t sa = 0, par = 0, it = 0, sq = 0, qpar = 0, qit = 0;
                for (uint32_t t = blockIdx.x; t < tiles && !failed; t += gridDim.x) {
                    const int32_t m0 = (int32_t)((t % m_tiles) * PF_BM), n0 = (int32_t)((t / m_tiles) * PF_BN);
                    for (uint32_t s = 0; s < num_k; s++, it++) {
                        if ((s & 1) == 0) {
                            if (qit >= PF_SQ && !pf_wait(&empty_q[sq], qpar ^ 1)) { failed = true; break; }
                            pf_mbar_expect_tx(&full_q[sq], PF_Q_BYTES);
                            pf_tma_load_2d(sQ + sq * PF_Q_BYTES, &qmap, (int32_t)(s * 8), n0, &full_q[sq]);  // x in u32 words
                            qit++;
                            if (++sq == PF_SQ) { sq = 0; qpar ^= 1; }
                        }
                        if (it >= PF_SA && !pf_wait(&empty_a[sa], par ^ 1)) { failed = true; break; }
                        pf_mbar_expect_tx(&full_a[sa], PF_A_BYTES);
                        pf_tma_load_2d(sA + sa * PF_A_BYTES, &xmap, (int32_t)(s * PF_BK), m0, &full_a[sa]);
                        if (++sa == PF_SA) { sa = 0; par ^= 1; }
                    }
                }
            }
        } else if (warp == 1) {
            // ---- MMA issuer ----
            if (lane == 0) {
                // f32 accumulate, bf16 x bf16, both K-major, N = 256, M = 128
                const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((PF_BN >> 3) << 17) | ((PF_BM >> 4) << 24);
                uint32_t sa = 0, pa = 0, sb = 0, pb = 0, gcount = 0;  // gcount: k-groups issued, over all tiles
                for (uint32_t t = blockIdx.x; t < tiles && !failed; t += gridDim.x) {
                    for (uint32_t s = 0; s < num_k; s++) {
                        const uint32_t buf = gcount & 1;
                        if ((s & 1) == 0 && gcount >= 2 && !pf_wait(&dempty[buf], ((gcount >> 1) & 1) ^ 1)) { failed = true; break; }
                        if (!pf_wait(&full_a[sa], pa) || !pf_wait(&full_b[sb], pb)) { failed = true; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t da = pf_desc(pf_smem(sA + sa * PF_A_BYTES)), db = pf_desc(pf_smem(sB + sb * PF_B_BYTES));
                        const uint32_t d = tmem_base + buf * PF_BN;
#pragma unroll
                        for (uint32_t kk = 0; kk < PF_BK / 16; kk++)
                            pf_mma(d, da + 2 * kk, db + 2 * kk, idesc, ((s & 1) | kk) ? 1u : 0u);  // +32 bytes per k16 step
                        pf_commit(&empty_a[sa]);
                        pf_commit(&empty_b[sb]);
                        if (s & 1) { pf_commit(&dfull[buf]); gcount++; }
                        if (++sa == PF_SA) { sa = 0; pa ^= 1; }
                        if (++sb == PF_SB) { sb = 0; pb ^= 1; }
                    }
                }
            }
        } else {
            // ---- scale stagers: thread j stages rows j, j + 64, ... of the tile, PF_CG groups per slot ----
            const uint32_t j = tid - 64;
            uint32_t slot = 0, par = 0, cit = 0;
            for (uint32_t t = blockIdx.x; t < tiles && !failed; t += gridDim.x) {
                const uint32_t n0 = (t / m_tiles) * PF_BN, m0 = (t % m_tiles) * PF_BM;
                for (uint32_t g0 = 0; g0 < groups; g0 += PF_CG, cit++) {
                    float sv[4][PF_CG], cv[2][PF_CG];
#pragma unroll
                    for (uint32_t i = 0; i < 4; i++) {
                        const uint32_t n = n0 + j + 64 * i;
                        const float* src = a.scales + (uint64_t)n * groups + g0;
                        if (n < a.N && g0 + PF_CG <= groups && (groups & 3u) == 0) {  // 16-byte aligned: one load
                            const float4 v = __ldg(reinterpret_cast<const float4*>(src));
                            sv[i][0] = v.x; sv[i][1] = v.y; sv[i][2] = v.z; sv[i][3] = v.w;
                        } else {
#pragma unroll
                            for (uint32_t g = 0; g < PF_CG; g++) sv[i][g] = (n < a.N && g0 + g < groups) ? __ldg(src + g) : 0.0f;
                        }
                    }
#pragma unroll
                    for (uint32_t i = 0; i < 2; i++) {
                        const uint32_t m = m0 + j + 64 * i;
#pragma unroll
                        for (uint32_t g = 0; g < PF_CG; g++)
                            cv[i][g] = (m < a.M && g0 + g < groups) ? __ldg(a.corr + (uint64_t)(g0 + g) * a.M + m) : 0.0f;
                    }
                    if (cit >= PF_SC && !pf_wait(&sempty[slot], par ^ 1)) { failed = true; break; }
                    float* S = sS + slot * PF_SLOT_FLOATS;
#pragma unroll
                    for (uint32_t g = 0; g < PF_CG; g++) {
#pragma unroll
                        for (uint32_t i = 0; i < 4; i++) S[g * PF_BN + j + 64 * i] = sv[i][g];
#pragma unroll
                        for (uint32_t i = 0; i < 2; i++)  // corrections in MMA units, negated
                            S[PF_CG * PF_BN + g * PF_BM + j + 64 * i] = -cv[i][g] * PF_RESCALE;
                    }
                    pf_mbar_arrive(&sfull[slot]);
                    if (++slot == PF_SC) { slot = 0; par ^= 1; }
                }
            }
        }
    } else if (warp < 8) {
        // ---- unpack warps: thread r owns rows r and r + 128 of the B tile ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        const uint32_t r = tid - 128;
        const uint32_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const uint32_t total = my_tiles * num_k;
        const uint32_t row_off = r * 128 + ((r & 7) << 4);
        // packed codes: row r of a slot is 64 bytes, its 16-byte chunk c sits at c ^ ((r >> 1) & 3)
        const uint32_t q_row = r * 64, q_sw = ((r >> 1) & 3) << 4;
        uint32_t sb = 0, pb = 0, sq = 0, qpar = 0;
        for (uint32_t it = 0; it < total; it++) {
            const uint32_t odd = it & 1;  // k-steps per tile are even: parity of the flat index = parity within the group
            if (!odd && !pf_wait(&full_q[sq], qpar)) { failed = true; break; }
            const uint8_t* qs = sQ + sq * PF_Q_BYTES + q_row;
            const uint4 lo0 = *reinterpret_cast<const uint4*>(qs + (((2 * odd) << 4) ^ q_sw));
            const uint4 hi0 = *reinterpret_cast<const uint4*>(qs + (((2 * odd + 1) << 4) ^ q_sw));
            const uint4 lo1 = *reinterpret_cast<const uint4*>(qs + 128 * 64 + (((2 * odd) << 4) ^ q_sw));
            const uint4 hi1 = *reinterpret_cast<const uint4*>(qs + 128 * 64 + (((2 * odd + 1) << 4) ^ q_sw));
            if (it >= PF_SB && !pf_wait(&empty_b[sb], pb ^ 1)) { failed = true; break; }
            uint8_t* dst = sB + sb * PF_B_BYTES;
            pf_unpack_row(dst, row_off, lo0, hi0);
            pf_unpack_row(dst + 128 * 128, row_off, lo1, hi1);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) {
                pf_mbar_arrive(&full_b[sb]);
                if (odd) pf_mbar_arrive(&empty_q[sq]);
            }
            if (odd && ++sq == PF_SQ) { sq = 0; qpar ^= 1; }
            if (++sb == PF_SB) { sb = 0; pb ^= 1; }
        }
    } else {
        // ---- epilogue warps: thread = accumulator row (TMEM lane), warpgroup = 128-column half ----
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
        const uint32_t quad = warp & 3, half = (warp - 8) >> 2, ml = quad * 32 + lane;
        uint32_t gcount = 0, slot = 0, spar = 0;
        for (uint32_t t = blockIdx.x; t < tiles && !failed; t += gridDim.x) {
            const uint32_t n0 = (t / m_tiles) * PF_BN + half * 128, m = (t % m_tiles) * PF_BM + ml;
            float total[128];
#pragma unroll
            for (uint32_t i = 0; i < 128; i++) total[i] = 0.0f;
            for (uint32_t g = 0; g < groups; g++, gcount++) {
                const uint32_t gi = g & (PF_CG - 1), buf = gcount & 1;
                if (gi == 0 && !pf_wait(&sfull[slot], spar)) { failed = true; break; }
                if (!pf_wait(&dfull[buf], (gcount >> 1) & 1)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // totals are kept in MMA units (2^-93): total += s * (D - corr * 2^-93), two columns per instruction
                const float* S = sS + slot * PF_SLOT_FLOATS;
                const float c = S[PF_CG * PF_BN + gi * PF_BM + ml];
                const uint64_t c2 = pf_pack2(c, c);
                const float4* sg = reinterpret_cast<const float4*>(S + gi * PF_BN + half * 128);
#pragma unroll
                for (uint32_t ch = 0; ch < 4; ch++) {
                    float v[32];
                    pf_tmem_ld32(tmem_base + ((quad * 32) << 16) + buf * PF_BN + half * 128 + ch * 32, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (uint32_t i = 0; i < 8; i++) {
                        const float4 s4 = sg[ch * 8 + i];
                        const uint32_t o = ch * 32 + 4 * i;
                        pf_fold2(total[o], total[o + 1], s4.x, s4.y, v[4 * i], v[4 * i + 1], c2);
                        pf_fold2(total[o + 2], total[o + 3], s4.z, s4.w, v[4 * i + 2], v[4 * i + 3], c2);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) pf_mbar_arrive(&dempty[buf]);
                if (gi == PF_CG - 1 || g + 1 == groups) {
                    if (lane == 0) pf_mbar_arrive(&sempty[slot]);
                    if (++slot == PF_SC) { slot = 0; spar ^= 1; }
                }
            }
            if (!failed && m < a.M && n0 < a.N) {
                YT* yrow = static_cast<YT*>(a.y) + (uint64_t)m * a.N + n0;
                const uint32_t ncols = a.N - n0 < 128u ? a.N - n0 : 128u;
#pragma unroll
                for (uint32_t i = 0; i < 128; i += 8) {
                    float v[8];
#pragma unroll
                    for (uint32_t e = 0; e < 8; e++) v[e] = total[i + e] * PF_UNSCALE;
                    if (a.vec_store && i + 8 <= ncols) {
                        if (a.bias) {
                            const float4 b0 = __ldg(reinterpret_cast<const float4*>(a.bias + n0 + i));
                            const float4 b1 = __ldg(reinterpret_cast<const float4*>(a.bias + n0 + i + 4));
                            v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                            v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                        }
                        if constexpr (sizeof(YT) == 4) {
                            *reinterpret_cast<float4*>(yrow + i) = make_float4(v[0], v[1], v[2], v[3]);
                            *reinterpret_cast<float4*>(yrow + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
                        } else {
                            uint4 o;
                            o.x = f32_to_bf16_bits(v[0]) | ((uint32_t)f32_to_bf16_bits(v[1]) << 16);
                            o.y = f32_to_bf16_bits(v[2]) | ((uint32_t)f32_to_bf16_bits(v[3]) << 16);
                            o.z = f32_to_bf16_bits(v[4]) | ((uint32_t)f32_to_bf16_bits(v[5]) << 16);
                            o.w = f32_to_bf16_bits(v[6]) | ((uint32_t)f32_to_bf16_bits(v[7]) << 16);
                            *reinterpret_cast<uint4*>(yrow + i) = o;
                        }
                    } else {
#pragma unroll
                        for (uint32_t e = 0; e < 8; e++) {
                            if (i + e < ncols) {
                                const float o = a.bias ? v[e] + __ldg(a.bias + n0 + i + e) : v[e];
                                if constexpr (sizeof(YT) == 4) yrow[i + e] = o;
                                else yrow[i + e] = f32_to_bf16_bits(o);
                            }
                        }
                    }
                }
            }
        }
    }
    if (failed) atomicExch(a.status, QB200_ERR_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}


// ---- host side ------------------------------------------------------------------------------------

bool gemm_i4_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* x) {
    if (bits != 4 || gr != 1 || gc != 128 || layout != QB200_OUT_IN || x_dtype != QB200_BF16) return false;
    if (m < 64 || m > 0x7FFFFFFF || in_dim % 128 != 0 || in_dim > 16384 || out_dim > 0x7FFFFFFF) return false;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return al(codes) && al(x);
}

// Scratch the prefill path needs for m rows: X' (m * K bf16) followed by corr (m * K/128 f32).
uint64_t gemm_i4_scratch_bytes(uint64_t m, uint64_t in_dim) {
    const uint64_t xs = (m * in_dim * 2 + 255) & ~uint64_t(255);
    return xs + m * (in_dim / 128) * 4;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

qb200_status gemm_i4_forward(const FwdArgs& f, int y_dtype, void* scratch, int32_t* status, cudaStream_t st) {
    const uint32_t M = (uint32_t)f.m, N = (uint32_t)f.out_dim, K = (uint32_t)f.in_dim, groups = K / 128;
    uint16_t* xs = static_cast<uint16_t*>(scratch);
    float* corr = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + (((uint64_t)M * K * 2 + 255) & ~uint64_t(255)));
    {
        const uint64_t units = (uint64_t)M * groups;
        k_prefill_prep<<<(uint32_t)((units + 7) / 8), 256, 0, st>>>(static_cast<const uint16_t*>(f.x), M, K, xs, corr);
        QB_CUDA_TRY(cudaGetLastError());
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(QB200_ERR_CUDA, "prefill GEMM: cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap map;
    const cuuint64_t dims[2] = {K, M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {PF_BK, PF_BM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(QB200_ERR_CUDA, "prefill GEMM: cuTensorMapEncodeTiled failed with code " + std::to_string((int)cr));
    // packed codes as a [N, K/8] u32 tensor: one box = 256 rows x 16 words (one k-group), 64-byte swizzle
    CUtensorMap qmap;
    const cuuint64_t qdims[2] = {K / 8, N};
    const cuuint64_t qstrides[1] = {(cuuint64_t)K / 2};
    const cuuint32_t qbox[2] = {16, PF_BN};
    cr = enc(&qmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(f.codes), qdims, qstrides, qbox, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(QB200_ERR_CUDA, "prefill GEMM: cuTensorMapEncodeTiled (codes) failed with code " + std::to_string((int)cr));

    PrefillArgs a;
    a.codes = static_cast<const uint32_t*>(f.codes);
    a.scales = f.scales;
    a.bias = f.bias;
    a.corr = corr;
    a.y = f.y;
    a.status = status;
    a.M = M;
    a.N = N;
    a.K = K;
    const uint32_t ysz = y_dtype == QB200_F32 ? 4 : 2;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    a.vec_store = (al16(f.y) && ((uint64_t)N * ysz) % 16 == 0 && (!f.bias || al16(f.bias))) ? 1u : 0u;
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    static int sm_count[64] = {};
    if (!sm_count[dev & 63]) QB_CUDA_TRY(cudaDeviceGetAttribute(&sm_count[dev & 63], cudaDevAttrMultiProcessorCount, dev));
    const uint32_t tiles = ((N + PF_BN - 1) / PF_BN) * ((M + PF_BM - 1) / PF_BM);
    const uint32_t grid = tiles < (uint32_t)sm_count[dev & 63] ? tiles : (uint32_t)sm_count[dev & 63];
    static bool attr_set[2][64] = {};
    if (y_dtype == QB200_F32) {
        if (!attr_set[0][dev & 63]) {
            QB_CUDA_TRY(cudaFuncSetAttribute(k_gemm_i4_tc<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM));
            attr_set[0][dev & 63] = true;
        }
        k_gemm_i4_tc<float><<<grid, PF_THREADS, PF_SMEM, st>>>(map, qmap, a);
    } else {
        if (!attr_set[1][dev & 63]) {
            QB_CUDA_TRY(cudaFuncSetAttribute(k_gemm_i4_tc<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM));
            attr_set[1][dev & 63] = true;
        }
        k_gemm_i4_tc<uint16_t><<<grid, PF_THREADS, PF_SMEM, st>>>(map, qmap, a);
    }
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

}  // namespace qb
