// Prefill GEMM (every M the decode kernel does not take: M > 16, or a wider input than it keeps on chip): Y[m, n] = sum_k X[m, k] * s[n, k/128] * q[n, k] over resident
// packed-int4 codes `[N, K/8]` with a 1x128 f32 scale grid, bf16 activations, f32 accumulation; and the same over
// int8 codes `[N, K]` with any scale grid whose tile width is a whole number of 16-k MMA steps (k_gemm_w8_tc).
// Tensor-core bound: tcgen05.mma over CTA pairs (cta_group::2) with the accumulator in TMEM.
//
// Staging (stated, and mirrored by the checker): the codes enter the tensor core as EXACT
// values q / 64 in bf16 and the activations as they are, so every product is exact in f32; a
// group's f32 scale is applied to the group's partial sum, never to a weight.  Unpacking a word
// of eight codes costs one shift, two LOP3 and four PRMT (which leave q + 8 in the low byte of
// each bf16, a subnormal worth (q + 8) * 2^-133) and four packed bf16 FMAs
// (q + 8) * 2^-133 * 2^127 - 1/8 = q / 64, exact.
//
// The WEIGHTS are the MMA's M side: a thread of the epilogue owns one weight row n, so the
// group scale s[n, g] is a per-thread scalar and the promotion total += s * D_g is one packed
// FMA per two outputs, with no shared-memory traffic.  The activations are the N side.
//
// A persistent kernel, one CTA per SM, CTAs paired in clusters of two.  A pair walks
// 256 (n) x 256 (m) output tiles, m fastest.  Per 64-k step each CTA unpacks ITS 128 weight
// rows (16 KB) and fetches ITS 128 activation rows (16 KB, TMA); one tcgen05.mma.cta_group::2
// of shape 256 x 256 x 16, issued by the pair's leader, reads both halves, so every byte staged
// in shared memory feeds two tensor cores.  Each CTA keeps its 128 x 256 f32 accumulator, twice
// (double buffered), in its own 512 TMEM columns.  Roles, by warp, in each CTA:
//   warp 0        TMA producer of activation tiles (128B swizzle)
//   warp 1        TMEM allocation; in the leader, the MMA issuer
//   warp 2        in the non-leader, tells the leader when an activation tile has landed
//   warp 3        TMA producer of packed-code tiles (64B swizzle), up to PF_SQ k-groups ahead
//   warps 4-7     unpack the packed codes from shared memory into the swizzled weight ring
//   warps 8-15    TMEM epilogue: per-group promotion into 128 f32 totals per thread, final store
// Registers are re-balanced between the roles with setmaxnreg.  All rings run across tile
// boundaries, so one tile's store overlaps the next tile's K loop.  Every wait on an mbarrier
// is bounded and reports through the handle's status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "forward.hpp"
#include "quant_math.cuh"

namespace qb {

constexpr uint32_t PF_TN = 256, PF_TM = 256, PF_BK = 64;  // pair tile; BK bf16 = one 128-byte swizzle row
constexpr uint32_t PF_S = 5;    // ring of k-steps: 128 unpacked weight rows + 128 activation rows, 128 B each
constexpr uint32_t PF_SQ = 4;   // ring of packed-code slots (128 rows x 64 B = one k-group)
constexpr uint32_t PF_THREADS = 512;
constexpr uint32_t PF_STAGE = 128 * 128, PF_Q_BYTES = 128 * 64;
constexpr uint32_t PF_Y_BYTES = 16384;  // output staging per 128-column half of the epilogue
constexpr uint32_t PF_SMEM = 1024 + 2 * PF_S * PF_STAGE + PF_SQ * PF_Q_BYTES + 2 * PF_Y_BYTES + 512;
constexpr uint32_t PF_SPIN = 1u << 22;

// ---- PTX helpers ------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t pf_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pf_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_smem(bar)), "r"(count));
}
__device__ __forceinline__ void pf_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pf_smem(bar)) : "memory");
}
// Arrive on a barrier of a CTA of this cluster (address from pf_map_to_cta).  What the arrival
// publishes has been ordered before it by its own fence (fence.proxy.async for shared-memory
// stages, tcgen05.fence for TMEM reads): a cluster-scope release here would add a full memory
// barrier per k-step, which stalled the unpack warps more than the unpacking itself.
__device__ __forceinline__ void pf_mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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
// One poll of a barrier phase (non-blocking): lets the next k-step's check overlap the MMA issue.
__device__ __forceinline__ uint32_t pf_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(pf_smem(bar)), "r"(parity)
        : "memory");
    return ok;
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ uint32_t pf_elect() {
    uint32_t e;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(e));
    return e;
}
__device__ __forceinline__ uint32_t pf_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Shared-memory address of this CTA mapped to the same offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t pf_map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void pf_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
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
// One MMA over the CTA pair: D (256 x N, 128 rows in each CTA's TMEM) (+)= A (128 rows from each
// CTA's shared memory) x B (N / 2 rows from each CTA's shared memory).  Issued by the leader.
__device__ __forceinline__ void pf_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// When the MMAs issued so far have completed, arrive on the barrier at this offset in BOTH CTAs.
__device__ __forceinline__ void pf_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     pf_smem(bar)),
                 "h"(both)
                 : "memory");
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
// (t0, t1) += (s, s) * (v0, v1) with the packed f32x2 FMA of sm_100
__device__ __forceinline__ void pf_fma2(float& t0, float& t1, uint64_t s2, float v0, float v1) {
    asm("{\n\t.reg .b64 t, v;\n\t"
        "mov.b64 t, {%0, %1};\n\tmov.b64 v, {%3, %4};\n\t"
        "fma.rn.f32x2 t, %2, v, t;\n\t"
        "mov.b64 {%0, %1}, t;\n\t}"
        : "+f"(t0), "+f"(t1)
        : "l"(s2), "f"(v0), "f"(v1));
}

struct PrefillArgs {
    const float* scales;  // [N, K/128]
    const float* bias;    // [N] or null
    void* y;              // [M, N] bf16 or f32
    int32_t* status;
    uint32_t M, N, K;
    uint32_t ksplit;     // K ranges per output tile (1: the kernel writes Y itself)
    uint32_t tma_store;  // 1 when Y's base and row pitch are multiples of 16 bytes
    // general grids (every int8 launch, int4 grids other than 1x128): the scale grid [ceil(N / gr), tc] and the scale
    // group's length in 16-k MMA steps
    uint32_t gr, tc, g16;
};

// One packed word -> eight bf16 values q / 64 in natural k order (four registers).
__device__ __forceinline__ void pf_unpack(uint32_t w, uint32_t (&r)[4]) {
    uint32_t t0, t1;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(t0) : "r"(w), "r"(0x0F0F0F0Fu), "r"(0x08080808u));       // nibbles 0,2,4,6: q + 8
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(t1) : "r"(w >> 4), "r"(0x0F0F0F0Fu), "r"(0x08080808u));  // nibbles 1,3,5,7
    // selector 8 replicates the (clear) sign bit of a byte: a zero byte for the bf16 high halves
    // (prmt.b32 in PTX: the __byte_perm intrinsic ignores the replicate bit)
    const uint32_t up = 0x7F007F00u, off = 0xBE00BE00u;  // bf16x2: 2^127, -1/8
#pragma unroll
    for (uint32_t j = 0; j < 4; j++) {
        uint32_t u;
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(u) : "r"(t0), "r"(t1), "r"(0x8480u + 0x0101u * j));
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r[j]) : "r"(u), "r"(up), "r"(off));  // subnormal in, q / 64 out
    }
}

// Unpacks the 64 codes of one row and k-step (two 16-byte loads) into the row's 128-byte line of a
// swizzled stage: chunk c lands at (row_off ^ (c << 4)).
__device__ __forceinline__ void pf_unpack_row(uint8_t* dst, uint32_t row_off, const uint4& lo, const uint4& hi) {
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (uint32_t c = 0; c < 8; c++) {
        uint32_t o[4];
        pf_unpack(w[c], o);
        *reinterpret_cast<uint4*>(dst + (row_off ^ (c << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// int8 codes: the 64 bytes of one row and k-step (four 16-byte loads) -> the row's 128-byte line of a swizzled stage.
// A byte b = q ^ 0x80 = q + 128 in the low byte of a bf16 is worth b * 2^-133 (exponent field 0 or 1), and
// b * 2^-133 * 2^127 - 2 = q / 64 exactly: one LOP3, two PRMT and two packed FMAs per four codes.
__device__ __forceinline__ void pf_widen_row(uint8_t* dst, uint32_t row_off, const uint4 (&q)[4]) {
    const uint32_t up = 0x7F007F00u, off = 0xC000C000u;  // bf16x2: 2^127, -2
#pragma unroll
    for (uint32_t c = 0; c < 8; c++) {  // chunk c: codes 8c .. 8c + 7
        const uint4& v = q[c >> 1];
        const uint32_t w0 = ((c & 1) ? v.z : v.x) ^ 0x80808080u, w1 = ((c & 1) ? v.w : v.y) ^ 0x80808080u;
        uint32_t o[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; j++) {
            uint32_t u;
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(u) : "r"(j < 2 ? w0 : w1), "r"(0u), "r"((j & 1) ? 0x4342u : 0x4140u));
            asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[j]) : "r"(u), "r"(up), "r"(off));
        }
        *reinterpret_cast<uint4*>(dst + (row_off ^ (c << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// The kernel's body for packed int4 (BITS = 4) and int8 (BITS = 8) codes.  A 64-byte slot of the code ring is one
// k-group of 128 int4 codes per row or one k-step of 64 int8 codes.  GEN = false is the int4 1x128 grid: a scale
// group is a slot.  GEN = true is any grid whose tile width is a multiple of 16: a scale group is `g16` MMA steps
// of 16 k, the issuer closes an accumulator every g16 steps wherever that falls, and the epilogue reads row n / gr
// of the grid.
template <typename YT, bool SPLIT, uint32_t BITS, bool GEN>
__device__ __forceinline__ void gemm_codes_tc(uint8_t* smem_raw, const CUtensorMap& xmap, const CUtensorMap& qmap,
                                              const CUtensorMap& ymap, const PrefillArgs& a) {
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // a work unit is one output tile over one of `ksplit` equal K ranges (whole scale groups); with ksplit > 1 the
    // units' f32 partial tiles go to a workspace [ksplit, M, N] that a second kernel folds
    const uint32_t ksplit = SPLIT ? a.ksplit : 1u;  // the unsplit instantiation folds every K-range term away
    // per unit: num_k k-steps of 64 and `groups` scale groups; a row of the scale grid holds row_groups scales
    static_assert(GEN || BITS == 4, "int8 codes take the general issuer");
    const uint32_t row_groups = GEN ? a.tc : a.K >> 7;
    const uint32_t num_k = BITS == 4 ? 2 * ((a.K >> 7) / ksplit) : (a.K >> 6) / ksplit;
    const uint32_t groups = GEN ? num_k * 4 / a.g16 : num_k >> 1;
    uint8_t* sA = smem;                  // [S][128 weight rows][128 B], unpacked bf16
    uint8_t* sX = sA + PF_S * PF_STAGE;  // [S][128 activation rows][128 B]
    uint8_t* sQ = sX + PF_S * PF_STAGE;  // [SQ][128 weight rows][64 B], packed codes
    uint8_t* sY = sQ + PF_SQ * PF_Q_BYTES;  // [2 halves][16 KB] output staging for the TMA store
    uint64_t* bars = reinterpret_cast<uint64_t*>(sY + 2 * PF_Y_BYTES);
    uint64_t* full = bars;               // leader: a k-step's operands are complete in BOTH CTAs
    uint64_t* full_x = full + PF_S;      // non-leader: its own activation tile has landed (TMA)
    uint64_t* empty = full_x + PF_S;     // the MMAs that read the stage are done (both CTAs)
    uint64_t* full_q = empty + PF_S;     // packed-code slot has landed (TMA)
    uint64_t* empty_q = full_q + PF_SQ;  // unpack warps are done with the slot
    uint64_t* dfull = empty_q + PF_SQ;   // a group's accumulator is complete (both CTAs)
    uint64_t* dempty = dfull + 2;        // leader: both CTAs' epilogues have read the accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dempty + 2);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = pf_cluster_rank();  // 0: the pair's leader
    const uint32_t pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    const uint32_t m_tiles = (a.M + PF_TM - 1) / PF_TM, n_tiles = (a.N + PF_TN - 1) / PF_TN;
    const uint32_t tiles = m_tiles * n_tiles * ksplit;  // units: K range fastest, then m; this pair takes pair, pair + pairs, ...
    const uint32_t my_tiles = pair < tiles ? (tiles - pair + pairs - 1) / pairs : 0;
    const uint32_t total = my_tiles * num_k;   // k-steps this CTA goes through

    if (tid == 0) {
        for (uint32_t s = 0; s < PF_S; s++) {
            // the leader's TMA (with its bytes), the non-leader's "landed" message, four unpack warps in each CTA
            pf_mbar_init(&full[s], 10);
            pf_mbar_init(&full_x[s], 1);
            pf_mbar_init(&empty[s], 1);
        }
        for (uint32_t s = 0; s < PF_SQ; s++) {
            pf_mbar_init(&full_q[s], 1);
            pf_mbar_init(&empty_q[s], 4);
        }
        for (uint32_t b = 0; b < 2; b++) {
            pf_mbar_init(&dfull[b], 1);
            pf_mbar_init(&dempty[b], 16);  // eight epilogue warps in each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // all 512 TMEM columns of this CTA: two 256-column f32 accumulators
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(pf_smem(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    pf_cluster_sync();  // both CTAs' barriers are initialised before either arrives on the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 0) {
            // ---- TMA producer of activation tiles, one per k-step ----
            if (lane == 0) {
                uint64_t* landed = rank == 0 ? full : full_x;  // the leader's tile counts towards `full` directly
                uint32_t st = 0, par = 0, it = 0;
                for (uint32_t t = pair; t < tiles && !failed; t += pairs) {
                    const uint32_t tile = t / ksplit, k_first = (t % ksplit) * num_k;
                    const int32_t x_row = (int32_t)((tile % m_tiles) * PF_TM + rank * 128);
                    for (uint32_t s = 0; s < num_k; s++, it++) {
                        if (it >= PF_S && !pf_wait(&empty[st], par ^ 1)) { failed = true; break; }
                        pf_mbar_expect_tx(&landed[st], PF_STAGE);
                        pf_tma_load_2d(sX + st * PF_STAGE, &xmap, (int32_t)((k_first + s) * PF_BK), x_row, &landed[st]);
                        if (++st == PF_S) { st = 0; par ^= 1; }
                    }
                }
            }
        } else if (warp == 1) {
            // ---- MMA issuer (the pair's leader only) ----
            // The whole warp runs the loop, so descriptors and addresses stay warp-uniform (an MMA issued
            // from divergent code pays for moving each operand to the uniform registers); one elected
            // lane issues.  The next k-step's barrier is polled before this step's MMAs are issued, so the
            // poll's latency is hidden behind them.
            if constexpr (GEN) {
              if (rank == 0) {
                // scale groups of g16 MMA steps, whatever their position in the k-steps: the accumulator changes
                // where a group ends, and a k-step's stage is released after its fourth MMA
                const uint32_t elected = pf_elect();
                const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((PF_TM >> 3) << 17) | ((PF_TN >> 4) << 24);
                uint32_t st = 0, par = 0, gcount = 0, in_group = 0, ready = 0;
                uint32_t dready = 0;  // the accumulator of the next group to start was seen read out by an early poll
                for (uint32_t it = 0; it < total && !failed; it++) {
                    if (!ready && !pf_wait(&full[st], par)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st1 = st + 1 == PF_S ? 0 : st + 1, par1 = st + 1 == PF_S ? par ^ 1 : par;
                    ready = it + 1 < total ? pf_test(&full[st1], par1) : 0;
                    // a group that starts in the next k-step (groups longer than a k-step): its accumulator is polled
                    // now, behind this k-step's MMAs
                    const uint32_t gn = gcount + (in_group ? 1u : 0u);
                    if (!dready && gn >= 2) dready = pf_test(&dempty[gn & 1], ((gn >> 1) & 1) ^ 1);
                    const uint64_t da = pf_desc(pf_smem(sA + st * PF_STAGE)), db = pf_desc(pf_smem(sX + st * PF_STAGE));
#pragma unroll
                    for (uint32_t kk = 0; kk < PF_BK / 16; kk++) {
                        const uint32_t buf = gcount & 1;
                        if (in_group == 0 && gcount >= 2) {
                            if (!dready && !pf_wait(&dempty[buf], ((gcount >> 1) & 1) ^ 1)) { failed = true; break; }
                            dready = 0;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        if (elected) pf_mma_pair(tmem_base + buf * PF_TM, da + 2 * kk, db + 2 * kk, idesc, in_group ? 1u : 0u);
                        if (++in_group == a.g16) {
                            if (elected) pf_commit_pair(&dfull[buf]);
                            in_group = 0;
                            gcount++;
                        }
                    }
                    if (failed) break;
                    if (elected) pf_commit_pair(&empty[st]);
                    st = st1;
                    par = par1;
                }
              }
            } else if (rank == 0) {
                const uint32_t elected = pf_elect();
                // f32 accumulate, bf16 x bf16, both K-major, N = 256, M = 256 over the pair
                const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((PF_TM >> 3) << 17) | ((PF_TN >> 4) << 24);
                uint32_t st = 0, par = 0, gcount = 0;  // gcount: k-groups issued, over all tiles
                uint32_t ready = 0;                    // this k-step's `full` phase was seen complete by the early poll
                uint32_t dready = 0;                   // the same for the next k-group's accumulator
                for (uint32_t it = 0; it < total; it++) {
                    const uint32_t odd = it & 1, buf = gcount & 1;
                    if (!odd && gcount >= 2 && !dready && !pf_wait(&dempty[buf], ((gcount >> 1) & 1) ^ 1)) { failed = true; break; }
                    if (!ready && !pf_wait(&full[st], par)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st1 = st + 1 == PF_S ? 0 : st + 1, par1 = st + 1 == PF_S ? par ^ 1 : par;
                    ready = it + 1 < total ? pf_test(&full[st1], par1) : 0;
                    // at a group's second k-step, poll for the accumulator the next group will use
                    dready = (odd && gcount >= 1) ? pf_test(&dempty[buf ^ 1], (((gcount + 1) >> 1) & 1) ^ 1) : 0;
                    const uint64_t da = pf_desc(pf_smem(sA + st * PF_STAGE)), db = pf_desc(pf_smem(sX + st * PF_STAGE));
                    const uint32_t d = tmem_base + buf * PF_TM;
                    if (elected) {
#pragma unroll
                        for (uint32_t kk = 0; kk < PF_BK / 16; kk++)
                            pf_mma_pair(d, da + 2 * kk, db + 2 * kk, idesc, (odd | kk) ? 1u : 0u);  // +32 bytes per k16 step
                        pf_commit_pair(&empty[st]);
                        if (odd) pf_commit_pair(&dfull[buf]);
                    }
                    gcount += odd;
                    st = st1;
                    par = par1;
                }
            }
        } else if (warp == 2) {
            // ---- non-leader: pass "activation tile landed" on to the leader's barrier ----
            if (lane == 0 && rank == 1) {
                const uint32_t remote = pf_map_to_cta(pf_smem(&full[0]), 0);
                uint32_t st = 0, par = 0;
                for (uint32_t it = 0; it < total; it++) {
                    if (!pf_wait(&full_x[st], par)) { failed = true; break; }
                    pf_mbar_arrive_cluster(remote + st * 8);
                    if (++st == PF_S) { st = 0; par ^= 1; }
                }
            }
        } else if (warp == 3) {
            // ---- TMA producer of packed-code tiles, one per k-group; runs ahead of the activation ring ----
            if (lane == 0) {
                uint32_t sq = 0, pq = 0, qit = 0;
                // a slot is 64 bytes of each row: one k-group of packed int4 (x in u32 words), one k-step of int8 (x in bytes)
                const uint32_t slots = BITS == 4 ? num_k >> 1 : num_k, x_step = BITS == 4 ? 16u : 64u;
                for (uint32_t t = pair; t < tiles && !failed; t += pairs) {
                    const uint32_t tile = t / ksplit, g_first = (t % ksplit) * slots;
                    const int32_t q_row = (int32_t)((tile / m_tiles) * PF_TN + rank * 128);
                    for (uint32_t g = 0; g < slots; g++, qit++) {
                        if (qit >= PF_SQ && !pf_wait(&empty_q[sq], pq ^ 1)) { failed = true; break; }
                        pf_mbar_expect_tx(&full_q[sq], PF_Q_BYTES);
                        pf_tma_load_2d(sQ + sq * PF_Q_BYTES, &qmap, (int32_t)((g_first + g) * x_step), q_row, &full_q[sq]);
                        if (++sq == PF_SQ) { sq = 0; pq ^= 1; }
                    }
                }
            }
        }
    } else if (warp < 8) {
        // ---- unpack warps: thread r owns weight row r of this CTA's half ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        const uint32_t r = tid - 128;
        const uint32_t row_off = r * 128 + ((r & 7) << 4);
        // packed codes: row r of a slot is 64 bytes, its 16-byte chunk c sits at c ^ ((r >> 1) & 3)
        const uint32_t q_row = r * 64, q_sw = ((r >> 1) & 3) << 4;
        const uint32_t remote_full = pf_map_to_cta(pf_smem(&full[0]), 0);
        uint32_t st = 0, par = 0, sq = 0, pq = 0;
        if constexpr (BITS == 8) {
            // a slot of 64 codes per row is one k-step; two per iteration (one fence and one round of barrier
            // latencies for both), a single one when the count is odd
            auto ring_next = [](uint32_t& i, uint32_t& p, uint32_t n) { if (++i == n) { i = 0; p ^= 1; } };
            uint32_t it = 0;
            for (; it + 1 < total; it += 2) {
                uint32_t sq1 = sq, pq1 = pq, st1 = st, par1 = par;
                ring_next(sq1, pq1, PF_SQ);
                ring_next(st1, par1, PF_S);
                uint4 q0[4], q1[4];
                if (!pf_wait(&full_q[sq], pq)) { failed = true; break; }
#pragma unroll
                for (uint32_t c = 0; c < 4; c++) q0[c] = *reinterpret_cast<const uint4*>(sQ + sq * PF_Q_BYTES + q_row + ((c << 4) ^ q_sw));
                if (!pf_wait(&full_q[sq1], pq1)) { failed = true; break; }
#pragma unroll
                for (uint32_t c = 0; c < 4; c++) q1[c] = *reinterpret_cast<const uint4*>(sQ + sq1 * PF_Q_BYTES + q_row + ((c << 4) ^ q_sw));
                if (it >= PF_S && !pf_wait(&empty[st], par ^ 1)) { failed = true; break; }
                if (it + 1 >= PF_S && !pf_wait(&empty[st1], par1 ^ 1)) { failed = true; break; }
                pf_widen_row(sA + st * PF_STAGE, row_off, q0);
                pf_widen_row(sA + st1 * PF_STAGE, row_off, q1);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    pf_mbar_arrive_cluster(remote_full + st * 8);
                    pf_mbar_arrive_cluster(remote_full + st1 * 8);
                    pf_mbar_arrive(&empty_q[sq]);
                    pf_mbar_arrive(&empty_q[sq1]);
                }
                sq = sq1; pq = pq1; st = st1; par = par1;
                ring_next(sq, pq, PF_SQ);
                ring_next(st, par, PF_S);
            }
            if (it < total && !failed) {
                uint4 q[4];
                if (!pf_wait(&full_q[sq], pq)) failed = true;
#pragma unroll
                for (uint32_t c = 0; c < 4; c++) q[c] = *reinterpret_cast<const uint4*>(sQ + sq * PF_Q_BYTES + q_row + ((c << 4) ^ q_sw));
                if (!failed && it >= PF_S && !pf_wait(&empty[st], par ^ 1)) failed = true;
                if (!failed) {
                    pf_widen_row(sA + st * PF_STAGE, row_off, q);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        pf_mbar_arrive_cluster(remote_full + st * 8);
                        pf_mbar_arrive(&empty_q[sq]);
                    }
                }
            }
        } else {
        // one k-group (two k-steps, one packed-code slot) per iteration: one fence and one round of
        // barrier latencies for 16 independent words per thread
        for (uint32_t it = 0; it < total; it += 2) {
            if (!pf_wait(&full_q[sq], pq)) { failed = true; break; }
            const uint8_t* qs = sQ + sq * PF_Q_BYTES + q_row;
            uint4 q[4];
#pragma unroll
            for (uint32_t c = 0; c < 4; c++) q[c] = *reinterpret_cast<const uint4*>(qs + ((c << 4) ^ q_sw));
            const uint32_t st1 = st + 1 == PF_S ? 0 : st + 1, par1 = st + 1 == PF_S ? par ^ 1 : par;
            if (it >= PF_S && !pf_wait(&empty[st], par ^ 1)) { failed = true; break; }
            if (it + 1 >= PF_S && !pf_wait(&empty[st1], par1 ^ 1)) { failed = true; break; }
            pf_unpack_row(sA + st * PF_STAGE, row_off, q[0], q[1]);
            pf_unpack_row(sA + st1 * PF_STAGE, row_off, q[2], q[3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) {
                pf_mbar_arrive_cluster(remote_full + st * 8);
                pf_mbar_arrive_cluster(remote_full + st1 * 8);
                pf_mbar_arrive(&empty_q[sq]);
            }
            if (++sq == PF_SQ) { sq = 0; pq ^= 1; }
            st = st1 + 1 == PF_S ? 0 : st1 + 1;
            par = st1 + 1 == PF_S ? par1 ^ 1 : par1;
        }
        }
    } else {
        // ---- epilogue warps: thread = weight row (TMEM lane), warpgroup = 128-column half of the m range ----
        asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
        const uint32_t quad = warp & 3, half = (warp - 8) >> 2, ml = quad * 32 + lane;
        const uint32_t remote_dempty = pf_map_to_cta(pf_smem(&dempty[0]), 0);
        // a unit's scales start on a 16-byte boundary (rows of whole 16-byte units from an aligned base)
        const bool vec_scales = ((row_groups | groups) & 3u) == 0 && (reinterpret_cast<uintptr_t>(a.scales) & 15u) == 0;
        const bool issuer = quad == 0 && lane == 0;  // the thread of this half that issues its TMA stores
        constexpr uint32_t ROWS = PF_Y_BYTES / 2 / (128 * sizeof(YT));  // activation rows per staging pass (two buffers)
        YT* stage = reinterpret_cast<YT*>(sY + half * PF_Y_BYTES);
        uint32_t gcount = 0;
        for (uint32_t t = pair; t < tiles && !failed; t += pairs) {
            const uint32_t tile = t / ksplit, ks = t % ksplit;
            const uint32_t n_cta = (tile / m_tiles) * PF_TN + rank * 128, n = n_cta + ml;
            const uint32_t m0 = (tile % m_tiles) * PF_TM + half * 128;
            const bool n_ok = n < a.N;
            const float* sp = a.scales + (uint64_t)(GEN ? (n_ok ? n : 0) / a.gr : (n_ok ? n : 0)) * row_groups + ks * groups;
            float total[128];
#pragma unroll
            for (uint32_t i = 0; i < 128; i++) total[i] = 0.0f;
            float nxt[4];
            auto load_scales = [&](uint32_t g0) {  // four groups of scales, times 64 (the codes enter as q / 64)
                if (vec_scales && g0 < groups) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(sp + g0));
                    nxt[0] = v.x; nxt[1] = v.y; nxt[2] = v.z; nxt[3] = v.w;
                } else {
#pragma unroll
                    for (uint32_t j = 0; j < 4; j++) nxt[j] = g0 + j < groups ? __ldg(sp + g0 + j) : 0.0f;
                }
#pragma unroll
                for (uint32_t j = 0; j < 4; j++) nxt[j] = n_ok ? nxt[j] * 64.0f : 0.0f;
            };
            load_scales(0);
            for (uint32_t g0 = 0; g0 < groups && !failed; g0 += 4) {
                const float cur[4] = {nxt[0], nxt[1], nxt[2], nxt[3]};
                load_scales(g0 + 4);
#pragma unroll
                for (uint32_t gi = 0; gi < 4; gi++) {
                    if (g0 + gi >= groups) break;
                    const uint32_t buf = gcount & 1;
                    if (!pf_wait(&dfull[buf], (gcount >> 1) & 1)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t s2 = pf_pack2(cur[gi], cur[gi]);
#pragma unroll
                    for (uint32_t ch = 0; ch < 4; ch++) {
                        float v[32];
                        pf_tmem_ld32(tmem_base + ((quad * 32) << 16) + buf * PF_TM + half * 128 + ch * 32, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (uint32_t i = 0; i < 16; i++)
                            pf_fma2(total[ch * 32 + 2 * i], total[ch * 32 + 2 * i + 1], s2, v[2 * i], v[2 * i + 1]);
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) pf_mbar_arrive_cluster(remote_dempty + buf * 8);
                    gcount++;
                }
            }
            if (failed) break;
            const float b = (a.bias && n_ok) ? __ldg(a.bias + n) : 0.0f;
            if (a.tma_store) {
                // column i of the accumulator is activation row m0 + i: ROWS rows at a time go through one of this
                // half's two staging buffers as [row][128 n] and leave by a TMA store, which clips at the edges of Y
#pragma unroll
                for (uint32_t p = 0; p < 128 / ROWS; p++) {
                    YT* buf = stage + (p & 1) * (ROWS * 128);
                    if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // the store before last has read `buf`
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
#pragma unroll
                    for (uint32_t i = 0; i < ROWS; i += 2) {
                        const float v0 = total[p * ROWS + i] + b, v1 = total[p * ROWS + i + 1] + b;
                        if constexpr (sizeof(YT) == 4) {
                            buf[i * 128 + ml] = v0;
                            buf[(i + 1) * 128 + ml] = v1;
                        } else {
                            uint16_t h0, h1;
                            asm("{\n\t.reg .b32 t;\n\tcvt.rn.bf16x2.f32 t, %3, %2;\n\tmov.b32 {%0, %1}, t;\n\t}" : "=h"(h0), "=h"(h1) : "f"(v0), "f"(v1));
                            buf[i * 128 + ml] = h0;
                            buf[(i + 1) * 128 + ml] = h1;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
                    if (issuer) {
                        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&ymap),
                                     "r"((int32_t)n_cta), "r"((int32_t)(m0 + p * ROWS)), "r"((int32_t)ks), "r"(pf_smem(buf))
                                     : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            } else if (n_ok) {  // rows of Y that TMA cannot address: lanes are consecutive n, 2 or 4 bytes each
                YT* yp = static_cast<YT*>(a.y) + (uint64_t)m0 * a.N + n;
#pragma unroll
                for (uint32_t i = 0; i < 128; i++) {
                    if (m0 + i < a.M) {
                        const float v = total[i] + b;
                        if constexpr (sizeof(YT) == 4) yp[(uint64_t)i * a.N] = v;
                        else yp[(uint64_t)i * a.N] = f32_to_bf16_bits(v);
                    }
                }
            }
        }
        if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores complete before shared memory goes away
    }
    if (failed) atomicExch(a.status, QB200_ERR_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    pf_cluster_sync();  // neither CTA leaves while the other may still signal its barriers
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}

template <typename YT, bool SPLIT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PF_THREADS, 1)
    k_gemm_i4_tc(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap qmap,
                 const __grid_constant__ CUtensorMap ymap, const PrefillArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    gemm_codes_tc<YT, SPLIT, 4, false>(smem_raw, xmap, qmap, ymap, a);
}

template <typename YT, bool SPLIT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PF_THREADS, 1)
    k_gemm_i4g_tc(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap qmap,
                  const __grid_constant__ CUtensorMap ymap, const PrefillArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    gemm_codes_tc<YT, SPLIT, 4, true>(smem_raw, xmap, qmap, ymap, a);
}

template <typename YT, bool SPLIT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PF_THREADS, 1)
    k_gemm_w8_tc(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap qmap,
                 const __grid_constant__ CUtensorMap ymap, const PrefillArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    gemm_codes_tc<YT, SPLIT, 8, true>(smem_raw, xmap, qmap, ymap, a);
}

// Folds the K ranges' partial tiles: y[m, n] = sum_s ws[s, m, n] (+ bias[n]), four outputs per thread.
template <typename YT>
__global__ void __launch_bounds__(256) k_gemm_i4_fold(const float* __restrict__ ws, uint32_t ksplit, uint64_t mn, uint32_t N,
                                                      const float* __restrict__ bias, YT* __restrict__ y) {
    const uint64_t i = ((uint64_t)blockIdx.x * 256 + threadIdx.x) * 4;  // N is a multiple of 4 on this path
    if (i >= mn) return;
    float4 v = *reinterpret_cast<const float4*>(ws + i);
    for (uint32_t s = 1; s < ksplit; s++) {
        const float4 e = *reinterpret_cast<const float4*>(ws + s * mn + i);
        v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
    }
    if (bias) {
        const float4 b = *reinterpret_cast<const float4*>(bias + (uint32_t)(i % N));
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    }
    if constexpr (sizeof(YT) == 4) {
        *reinterpret_cast<float4*>(y + i) = v;
    } else {
        uint2 o;
        o.x = f32_to_bf16_bits(v.x) | ((uint32_t)f32_to_bf16_bits(v.y) << 16);
        o.y = f32_to_bf16_bits(v.z) | ((uint32_t)f32_to_bf16_bits(v.w) << 16);
        *reinterpret_cast<uint2*>(y + i) = o;
    }
}

// ---- host side ------------------------------------------------------------------------------------

// The int4 grid with a kernel instantiation of its own (a scale group is one 64-byte slot of codes).
static bool int4_special(uint64_t gr, uint64_t gc) { return gr == 1 && gc == 128; }

// K ranges per output tile: when the output has fewer 256 x 256 tiles than the device has SM pairs, the K loop is cut
// into equal runs of whole scale groups (at least four each) so that the idle pairs take a share.
static uint32_t gemm_i4_ksplit(uint64_t m, uint64_t out_dim, uint64_t in_dim, const void* bias) {
    const uint64_t tiles = ((out_dim + PF_TN - 1) / PF_TN) * ((m + PF_TM - 1) / PF_TM), pairs = 74;
    const uint32_t groups = (uint32_t)(in_dim / 128);
    if (tiles * 2 > pairs || out_dim % 4 != 0 || (bias && (reinterpret_cast<uintptr_t>(bias) & 15u))) return 1;
    uint32_t best = 1;
    for (uint32_t s = 2; s <= pairs / tiles && s <= groups / 4; s++)
        if (groups % s == 0) best = s;
    return best;
}


bool gemm_i4_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* x) {
    if (bits != 4 || layout != QB200_OUT_IN || x_dtype != QB200_BF16 || gr == 0 || gr > 0x7FFFFFFF) return false;
    if (m == 0 || m > 0x7FFFFFFF || in_dim % 128 != 0 || in_dim > (1u << 20) || out_dim > 0x7FFFFFFF) return false;
    if (!int4_special(gr, gc)) {
        // other grids: tiles of whole 16-k steps that divide the row (or span it); the smallest batches keep the generic
        // kernel (one [4096, 4096] layer: 9 us at one row and 2 us more per row, against 18 - 29 us here at any batch)
        if (m <= 8 || (gc < in_dim && (gc % 16 != 0 || in_dim % gc != 0))) return false;
    }
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return al(codes) && al(x);
}

// General grids: a scale group's length in MMA steps of 16 k (a tile wider than the row is the whole row).
static uint32_t gemm_gen_g16(uint64_t gc, uint64_t in_dim) { return (uint32_t)((gc >= in_dim ? in_dim : gc) / 16); }

// The same for general grids: equal runs of whole k-steps (at least four each; whole 128-k slots for int4 codes) that
// are also whole scale groups.
static uint32_t gemm_gen_ksplit(uint32_t bits, uint64_t m, uint64_t out_dim, uint64_t in_dim, uint64_t gc, const void* bias) {
    const uint64_t tiles = ((out_dim + PF_TN - 1) / PF_TN) * ((m + PF_TM - 1) / PF_TM), pairs = 74;
    const uint32_t steps = (uint32_t)(in_dim / PF_BK), g16 = gemm_gen_g16(gc, in_dim);
    if (tiles * 2 > pairs || out_dim % 4 != 0 || (bias && (reinterpret_cast<uintptr_t>(bias) & 15u))) return 1;
    uint32_t best = 1;
    for (uint32_t s = 2; s <= pairs / tiles && s <= steps / 4; s++)
        if (steps % s == 0 && (steps / s * 4) % g16 == 0 && (bits == 8 || (steps / s) % 2 == 0)) best = s;
    return best;
}

bool gemm_i8_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* x) {
    if (bits != 8 || layout != QB200_OUT_IN || x_dtype != QB200_BF16 || gr == 0 || gr > 0x7FFFFFFF) return false;
    // up to four rows the generic kernel is the faster one (the decode kernel takes what it can before this is asked)
    if (m <= 4 || m > 0x7FFFFFFF || in_dim % PF_BK != 0 || in_dim > (1u << 20) || out_dim > 0x7FFFFFFF) return false;
    if (gc < in_dim && (gc % 16 != 0 || in_dim % gc != 0)) return false;  // whole groups of whole MMA steps
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return al(codes) && al(x);
}

uint64_t gemm_i8_scratch_bytes(uint64_t m, uint64_t in_dim, uint64_t out_dim, uint64_t gc, const void* bias) {
    const uint32_t ks = gemm_gen_ksplit(8, m, out_dim, in_dim, gc, bias);
    return ks > 1 ? (uint64_t)ks * m * out_dim * 4 : 0;
}

// Scratch: only the workspace of partial tiles when the K loop is split ([ksplit, m, out] f32).
uint64_t gemm_i4_scratch_bytes(uint64_t m, uint64_t in_dim, uint64_t out_dim, uint64_t gr, uint64_t gc, const void* bias) {
    const uint32_t ks = int4_special(gr, gc) ? gemm_i4_ksplit(m, out_dim, in_dim, bias) : gemm_gen_ksplit(4, m, out_dim, in_dim, gc, bias);
    return ks > 1 ? (uint64_t)ks * m * out_dim * 4 : 0;
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

// variant: 0 = int4 1x128, 1 = int4 general grid, 2 = int8
template <typename YT, bool SPLIT>
static qb200_status launch_prefill(int variant, uint32_t grid, const CUtensorMap& xmap, const CUtensorMap& qmap,
                                   const CUtensorMap& ymap, const PrefillArgs& a, int dev, cudaStream_t st) {
    static bool attr_set[3][64] = {};
    auto kern = variant == 2 ? k_gemm_w8_tc<YT, SPLIT> : variant == 1 ? k_gemm_i4g_tc<YT, SPLIT> : k_gemm_i4_tc<YT, SPLIT>;
    if (!attr_set[variant][dev & 63]) {
        QB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM));
        attr_set[variant][dev & 63] = true;
    }
    kern<<<grid, PF_THREADS, PF_SMEM, st>>>(xmap, qmap, ymap, a);
    return QB200_OK;
}

static qb200_status gemm_tc_forward(const FwdArgs& f, uint32_t bits, int y_dtype, void* scratch, int32_t* status, cudaStream_t st) {
    const uint32_t M = (uint32_t)f.m, N = (uint32_t)f.out_dim, K = (uint32_t)f.in_dim;
    const bool gen = bits == 8 || !int4_special(f.gr, f.gc);
    const uint32_t ksplit = !scratch ? 1 : gen ? gemm_gen_ksplit(bits, M, N, K, f.gc, f.bias) : gemm_i4_ksplit(M, N, K, f.bias);
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(QB200_ERR_CUDA, "prefill GEMM: cuTensorMapEncodeTiled is not available from this driver");
    // activations as a [M, K] bf16 tensor: one box = 128 rows x 64 elements (one 128-byte swizzle row each)
    CUtensorMap xmap;
    const cuuint64_t dims[2] = {K, M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {PF_BK, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(f.x), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(QB200_ERR_CUDA, "prefill GEMM: cuTensorMapEncodeTiled failed with code " + std::to_string((int)cr));
    // packed codes as a [N, K/8] u32 tensor: one box = 128 rows x 16 words (one k-group), 64-byte swizzle;
    // int8 codes as a [N, K] byte tensor: one box = 128 rows x 64 bytes (one k-step)
    CUtensorMap qmap;
    const cuuint64_t qdims[2] = {bits == 8 ? K : K / 8, N};
    const cuuint64_t qstrides[1] = {bits == 8 ? (cuuint64_t)K : (cuuint64_t)K / 2};
    const cuuint32_t qbox[2] = {bits == 8 ? 64u : 16u, 128};
    cr = enc(&qmap, bits == 8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(f.codes), qdims, qstrides, qbox, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(QB200_ERR_CUDA, "prefill GEMM: cuTensorMapEncodeTiled (codes) failed with code " + std::to_string((int)cr));

    // Y as a [1, M, N] tensor (the workspace of partial tiles as [ksplit, M, N] f32 when the K loop is split): one box =
    // (8 KB / 128 / element size) rows x 128 columns of one plane
    const int k_dtype = ksplit > 1 ? (int)QB200_F32 : y_dtype;  // what the GEMM kernel itself writes
    void* k_out = ksplit > 1 ? scratch : f.y;
    const uint32_t ysz = k_dtype == QB200_F32 ? 4 : 2;
    const bool tma_store = (reinterpret_cast<uintptr_t>(k_out) & 15u) == 0 && ((uint64_t)N * ysz) % 16 == 0;
    CUtensorMap ymap = xmap;  // a valid map either way; unused without tma_store
    if (tma_store) {
        const cuuint64_t ydims[3] = {N, M, ksplit};
        const cuuint64_t ystrides[2] = {(cuuint64_t)N * ysz, (cuuint64_t)M * N * ysz};
        const cuuint32_t ybox[3] = {128, PF_Y_BYTES / 2 / (128 * ysz), 1};
        const cuuint32_t estr3[3] = {1, 1, 1};
        cr = enc(&ymap, k_dtype == QB200_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, k_out, ydims,
                 ystrides, ybox, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(QB200_ERR_CUDA, "prefill GEMM: cuTensorMapEncodeTiled (output) failed with code " + std::to_string((int)cr));
    }

    PrefillArgs a;
    a.tma_store = tma_store ? 1u : 0u;
    a.scales = f.scales;
    a.bias = ksplit > 1 ? nullptr : f.bias;  // the fold kernel adds it
    a.y = k_out;
    a.ksplit = ksplit;
    a.status = status;
    a.M = M;
    a.N = N;
    a.K = K;
    a.gr = (uint32_t)f.gr;
    a.tc = (uint32_t)f.tc;
    a.g16 = gen ? gemm_gen_g16(f.gc, K) : 8;
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    static int sm_count[64] = {};
    if (!sm_count[dev & 63]) QB_CUDA_TRY(cudaDeviceGetAttribute(&sm_count[dev & 63], cudaDevAttrMultiProcessorCount, dev));
    const uint32_t tiles = ((N + PF_TN - 1) / PF_TN) * ((M + PF_TM - 1) / PF_TM) * ksplit;
    const uint32_t max_pairs = (uint32_t)sm_count[dev & 63] / 2;
    const uint32_t grid = 2 * (tiles < max_pairs ? tiles : max_pairs);  // one CTA per SM, in clusters of two
    qb200_status ls;
    const int variant = bits == 8 ? 2 : gen ? 1 : 0;
    if (k_dtype != QB200_F32) ls = launch_prefill<uint16_t, false>(variant, grid, xmap, qmap, ymap, a, dev, st);
    else if (ksplit > 1) ls = launch_prefill<float, true>(variant, grid, xmap, qmap, ymap, a, dev, st);
    else ls = launch_prefill<float, false>(variant, grid, xmap, qmap, ymap, a, dev, st);
    if (ls) return ls;
    QB_CUDA_TRY(cudaGetLastError());
    if (ksplit > 1) {
        if (!tma_store) return fail(QB200_ERR_CUDA, "prefill GEMM: the split-K workspace is not 16-byte aligned");
        const uint64_t mn = (uint64_t)M * N;
        const uint32_t blocks = (uint32_t)((mn / 4 + 255) / 256);
        if (y_dtype == QB200_F32)
            k_gemm_i4_fold<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(scratch), ksplit, mn, N, f.bias, static_cast<float*>(f.y));
        else
            k_gemm_i4_fold<uint16_t><<<blocks, 256, 0, st>>>(static_cast<const float*>(scratch), ksplit, mn, N, f.bias,
                                                             static_cast<uint16_t*>(f.y));
        QB_CUDA_TRY(cudaGetLastError());
    }
    return QB200_OK;
}

qb200_status gemm_i4_forward(const FwdArgs& f, int y_dtype, void* scratch, int32_t* status, cudaStream_t st) {
    return gemm_tc_forward(f, 4, y_dtype, scratch, status, st);
}

qb200_status gemm_i8_forward(const FwdArgs& f, int y_dtype, void* scratch, int32_t* status, cudaStream_t st) {
    return gemm_tc_forward(f, 8, y_dtype, scratch, status, st);
}

}  // namespace qb
