// Quantized GEMM / GEMV over integer codes for BOTH operands with per-tensor symmetric scales:
// C <- alpha * (sa * A) * (sb * B) + beta * C, A [m, k] and B [k, n] row-major codes (int8 codes one per
// i32 word, or int4 codes packed eight per u32 word by FLAT element index), C [m, n] f32.  The scales fold
// into alpha_eff = alpha * sa * sb, so the kernels work on the raw codes.
//
// The sum of code products is computed EXACTLY, in integers: tcgen05.mma kind::i8 accumulates s8 x s8 into
// s32 in TMEM, so the only roundings are the conversion of the integer sum to f32 (none below 2^24) and
// the two products and one sum of alpha_eff * acc + beta * c.
//
// Three steps on the caller's stream:
//   1. k_pack_rows:  A codes -> int8 [m, kp] (kp = k rounded up to 128, zero filled): K-major rows.
//   2. k_pack_cols:  B codes -> int8 [n, kp], transposed through shared memory, so B is K-major as well.
//   3. k_gemm_i8_tc: persistent, one CTA per SM, CTAs paired in clusters of two; a pair walks 256 (m) x 256 (n) tiles
//      of C.  Per stage (128 k) each CTA's TMA warp fetches ITS 128 rows of A and ITS 128 rows of B (128-byte swizzle);
//      one elected thread of the pair's leader issues four tcgen05.mma.cta_group::2 (256 x 256 x 32) that read both
//      CTAs' halves, so every byte staged in shared memory feeds two tensor cores — at int8 rates a single CTA's
//      shared-memory bandwidth (operand reads plus TMA fills) would cap the tensor pipe at about two thirds.
//      Each CTA keeps its 128 rows of the accumulator in TMEM, twice; four warps read one back (tcgen05.ld) and
//      write alpha_eff * acc + beta * c while the other is being accumulated.
// n = 1 (the GEMV entries) skips all of it: one warp per row of A reads the codes once, HBM bound.
// Every wait on an mbarrier is bounded; a wait that runs out records QB200_ERR_TIMEOUT in the status word
// that qb200_gemm_quant_check reads.
#include <cuda.h>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <utility>

#include "common.hpp"

namespace qb {

constexpr uint32_t BQ_TM = 256, BQ_TN = 256, BQ_BK = 128;  // a CTA pair's tile of C; k per stage (128 int8 = one swizzle row)
constexpr uint32_t BQ_S = 6;
constexpr uint32_t BQ_THREADS = 256;  // warp 0 TMA, warp 1 MMA + TMEM, warp 2 forwarder, warps 4-7 epilogue
constexpr uint32_t BQ_HALF = 128 * BQ_BK, BQ_STAGE = 2 * BQ_HALF;  // per CTA and stage: 128 rows of A, 128 rows of B
constexpr uint32_t BQ_SMEM = 1024 + BQ_S * BQ_STAGE + 256;
constexpr uint32_t BQ_SPIN = 1u << 22;
constexpr int32_t BQ_FLAG_RANGE = 1, BQ_FLAG_TIMEOUT = 2;

struct BqArgs {
    float* c;
    int32_t* status;
    uint32_t m, n, kp;
    float alpha_eff, beta;
};

__device__ __forceinline__ uint32_t bq_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// The code at flat element index idx: an i32 word (int8 codes; outside [-128, 127] raises the range flag)
// or nibble idx % 8 of word idx / 8, sign extended (int4 codes).
template <int BITS>
__device__ __forceinline__ int32_t bq_code(const void* p, uint64_t idx, int32_t& flag) {
    if (BITS == 8) {
        const int32_t v = static_cast<const int32_t*>(p)[idx];
        if (v < -128 || v > 127) flag = BQ_FLAG_RANGE;
        return v;
    }
    const uint32_t w = static_cast<const uint32_t*>(p)[idx >> 3];
    return (int32_t)(w << (28 - 4 * (uint32_t)(idx & 7))) >> 28;
}

// A [rows, k] codes -> int8 [rows, kp], zero beyond k.  One thread per sixteen output bytes: four 16-byte loads of
// i32 codes in flight per thread where the row allows it (int8 codes, k % 4 == 0, aligned base), scalar reads at
// the ragged end of a row and for int4 codes; one block round per thread.
template <int BITS>
__global__ void __launch_bounds__(256) k_pack_rows(const void* __restrict__ src, uint32_t rows, uint32_t k, uint32_t kp,
                                                    uint4* __restrict__ dst, int32_t* status, int vec_ok) {
    const uint64_t units_per_row = kp >> 4, total = (uint64_t)rows * units_per_row;
    const uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (i >= total) return;
    int32_t flag = 0;
    const uint64_t r = i / units_per_row;
    const uint32_t c0 = (uint32_t)(i - r * units_per_row) * 16;
    uint32_t out[4] = {0, 0, 0, 0};
    if (BITS == 8 && vec_ok && c0 + 16 <= k) {
        const int4* p = reinterpret_cast<const int4*>(static_cast<const int32_t*>(src) + r * k + c0);
        int4 v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = __ldcs(p + j);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int32_t lo = min(min(v[j].x, v[j].y), min(v[j].z, v[j].w)), hi = max(max(v[j].x, v[j].y), max(v[j].z, v[j].w));
            if (lo < -128 || hi > 127) flag = BQ_FLAG_RANGE;
            out[j] = ((uint32_t)v[j].x & 0xFFu) | (((uint32_t)v[j].y & 0xFFu) << 8) | (((uint32_t)v[j].z & 0xFFu) << 16) | ((uint32_t)v[j].w << 24);
        }
    } else {
#pragma unroll
        for (uint32_t j = 0; j < 16; j++)
            if (c0 + j < k) out[j >> 2] |= ((uint32_t)bq_code<BITS>(src, r * k + c0 + j, flag) & 0xFFu) << (8 * (j & 3));
    }
    dst[i] = make_uint4(out[0], out[1], out[2], out[3]);
    if (flag) atomicOr(status, flag);
}

// B [k, n] codes -> int8 [n, kp] (transposed), zero beyond k.  A block moves a 128 (k) x 32 (n) tile through
// shared memory.  A thread owns four consecutive k of four consecutive n: four 16-byte loads along n (int8 codes,
// n % 4 == 0, aligned base; scalar reads otherwise), four words of four packed k each, parked at [n][k / 4]
// (pitch 33 words: no bank conflicts either way); writes are 16 bytes along k.
template <int BITS>
__global__ void __launch_bounds__(256) k_pack_cols(const void* __restrict__ src, uint32_t k, uint32_t n, uint32_t kp,
                                                    uint8_t* __restrict__ dst, int32_t* status, int vec_ok) {
    __shared__ uint32_t tile[32][33];
    const uint32_t n0 = blockIdx.x * 32, k0 = blockIdx.y * 128;
    const uint32_t nq = threadIdx.x & 7, q = threadIdx.x >> 3;  // columns n0 + 4 nq .. + 3, rows k0 + 4 q .. + 3
    const uint32_t nn = n0 + 4 * nq, kk = k0 + 4 * q;
    int32_t flag = 0;
    int32_t v[4][4];  // [k][n]
    if (BITS == 8 && vec_ok && nn + 4 <= n && kk + 4 <= k) {
        const int32_t* p = static_cast<const int32_t*>(src) + (uint64_t)kk * n + nn;
        int4 r[4];
#pragma unroll
        for (int j = 0; j < 4; j++) r[j] = __ldcs(reinterpret_cast<const int4*>(p + (uint64_t)j * n));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            v[j][0] = r[j].x; v[j][1] = r[j].y; v[j][2] = r[j].z; v[j][3] = r[j].w;
            const int32_t lo = min(min(r[j].x, r[j].y), min(r[j].z, r[j].w)), hi = max(max(r[j].x, r[j].y), max(r[j].z, r[j].w));
            if (lo < -128 || hi > 127) flag = BQ_FLAG_RANGE;
        }
    } else {
#pragma unroll
        for (uint32_t j = 0; j < 4; j++)
#pragma unroll
            for (uint32_t e = 0; e < 4; e++)
                v[j][e] = (kk + j < k && nn + e < n) ? bq_code<BITS>(src, (uint64_t)(kk + j) * n + nn + e, flag) : 0;
    }
#pragma unroll
    for (uint32_t e = 0; e < 4; e++)
        tile[4 * nq + e][q] = ((uint32_t)v[0][e] & 0xFFu) | (((uint32_t)v[1][e] & 0xFFu) << 8) | (((uint32_t)v[2][e] & 0xFFu) << 16) |
                              ((uint32_t)v[3][e] << 24);
    __syncthreads();
    const uint32_t row = threadIdx.x >> 3, chunk = threadIdx.x & 7;  // 32 rows of n, eight 16-byte pieces of k each
    if (n0 + row < n)
        *reinterpret_cast<uint4*>(dst + (uint64_t)(n0 + row) * kp + k0 + chunk * 16) =
            make_uint4(tile[row][chunk * 4], tile[row][chunk * 4 + 1], tile[row][chunk * 4 + 2], tile[row][chunk * 4 + 3]);
    if (flag) atomicOr(status, flag);
}

// y[r] <- alpha_eff * sum_p A[r, p] * x[p] + beta * y[r]: one warp per row, the integer sum kept in 64 bits.
template <int BITS>
__global__ void __launch_bounds__(256) k_gemv_q(const void* __restrict__ a, const void* __restrict__ x, uint32_t m, uint32_t k,
                                                 float alpha_eff, float beta, float* __restrict__ y, int32_t* status) {
    const uint32_t lane = threadIdx.x & 31, row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= m) return;
    int32_t flag = 0;
    long long acc = 0;
    if (BITS == 8) {
        const int32_t* ar = static_cast<const int32_t*>(a) + (uint64_t)row * k;
        const int32_t* xs = static_cast<const int32_t*>(x);
        if ((k & 3) == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
            int32_t part = 0;  // at most k / 32 products of at most 2^14 each per lane before the fold below
            uint32_t since = 0;
            auto step = [&](const int4& av, const int4& xv) {
                const int32_t lo = min(min(av.x, av.y), min(av.z, av.w)), hi = max(max(av.x, av.y), max(av.z, av.w));
                const int32_t xlo = min(min(xv.x, xv.y), min(xv.z, xv.w)), xhi = max(max(xv.x, xv.y), max(xv.z, xv.w));
                if (lo < -128 || hi > 127 || xlo < -128 || xhi > 127) flag = BQ_FLAG_RANGE;
                part += av.x * xv.x + av.y * xv.y + av.z * xv.z + av.w * xv.w;
                if (++since == 8192) { acc += part; part = 0; since = 0; }
            };
            uint32_t p = lane * 4;
            for (; p + 384 < k; p += 512) {  // four 16-byte loads of A's codes in flight per lane
                int4 av[4];
#pragma unroll
                for (int u = 0; u < 4; u++) av[u] = __ldcs(reinterpret_cast<const int4*>(ar + p + u * 128));
#pragma unroll
                for (int u = 0; u < 4; u++) step(av[u], __ldg(reinterpret_cast<const int4*>(xs + p + u * 128)));
            }
            for (; p < k; p += 128) step(*reinterpret_cast<const int4*>(ar + p), __ldg(reinterpret_cast<const int4*>(xs + p)));
            acc += part;
        } else {
            for (uint32_t p = lane; p < k; p += 32)
                acc += (long long)bq_code<8>(ar, p, flag) * bq_code<8>(xs, p, flag);
        }
    } else {
        // walk the words that hold the row's nibbles; a row may start and end inside a word
        const uint64_t first = (uint64_t)row * k, last = first + k;
        const uint32_t* aw = static_cast<const uint32_t*>(a);
        for (uint64_t w = (first >> 3) + lane; w * 8 < last; w += 32) {
            const uint32_t word = aw[w];
#pragma unroll
            for (uint32_t j = 0; j < 8; j++) {
                const uint64_t idx = w * 8 + j;
                if (idx >= first && idx < last) {
                    const int32_t q = (int32_t)(word << (28 - 4 * j)) >> 28;
                    acc += q * bq_code<4>(x, idx - first, flag);
                }
            }
        }
    }
#pragma unroll
    for (uint32_t o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) y[row] = __fadd_rn(__fmul_rn(alpha_eff, (float)acc), __fmul_rn(beta, y[row]));
    if (flag) atomicOr(status, flag);
}

// ---- the tensor-core kernel ----

__device__ __forceinline__ void bq_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bq_smem(bar)), "r"(count));
}
__device__ __forceinline__ void bq_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bq_smem(bar)), "r"(bytes) : "memory");
}
// Bounded wait: false when the poll limit ran out.
__device__ __forceinline__ bool bq_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < BQ_SPIN; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bq_smem(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ uint32_t bq_elect() {
    uint32_t e;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(e));
    return e;
}
__device__ __forceinline__ void bq_tma_load_2d(void* dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            bq_smem(dst)),
        "l"(map), "r"(x), "r"(y), "r"(bq_smem(bar))
        : "memory");
}
// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t bq_desc(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void bq_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// When the MMAs issued so far have completed, arrive on the barrier at this offset in BOTH CTAs of the pair.
__device__ __forceinline__ void bq_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     bq_smem(bar)),
                 "h"(both)
                 : "memory");
}
__device__ __forceinline__ uint32_t bq_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Shared-memory address of this CTA mapped to the same offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t bq_map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
// Arrive on a barrier of a CTA of this cluster.  What the arrival publishes was ordered before it by its own fence
// (the TMA's completion, tcgen05.fence for TMEM reads); default semantics, no cluster-scope release.
__device__ __forceinline__ void bq_mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void bq_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void bq_tmem_ld32(uint32_t taddr, int32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(BQ_THREADS, 1)
    k_gemm_i8_tc(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, BqArgs a) {
    extern __shared__ __align__(1024) uint8_t bq_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bq_smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BQ_S * BQ_STAGE);
    uint64_t* full = bars;            // leader: a stage's tiles have landed in BOTH CTAs
    uint64_t* full_x = full + BQ_S;   // non-leader: its own tiles have landed (TMA)
    uint64_t* empty = full_x + BQ_S;  // the MMAs that read the stage are done (arrives in both CTAs)
    uint64_t* dfull = empty + BQ_S;   // [2] an accumulator is complete (arrives in both CTAs)
    uint64_t* dempty = dfull + 2;     // [2] leader: the epilogue warps of both CTAs have read it out of TMEM
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dempty + 2);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = bq_cluster_rank();  // 0: the pair's leader
    // persistent: pair p takes tiles p, p + pairs, ...; m runs fastest, so the pairs of one round share B's tiles
    // in L2.  The stage ring and the two accumulators run across tile boundaries, so one tile's read-out and store
    // overlap the next tile's K loop.
    const uint32_t pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    const uint32_t m_tiles = (a.m + BQ_TM - 1) / BQ_TM;
    const uint32_t tiles = m_tiles * ((a.n + BQ_TN - 1) / BQ_TN);
    const uint32_t num_k = a.kp / BQ_BK;

    if (tid == 0) {
        for (uint32_t s = 0; s < BQ_S; s++) {
            bq_mbar_init(&full[s], 2);  // the leader's TMA (with its bytes) and the non-leader's "landed" message
            bq_mbar_init(&full_x[s], 1);
            bq_mbar_init(&empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; b++) {
            bq_mbar_init(&dfull[b], 1);
            bq_mbar_init(&dempty[b], 8);  // four epilogue warps in each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // all 512 TMEM columns of this CTA: two 128 x 256 s32 accumulators (this CTA's half of the rows)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(bq_smem(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    bq_cluster_sync();  // both CTAs' barriers are initialised before either arrives on the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        // ---- TMA producer: this CTA's 128 rows of A and 128 rows of B per stage ----
        if (lane == 0) {
            uint64_t* landed = rank == 0 ? full : full_x;
            uint32_t st = 0, par = 0, filled = 0;
            for (uint32_t t = pair; t < tiles && !failed; t += pairs) {
                const int32_t a_row = (int32_t)((t % m_tiles) * BQ_TM + rank * 128), b_row = (int32_t)((t / m_tiles) * BQ_TN + rank * 128);
                for (uint32_t it = 0; it < num_k; it++, filled++) {
                    if (filled >= BQ_S && !bq_wait(&empty[st], par ^ 1)) { failed = true; break; }
                    uint8_t* sa = smem + st * BQ_STAGE;
                    bq_mbar_expect_tx(&landed[st], BQ_STAGE);
                    bq_tma_load_2d(sa, &amap, (int32_t)(it * BQ_BK), a_row, &landed[st]);
                    bq_tma_load_2d(sa + BQ_HALF, &bmap, (int32_t)(it * BQ_BK), b_row, &landed[st]);
                    if (++st == BQ_S) { st = 0; par ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer (the pair's leader): the whole warp walks the loop, one elected lane issues ----
        if (rank == 0) {
            const uint32_t elected = bq_elect();
            // s32 accumulate, s8 x s8, both K-major, N = 256, M = 256 over the pair
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((BQ_TN >> 3) << 17) | ((BQ_TM >> 4) << 24);
            uint32_t st = 0, par = 0, lt = 0;  // lt: tiles this pair has started
            for (uint32_t t = pair; t < tiles && !failed; t += pairs, lt++) {
                const uint32_t buf = lt & 1;
                // the accumulator was last used by tile lt - 2: wait until its read-out is over in both CTAs
                if (lt >= 2 && !bq_wait(&dempty[buf], ((lt >> 1) & 1) ^ 1)) { failed = true; break; }
                for (uint32_t it = 0; it < num_k; it++) {
                    if (!bq_wait(&full[st], par)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = bq_desc(bq_smem(smem + st * BQ_STAGE)), db = bq_desc(bq_smem(smem + st * BQ_STAGE + BQ_HALF));
                    if (elected) {
#pragma unroll
                        for (uint32_t kk = 0; kk < BQ_BK / 32; kk++)  // +32 bytes per K = 32 step
                            bq_mma_i8(tmem_base + buf * BQ_TN, da + 2 * kk, db + 2 * kk, idesc, (it | kk) ? 1u : 0u);
                        bq_commit_pair(&empty[st]);
                    }
                    if (++st == BQ_S) { st = 0; par ^= 1; }
                }
                if (elected && !failed) bq_commit_pair(&dfull[buf]);
            }
        }
    } else if (warp == 2) {
        // ---- non-leader: pass "tiles landed" on to the leader's barrier ----
        if (lane == 0 && rank == 1) {
            const uint32_t remote = bq_map_to_cta(bq_smem(&full[0]), 0);
            uint32_t st = 0, par = 0;
            for (uint32_t t = pair; t < tiles && !failed; t += pairs)
                for (uint32_t it = 0; it < num_k; it++) {
                    if (!bq_wait(&full_x[st], par)) { failed = true; break; }
                    bq_mbar_arrive_cluster(remote + st * 8);
                    if (++st == BQ_S) { st = 0; par ^= 1; }
                }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ---- epilogue: a warp reads the TMEM lanes of its quarter (warp index mod 4), a thread owns one row of C ----
        const uint32_t quarter = warp & 3;
        const bool vec = (a.n & 3) == 0 && (reinterpret_cast<uintptr_t>(a.c) & 15) == 0;
        const uint32_t remote_dempty = bq_map_to_cta(bq_smem(&dempty[0]), 0);
        uint32_t lt = 0;
        for (uint32_t t = pair; t < tiles; t += pairs, lt++) {
            const uint32_t m_tile = t % m_tiles, n_tile = t / m_tiles, buf = lt & 1;
            const uint32_t row = m_tile * BQ_TM + rank * 128 + quarter * 32 + lane;
            if (!bq_wait(&dfull[buf], (lt >> 1) & 1)) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (uint32_t ch = 0; ch < BQ_TN / 32; ch++) {
                const uint32_t col0 = n_tile * BQ_TN + ch * 32;
                if (col0 >= a.n) break;  // warp-uniform
                int32_t acc[32];
                bq_tmem_ld32(tmem_base + ((quarter * 32) << 16) + buf * BQ_TN + ch * 32, acc);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < a.m) {
                    float* cr = a.c + (uint64_t)row * a.n + col0;
                    if (vec && col0 + 32 <= a.n) {
#pragma unroll
                        for (uint32_t j = 0; j < 32; j += 4) {
                            float4 cv = *reinterpret_cast<const float4*>(cr + j);
                            cv.x = __fadd_rn(__fmul_rn(a.alpha_eff, (float)acc[j]), __fmul_rn(a.beta, cv.x));
                            cv.y = __fadd_rn(__fmul_rn(a.alpha_eff, (float)acc[j + 1]), __fmul_rn(a.beta, cv.y));
                            cv.z = __fadd_rn(__fmul_rn(a.alpha_eff, (float)acc[j + 2]), __fmul_rn(a.beta, cv.z));
                            cv.w = __fadd_rn(__fmul_rn(a.alpha_eff, (float)acc[j + 3]), __fmul_rn(a.beta, cv.w));
                            *reinterpret_cast<float4*>(cr + j) = cv;
                        }
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < 32; j++)
                            if (col0 + j < a.n) cr[j] = __fadd_rn(__fmul_rn(a.alpha_eff, (float)acc[j]), __fmul_rn(a.beta, cr[j]));
                    }
                }
            }
            // this warp's reads of the accumulator are complete (wait::ld above): hand it back to the leader's MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bq_mbar_arrive_cluster(remote_dempty + buf * 8);
        }
    }
    if (failed) atomicOr(a.status, BQ_FLAG_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    bq_cluster_sync();  // neither CTA leaves while the other may still signal its barriers
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}

// ---- host side ----

typedef CUresult (*BqEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static BqEncodeFn bq_encode_fn() {
    static BqEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<BqEncodeFn>(p);
    }
    return fn;
}

// Packed operands and the status word live in a grow-only buffer per (device, stream): calls on one stream
// reuse it in stream order; calls on different streams never share one.
struct BqWorkspace {
    uint8_t* base = nullptr;
    size_t bytes = 0;
};
static std::mutex bq_mutex;
static std::map<std::pair<int, cudaStream_t>, BqWorkspace> bq_workspaces;

static qb200_status bq_workspace(cudaStream_t st, size_t need, uint8_t** out) {
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(bq_mutex);
    BqWorkspace& w = bq_workspaces[std::make_pair(dev, st)];
    if (w.bytes < need) {
        int32_t carried = 0;
        if (w.base) {  // keep what the status word holds: cudaFree waits for the stream's work first
            QB_CUDA_TRY(cudaStreamSynchronize(st));
            QB_CUDA_TRY(cudaMemcpy(&carried, w.base, 4, cudaMemcpyDeviceToHost));
            QB_CUDA_TRY(cudaFree(w.base));
            w.base = nullptr;
            w.bytes = 0;
        }
        const size_t grown = need + need / 4;
        QB_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&w.base), grown));
        w.bytes = grown;
        QB_CUDA_TRY(cudaMemcpyAsync(w.base, &carried, 4, cudaMemcpyHostToDevice, st));
        QB_CUDA_TRY(cudaStreamSynchronize(st));
    }
    *out = w.base;
    return QB200_OK;
}

template <int BITS>
static qb200_status bq_run(const char* who, uint32_t m, uint32_t n, uint32_t k, float alpha_eff, const void* a, const void* b,
                           float beta, float* c, cudaStream_t st) {
    if (m == 0 || n == 0) return QB200_OK;
    if (!a || !b || !c) return fail(QB200_ERR_INVALID_PARAM, std::string(who) + ": null device pointer");
    // the s32 accumulator holds every sum of k products of two codes
    const uint64_t max_k = BITS == 8 ? 131071ull : (1ull << 24);
    if (k > max_k) return fail(QB200_ERR_NOT_SUPPORTED, std::string(who) + ": k = " + std::to_string(k) + " exceeds " + std::to_string(max_k));
    const uint32_t kp = k == 0 ? BQ_BK : (uint32_t)(div_ceil(k, BQ_BK) * BQ_BK);
    const size_t a_bytes = (size_t)m * kp, b_bytes = (size_t)n * kp;
    const size_t a_off = 256, b_off = a_off + ((a_bytes + 255) & ~size_t(255));
    uint8_t* ws = nullptr;
    const bool gemv = n == 1;
    if (qb200_status s = bq_workspace(st, gemv ? 256 : b_off + b_bytes, &ws)) return s;
    int32_t* status = reinterpret_cast<int32_t*>(ws);
    if (gemv) {
        k_gemv_q<BITS><<<(m + 7) / 8, 256, 0, st>>>(a, b, m, k, alpha_eff, beta, c, status);
        QB_CUDA_TRY(cudaGetLastError());
        return QB200_OK;
    }
    BqEncodeFn enc = bq_encode_fn();
    if (!enc) return fail(QB200_ERR_CUDA, std::string(who) + ": cuTensorMapEncodeTiled is not available from this driver");
    uint8_t* a8 = ws + a_off;
    uint8_t* b8 = ws + b_off;
    {
        const uint64_t units = (uint64_t)m * (kp >> 4), blocks = (units + 255) / 256;
        if (blocks > 0x7FFFFFFFull) return fail(QB200_ERR_NOT_SUPPORTED, std::string(who) + ": A is too large for one launch");
        const int vec_ok = (k % 4 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0) ? 1 : 0;
        k_pack_rows<BITS><<<(uint32_t)blocks, 256, 0, st>>>(a, m, k, kp, reinterpret_cast<uint4*>(a8), status, vec_ok);
        QB_CUDA_TRY(cudaGetLastError());
        const int bvec_ok = (n % 4 == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0) ? 1 : 0;
        k_pack_cols<BITS><<<dim3((n + 31) / 32, kp / 128), 256, 0, st>>>(b, k, n, kp, b8, status, bvec_ok);
        QB_CUDA_TRY(cudaGetLastError());
    }
    CUtensorMap amap, bmap;
    const cuuint32_t estr[2] = {1, 1};
    const cuuint64_t strides[1] = {kp};
    {
        const cuuint64_t dims[2] = {kp, m};
        const cuuint32_t box[2] = {BQ_BK, 128};
        CUresult cr = enc(&amap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a8, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(QB200_ERR_CUDA, std::string(who) + ": cuTensorMapEncodeTiled (A) failed with code " + std::to_string((int)cr));
    }
    {
        const cuuint64_t dims[2] = {kp, n};
        const cuuint32_t box[2] = {BQ_BK, 128};
        CUresult cr = enc(&bmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, b8, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(QB200_ERR_CUDA, std::string(who) + ": cuTensorMapEncodeTiled (B) failed with code " + std::to_string((int)cr));
    }
    BqArgs args;
    args.c = c;
    args.status = status;
    args.m = m;
    args.n = n;
    args.kp = kp;
    args.alpha_eff = alpha_eff;
    args.beta = beta;
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    static bool attr_set[64] = {};
    if (!attr_set[dev & 63]) {
        QB_CUDA_TRY(cudaFuncSetAttribute(k_gemm_i8_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BQ_SMEM));
        attr_set[dev & 63] = true;
    }
    const uint64_t tiles = div_ceil(m, BQ_TM) * div_ceil(n, BQ_TN);
    if (tiles > 0x7FFFFFFFull) return fail(QB200_ERR_NOT_SUPPORTED, std::string(who) + ": too many output tiles");
    static int sm_count[64] = {};
    if (!sm_count[dev & 63]) QB_CUDA_TRY(cudaDeviceGetAttribute(&sm_count[dev & 63], cudaDevAttrMultiProcessorCount, dev));
    const uint64_t max_pairs = (uint64_t)sm_count[dev & 63] / 2;
    const uint32_t grid = 2 * (uint32_t)(tiles < max_pairs ? tiles : max_pairs);  // one CTA per SM, in clusters of two
    k_gemm_i8_tc<<<grid, BQ_THREADS, BQ_SMEM, st>>>(amap, bmap, args);
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

}  // namespace qb

using qb::fail;

extern "C" {

qb200_status qb200_gemm_quant(int qty, uint32_t m, uint32_t n, uint32_t k, float alpha, float a_scale, float b_scale,
                              const int32_t* a_dev, const int32_t* b_dev, float beta, float* c_dev, void* stream) {
    if (qty != QB200_Q8_SYMMETRIC)
        return fail(QB200_ERR_INVALID_PARAM, "gemm_quant: only Q8Symmetric rides one code per i32 word — use gemm_quant4 for Q4");
    return qb::bq_run<8>("gemm_quant", m, n, k, alpha * a_scale * b_scale, a_dev, b_dev, beta, c_dev, static_cast<cudaStream_t>(stream));
}

qb200_status qb200_gemm_quant4(int qty, uint32_t m, uint32_t n, uint32_t k, float alpha, float a_scale, float b_scale,
                               const uint32_t* a_dev, const uint32_t* b_dev, float beta, float* c_dev, void* stream) {
    if (qty != QB200_Q4_SYMMETRIC)
        return fail(QB200_ERR_INVALID_PARAM, "gemm_quant4: only Q4Symmetric rides packed u32 words — use gemm_quant for Q8");
    return qb::bq_run<4>("gemm_quant4", m, n, k, alpha * a_scale * b_scale, a_dev, b_dev, beta, c_dev, static_cast<cudaStream_t>(stream));
}

qb200_status qb200_gemv_quant(int qty, uint32_t m, uint32_t n, float alpha, float a_scale, float x_scale, const int32_t* a_dev,
                              const int32_t* x_dev, float beta, float* y_dev, void* stream) {
    return qb200_gemm_quant(qty, m, 1, n, alpha, a_scale, x_scale, a_dev, x_dev, beta, y_dev, stream);
}

qb200_status qb200_gemv_quant4(int qty, uint32_t m, uint32_t n, float alpha, float a_scale, float x_scale, const uint32_t* a_dev,
                               const uint32_t* x_dev, float beta, float* y_dev, void* stream) {
    return qb200_gemm_quant4(qty, m, 1, n, alpha, a_scale, x_scale, a_dev, x_dev, beta, y_dev, stream);
}

qb200_status qb200_gemm_quant_check(void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    uint8_t* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(qb::bq_mutex);
        auto it = qb::bq_workspaces.find(std::make_pair(dev, st));
        if (it != qb::bq_workspaces.end()) base = it->second.base;
    }
    QB_CUDA_TRY(cudaStreamSynchronize(st));
    if (!base) return QB200_OK;
    int32_t flags = 0;
    const int32_t zero = 0;
    QB_CUDA_TRY(cudaMemcpy(&flags, base, 4, cudaMemcpyDeviceToHost));
    if (flags) QB_CUDA_TRY(cudaMemcpy(base, &zero, 4, cudaMemcpyHostToDevice));
    if (flags & qb::BQ_FLAG_TIMEOUT) return fail(QB200_ERR_TIMEOUT, "gemm_quant: a wait inside the kernel ran out of polls; the result is not valid");
    if (flags & qb::BQ_FLAG_RANGE) return fail(QB200_ERR_INVALID_PARAM, "gemm_quant: an int8 code outside [-128, 127]");
    return QB200_OK;
}

}  // extern "C"
