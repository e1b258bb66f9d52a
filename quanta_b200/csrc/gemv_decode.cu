// Decode GEMV (M <= 16): y[m, n] = sum_k x[m, k] * s[n, k/128] * q[n, k] over resident
// packed-int4 codes `[N, K/8]` (u32, low nibble first) with a 1x128 f32 scale grid and bf16
// activations.  HBM-bound: the kernel's job is to keep the codes streaming.
//
// Layout and flow, one CTA per contiguous slab of output rows:
//   1. one warp issues bulk async copies (cp.async.bulk, completion on an mbarrier per
//      16-row block) for the slab's codes — every row a contiguous K/2-byte burst — and all
//      threads fetch its scales; nothing here depends on the previous kernel, so with programmatic dependent
//      launch this prefetch overlaps the previous layer's tail;
//   2. griddepcontrol.wait, then each warp takes a slice of the scale groups: it loads its
//      x fragment from L2, unpacks nibbles to exact bf16 integers in registers
//      (lop3 with the 136.0 magic constant, one bf16x2 subtract), multiplies on the tensor
//      pipe (mma.sync m16n8k16, f32 accumulate: W rows are the M side, the batch is the N
//      side) and applies the f32 scale once per 128-k group to the group's partial sum;
//   3. warps fold their K slices through shared memory and write y (+ bias).
// Codes are exact in bf16 and products accumulate in f32, so the only rounding is the f32
// accumulation order.
#include <cuda_bf16.h>
#include <cstdint>

#include "forward.hpp"
#include "quant_math.cuh"

namespace qb {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr uint32_t GEMV_ROW_PAD = 64;        // bytes added to each smem row: shifts banks by 16
constexpr uint32_t GEMV_SPIN_LIMIT = 1u << 22;  // mbarrier polls before giving up (~ seconds)

struct GemvArgs {
    const uint32_t* codes;  // [N, K/8]
    const float* scales;    // [N, K/128]
    const float* bias;      // [N] or null
    const uint16_t* x;      // bf16 [M, K]
    void* y;                // [M, N] f32 or bf16
    int32_t* status;        // device status word (0 = ok, QB200_ERR_TIMEOUT on a wait that ran out)
    uint32_t M, N, K, rows_per_cta;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
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

// One packed word -> four bf16x2 registers of exact integer codes:
// r[i] = (q_i, q_{i+4}).  0x4308 is bf16 136.0 = 128 + 8: xor-ing it onto a masked nibble n
// sets the exponent and flips bit 3, giving 128 + (n ^ 8) = 136 + q; one subtract leaves q.
__device__ __forceinline__ void unpack_word(uint32_t w, uint32_t (&r)[4]) {
    constexpr uint32_t MASK = 0x000F000Fu, MAGIC = 0x43084308u;
    const __nv_bfloat162 bias = *reinterpret_cast<const __nv_bfloat162*>(&MAGIC);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t v = lop3_and_xor(w >> (4 * i), MASK, MAGIC);
        __nv_bfloat162 q = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias);
        r[i] = *reinterpret_cast<uint32_t*>(&q);
    }
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

// RB: 16-row blocks per CTA; NT: 8-wide batch tiles (M <= 8 * NT).
template <int RB, int NT, typename YT>
__global__ void __launch_bounds__(GEMV_THREADS) k_gemv_i4(GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t groups = a.K >> 7;               // scale groups per row
    const uint32_t row_bytes = a.K >> 1;            // packed codes per row
    const uint32_t stride = row_bytes + GEMV_ROW_PAD;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                     // RB barriers
    float* s_scales = reinterpret_cast<float*>(smem + 64);                  // [RB*16][groups]
    uint8_t* s_codes = smem + 64 + (((uint32_t)RB * 16 * groups * 4 + 127) & ~127u);  // [RB*16][stride]

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t row0 = blockIdx.x * a.rows_per_cta;
    const uint32_t nrows = min(a.rows_per_cta, a.N - row0);

    if (tid == 0) {
#pragma unroll
        for (int rb = 0; rb < RB; rb++) mbar_init(&bars[rb], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        // lane rb arms barrier rb with the byte count of its rows, then lanes share the row copies
#pragma unroll
        for (int rb = 0; rb < RB; rb++) {
            const uint32_t lo = rb * 16, hi = min(nrows, lo + 16u);
            if (lane == 0 && hi > lo) {
                mbar_expect_tx(&bars[rb], (hi - lo) * row_bytes);
            }
        }
        __syncwarp();
        for (uint32_t r = lane; r < nrows; r += 32)
            bulk_g2s(s_codes + r * stride, reinterpret_cast<const uint8_t*>(a.codes) + (uint64_t)(row0 + r) * row_bytes,
                     row_bytes, &bars[r >> 4]);
    }
    // The slab's scales are a few KB at any alignment: plain loads, also ahead of the wait.
    for (uint32_t i = tid; i < nrows * groups; i += GEMV_THREADS) s_scales[i] = __ldg(a.scales + (uint64_t)row0 * groups + i);
    // Let the next kernel in the stream start its own prefetch; then wait for the previous
    // one to finish before touching x or y (both no-ops without programmatic launch).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();

    float acc[RB][NT][4];
#pragma unroll
    for (int rb = 0; rb < RB; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[rb][nt][i] = 0.0f;

    bool ready[RB];
#pragma unroll
    for (int rb = 0; rb < RB; rb++) ready[rb] = false;
    bool failed = false;

    for (uint32_t G = warp; G < groups && !failed; G += GEMV_WARPS) {
        // x fragments of this group, permuted to the nibble order of unpack_word
        uint32_t bx[NT][8][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint32_t b = g + 8 * nt;
            uint32_t xr[16];
            if (b < a.M) {
                const uint4* xp = reinterpret_cast<const uint4*>(a.x + (uint64_t)b * a.K + G * 128 + t * 32);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    uint4 v = __ldg(xp + i);
                    xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; i++) xr[i] = 0;
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    bx[nt][2 * j + h][0] = __byte_perm(xr[4 * j + h], xr[4 * j + h + 2], 0x5410);
                    bx[nt][2 * j + h][1] = __byte_perm(xr[4 * j + h], xr[4 * j + h + 2], 0x7632);
                }
        }
#pragma unroll
        for (int rb = 0; rb < RB; rb++) {
            if (rb * 16u >= nrows) break;
            if (!ready[rb]) {
                if (!mbar_wait_bounded(&bars[rb], 0)) {
                    failed = true;
                    break;
                }
                ready[rb] = true;
            }
            const uint32_t ra = rb * 16 + g, rc = ra + 8;
            const uint4 c0 = *reinterpret_cast<const uint4*>(s_codes + ra * stride + G * 64 + t * 16);
            const uint4 c1 = *reinterpret_cast<const uint4*>(s_codes + rc * stride + G * 64 + t * 16);
            const uint32_t w0[4] = {c0.x, c0.y, c0.z, c0.w}, w1[4] = {c1.x, c1.y, c1.z, c1.w};
            float part[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) part[nt][i] = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t r0[4], r1[4];
                unpack_word(w0[j], r0);
                unpack_word(w1[j], r1);
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
                        mma_bf16(part[nt], r0[2 * h], r1[2 * h], r0[2 * h + 1], r1[2 * h + 1], bx[nt][2 * j + h][0],
                                 bx[nt][2 * j + h][1]);
            }
            const float s0 = s_scales[ra * groups + G], s1 = s_scales[rc * groups + G];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                acc[rb][nt][0] = fmaf(s0, part[nt][0], acc[rb][nt][0]);
                acc[rb][nt][1] = fmaf(s0, part[nt][1], acc[rb][nt][1]);
                acc[rb][nt][2] = fmaf(s1, part[nt][2], acc[rb][nt][2]);
                acc[rb][nt][3] = fmaf(s1, part[nt][3], acc[rb][nt][3]);
            }
        }
    }
    if (failed) atomicExch(a.status, QB200_ERR_TIMEOUT);
    // Every thread must have seen the copies land before the buffer is reused below.
    if (__syncthreads_or(failed ? 1 : 0)) {
        // A copy never completed: wait (bounded) for whatever is still in flight, then leave.
#pragma unroll
        for (int rb = 0; rb < RB; rb++)
            if (rb * 16u < nrows) mbar_wait_bounded(&bars[rb], 0);
        return;
    }

    // fold the K slices of the 8 warps: red[warp][row][batch] aliases the codes buffer
    constexpr int BATCH = NT * 8;
    float* red = reinterpret_cast<float*>(s_codes);
#pragma unroll
    for (int rb = 0; rb < RB; rb++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float* base = red + ((warp * RB * 16 + rb * 16) * BATCH) + nt * 8;
            base[(g)*BATCH + 2 * t] = acc[rb][nt][0];
            base[(g)*BATCH + 2 * t + 1] = acc[rb][nt][1];
            base[(g + 8) * BATCH + 2 * t] = acc[rb][nt][2];
            base[(g + 8) * BATCH + 2 * t + 1] = acc[rb][nt][3];
        }
    __syncthreads();
    for (uint32_t e = tid; e < nrows * a.M; e += GEMV_THREADS) {
        const uint32_t r = e % nrows, b = e / nrows;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; w++) v += red[(w * RB * 16 + r) * BATCH + b];
        const uint32_t n = row0 + r;
        if (a.bias) v += a.bias[n];
        store_y<YT>(static_cast<YT*>(a.y) + (uint64_t)b * a.N + n, v);
    }
}

// ---- host side ------------------------------------------------------------------

struct GemvPlan {
    uint32_t ctas, rows_per_cta, rb, smem;
};

static uint32_t gemv_smem(uint32_t rb, uint32_t K, uint32_t nt) {
    const uint32_t groups = K / 128;
    uint32_t codes = rb * 16 * (K / 2 + GEMV_ROW_PAD);
    uint32_t red = GEMV_WARPS * rb * 16 * nt * 8 * 4;
    return 64 + ((rb * 16 * groups * 4 + 127) & ~127u) + (codes > red ? codes : red);
}

bool gemv_i4_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* scales, const void* x) {
    if (bits != 4 || gr != 1 || gc != 128 || layout != QB200_OUT_IN || x_dtype != QB200_BF16) return false;
    if (m == 0 || m > 16 || in_dim % 128 != 0 || in_dim > 32768 || out_dim > 0x7FFFFFFF) return false;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return al(codes) && al(scales) && al(x);
}

static bool gemv_plan(uint32_t N, uint32_t K, uint32_t nt, GemvPlan& p) {
    for (uint32_t c = 1; c <= 64; c++) {
        uint32_t ctas = 148 * c;
        if (ctas > N) ctas = N;
        uint32_t rows = (N + ctas - 1) / ctas;
        uint32_t rb = (rows + 15) / 16;
        if (rb <= 4) {
            uint32_t smem = gemv_smem(rb, K, nt);
            if (smem <= 100 * 1024 || (ctas == N && smem <= 200 * 1024)) {
                p.ctas = (N + rows - 1) / rows;
                p.rows_per_cta = rows;
                p.rb = rb;
                p.smem = smem;
                return true;
            }
        }
        if (ctas == N) break;
    }
    return false;
}

template <int RB, int NT, typename YT>
static qb200_status launch_gemv(const GemvArgs& a, const GemvPlan& p, cudaStream_t st) {
    auto kern = k_gemv_i4<RB, NT, YT>;
    static bool attr_set[64] = {};  // per instantiation and device
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        QB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.ctas);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a));
    return QB200_OK;
}

template <int NT, typename YT>
static qb200_status by_rb(const GemvArgs& a, const GemvPlan& p, cudaStream_t st) {
    switch (p.rb) {
        case 1: return launch_gemv<1, NT, YT>(a, p, st);
        case 2: return launch_gemv<2, NT, YT>(a, p, st);
        case 3: return launch_gemv<3, NT, YT>(a, p, st);
        default: return launch_gemv<4, NT, YT>(a, p, st);
    }
}

// Returns QB200_ERR_NOT_SUPPORTED (without setting an error) when no launch plan fits.
qb200_status gemv_i4_forward(const FwdArgs& f, int y_dtype, int32_t* status, cudaStream_t st) {
    GemvArgs a;
    a.codes = static_cast<const uint32_t*>(f.codes);
    a.scales = f.scales;
    a.bias = f.bias;
    a.x = static_cast<const uint16_t*>(f.x);
    a.y = f.y;
    a.status = status;
    a.M = (uint32_t)f.m;
    a.N = (uint32_t)f.out_dim;
    a.K = (uint32_t)f.in_dim;
    const uint32_t nt = f.m <= 8 ? 1 : 2;
    GemvPlan p;
    if (!gemv_plan(a.N, a.K, nt, p)) return QB200_ERR_NOT_SUPPORTED;
    a.rows_per_cta = p.rows_per_cta;
    if (y_dtype == QB200_F32) return nt == 1 ? by_rb<1, float>(a, p, st) : by_rb<2, float>(a, p, st);
    return nt == 1 ? by_rb<1, uint16_t>(a, p, st) : by_rb<2, uint16_t>(a, p, st);
}

}  // namespace qb
