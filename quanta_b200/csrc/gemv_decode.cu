// Decode GEMV (M <= 16): y[m, n] = sum_k x[m, k] * s[n, k/128] * q[n, k] over resident
// packed-int4 codes `[N, K/8]` (u32, low nibble first) with a 1x128 f32 scale grid and bf16
// activations, K <= 4096 per launch (wider inputs run as column slices, one launch over all of them).
// HBM-bound: the kernel's job is to keep the codes streaming and to spend as few issue slots per
// weight as possible.
//
// The kernel is persistent: one CTA per SM walks work items (a slab of <= 16 * RB contiguous rows of
// one layer: ONE bulk async copy) through a ring of shared-memory stages, so the copies of later
// items are in flight while the current one is multiplied.  Each of 16 warps owns two 128-k scale
// groups and keeps its activation fragments in registers for the whole launch; W rows are the M side
// of mma.sync m16n8k16 (f32 accumulate), the batch is the N side.  One launch can serve several
// layers (grouped forward); a single layer is the same kernel with one descriptor.  Nothing the
// prologue touches depends on the previous kernel, so with programmatic dependent launch the first
// copies overlap the previous kernel's tail.
//
// Unpacking costs five integer instructions per packed word.  A bf16 whose exponent field is
// 0 or 1 is linear in its bit pattern (value = bits * 2^-133), and the tensor pipe honours
// such inputs exactly, so a masked nibble IS a bf16 operand: `(w & 0x000F000F) ^ 0x00080008`
// holds (q + 8) for nibbles 0 and 4, `(w & 0x00F000F0) ^ 0x00800080` holds 16 (q + 8) for
// nibbles 1 and 5, and one shift by 8 exposes nibbles 2, 3, 6, 7 the same way.  x is scaled by
// 2^40 (2^36 against the 16x positions) so products stay normal f32; the "+ 8" is removed by
// subtracting 8 * sum_k x_k per group, and the group's f32 scale and 2^93 are applied once per
// 128-k group.  Every product (integer code times bf16 activation) is exact in f32; the only
// rounding is f32 accumulation.  Activations must satisfy |x| < 2^87 (the host entry points
// check this bound where they can: see qlinear.cu).
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdlib>

#include "forward.hpp"
#include "quant_math.cuh"

namespace qb {

constexpr uint32_t GEMV_SPIN_LIMIT = 1u << 22;  // mbarrier polls before giving up (~ seconds)
constexpr int GEMV_MAX_LAYERS = 40;             // descriptors travel by value in the kernel parameters

struct GemvLayer {
    const uint32_t* codes;  // [N, K/8]
    const float* scales;    // [N, K/128]
    const float* bias;      // [N] or null
    const uint16_t* x;      // bf16 [M, K], rows ldx elements apart
    void* y;                // [M, N] f32 or bf16
    uint32_t N, rows_per_item, item0;  // this layer owns items [item0, item0 + ceil(N / rows_per_item))
    uint32_t ldx, kvalid;   // x's row stride; columns >= kvalid of x do not exist and read as zero
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
    uint32_t ll_mode;  // outputs are LLPair elements stamped with the exchange number; no barrier in the launch
    uint64_t ll_slot_stride;  // pushed all-gather: bytes between the ranks' slots of an arena (0: the launch does not wait for the peers)
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

// An output pushed to the ranks of a node as a self-validating element: the f32 bits and the number of the exchange
// that wrote them, stored (and polled by the consumer) as ONE 8-byte access, so that no fence and no barrier
// has to order data and flag — the element is either the old pair or the new one.
struct LLPair {
    uint32_t bits, flag;
};
__device__ __forceinline__ void store_ll(LLPair* p, float v, uint32_t flag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(flag) : "memory");
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

}  // namespace qb

#include "gemv_reg.cuh"
#include "gemv_reg_async.cuh"
#include "gemv_i8.cuh"

namespace qb {

// ---- host side ------------------------------------------------------------------

template <int NT, int RB, int NSERV, typename YT>
static qb200_status launch_gemv_async(const GemvBatch& b, uint32_t smem, uint32_t ctas, cudaStream_t st) {
    auto kern = k_gemv_i4_async<NT, RB, NSERV, YT>;
    static bool attr_set[64] = {};  // per instantiation and device
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        if (NT == 2) {
            // the kernel's warps re-balance their registers; the arithmetic holds only if every warp starts with
            // ASYNC_REGS_LAUNCH of them (a request for registers nobody releases would wait for ever)
            cudaFuncAttributes fa;
            QB_CUDA_TRY(cudaFuncGetAttributes(&fa, kern));
            if (fa.numRegs != (int)ASYNC_REGS_LAUNCH) return QB200_ERR_NOT_SUPPORTED;
        }
        QB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(async_threads(NT, NSERV));
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

bool gemv_i4_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* scales, const void* x) {
    if (bits != 4 || gr != 1 || gc != 128 || layout != QB200_OUT_IN || x_dtype != QB200_BF16) return false;
    if (m == 0 || m > 16 || in_dim % 128 != 0 || in_dim > 128 * 2 * REG_WARPS || out_dim > 0x7FFFFFFF) return false;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return al(codes) && al(scales) && al(x);
}

// Rows per work item of a launch over layers with `all_rows` output rows and `all_tiles` row tiles in total.  A
// launch with few items per CTA cuts the rows into a multiple of 148 items of at most 16 * rb rows (sized over
// the whole launch, not layer by layer), so the last wave of items is as full as the others; a launch with many
// items per CTA (`full_tiles`) takes whole 16 * rb-row items instead — the MMA and the unpack cost the same for
// a 28-row item as for a 32-row one, and the waves even out by number.
static uint32_t gemv_rows_per_item(uint64_t all_rows, uint64_t all_tiles, uint32_t rb, bool full_tiles) {
    if (full_tiles) return 16 * rb;
    const uint64_t k = (all_tiles + 147) / 148;
    uint64_t rows = (all_rows + 148 * k - 1) / (148 * k);
    if (rows > 16 * rb) rows = 16 * rb;
    return rows < 1 ? 1 : (uint32_t)rows;
}

// Grouped forward over `count` layers that share K and M.  Returns QB200_ERR_NOT_SUPPORTED
// (without setting an error) when the shape does not fit the kernel.
qb200_status gemv_i4_forward_many(const FwdArgs* f, uint32_t count, int y_dtype, int32_t* status, cudaStream_t st,
                                  const PeerSpec* peers) {
    if (count == 0) return QB200_OK;
    const uint32_t K = (uint32_t)f[0].in_dim, M = (uint32_t)f[0].m;
    if (K / 128 > 2 * REG_WARPS) return QB200_ERR_NOT_SUPPORTED;  // wider inputs run as column slices
    // Row blocks per item: a lone small layer keeps 16-row items (more items to pipeline and to
    // overlap with the neighbouring launches); grouped launches take 32-row items.
    const uint32_t rb = (count > 1 || peers) ? 2 : 1;
    uint64_t all_tiles = 0, all_rows = 0;
    for (uint32_t i = 0; i < count; i++) {
        all_tiles += (f[i].out_dim + 16 * rb - 1) / (16 * rb);
        all_rows += f[i].out_dim;
    }
    const bool full_tiles = all_tiles >= 8 * 148;  // eight or more items per CTA
    const uint32_t rpi = gemv_rows_per_item(all_rows, all_tiles, rb, full_tiles);
    for (uint32_t base = 0, n = 0; base < count; base += n) {
        // as many layers as fit the descriptor table and the per-CTA item table
        n = 0;
        for (uint32_t items = 0; base + n < count && n < (uint32_t)GEMV_MAX_LAYERS; n++) {
            const uint32_t N = (uint32_t)f[base + n].out_dim;
            items += (N + rpi - 1) / rpi;
            if (n > 0 && items > REG_MAX_ITEMS * 148) break;
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
            ly.rows_per_item = rpi;
            ly.item0 = items;
            ly.ldx = a.x_stride ? (uint32_t)a.x_stride : K;
            ly.kvalid = a.k_valid ? (uint32_t)a.k_valid : K;
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
        b.ll_mode = y_dtype == QB_Y_PUSHED ? 1 : 0;
        b.ll_slot_stride = b.ll_mode && peers ? peers->slot_stride : 0;
        if (b.ll_mode && (!peers || !peers->flags[peers->rank] || n < count)) return QB200_ERR_NOT_SUPPORTED;  // one launch, one exchange number
        b.peer_spin_limit = peer_spin_limit();
        b.count = n;
        b.total_items = items;
        b.M = M;
        b.K = K;
        if ((items + 147) / 148 > REG_MAX_ITEMS) return QB200_ERR_NOT_SUPPORTED;  // one layer with more items than a CTA describes
        const uint32_t nt = M <= 8 ? 1 : 2;
        // Slots of partial sums keep only the batch's columns (in fours), which for a small batch frees the room of
        // one more stage; the 16-column batch tile (nt == 2) folds 16-row sub-items.
        b.red_cols = M <= 2 ? 2 : (M + 3) & ~3u;
        b.red_stride = async_red_stride(b.red_cols);
        const uint32_t sub_rows = nt == 2 ? 16 : rb * 16;
        const uint32_t ctas = items < 148 ? items : 148, per_cta = (items + ctas - 1) / ctas;
        uint32_t stages = per_cta < 2 ? 2 : (per_cta > 6 ? 6 : per_cta);
        while (stages > 2 && async_smem_layout(K, rb, sub_rows, b.red_stride, stages).total > 227u * 1024) stages--;
        b.stages = stages;
        const uint32_t smem = async_smem_layout(K, rb, sub_rows, b.red_stride, stages).total;
        if (smem > 227u * 1024) return QB200_ERR_NOT_SUPPORTED;
        // one service warp folds up to four batch columns; two share the wider batches
#define QB_LAUNCH(YT)                                                                                                           \
    (nt == 2 ? (rb == 2 ? launch_gemv_async<2, 2, 2, YT>(b, smem, ctas, st) : launch_gemv_async<2, 1, 2, YT>(b, smem, ctas, st)) \
     : M > 4 ? (rb == 2 ? launch_gemv_async<1, 2, 2, YT>(b, smem, ctas, st) : launch_gemv_async<1, 1, 2, YT>(b, smem, ctas, st)) \
             : (rb == 2 ? launch_gemv_async<1, 2, 1, YT>(b, smem, ctas, st) : launch_gemv_async<1, 1, 1, YT>(b, smem, ctas, st)))
        const qb200_status r = y_dtype == QB200_F32 ? QB_LAUNCH(float) : y_dtype == QB_Y_PUSHED ? QB_LAUNCH(LLPair) : QB_LAUNCH(uint16_t);
#undef QB_LAUNCH
        if (r) return r;
    }
    return QB200_OK;
}

// ---- int8 ----

bool gemv_i8_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim, uint64_t m,
                      int x_dtype, const void* codes, const void* x) {
    if (bits != 8 || layout != QB200_OUT_IN || x_dtype != QB200_BF16 || gr == 0 || gc == 0) return false;
    if (m == 0 || m > 8 || in_dim % 128 != 0 || in_dim > 128 * 2 * REG_WARPS || out_dim > 0x7FFFFFFF) return false;
    if (gc % 32 != 0) return false;  // a run of 32 columns shares its scale
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return al(codes) && al(x);
}

template <int NSERV, typename YT>
static qb200_status launch_gemv_i8(const GemvBatchI8& b, uint32_t smem, uint32_t ctas, cudaStream_t st) {
    auto kern = k_gemv_i8_async<NSERV, YT>;
    static bool attr_set[64] = {};
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        QB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(REG_THREADS + 32 * NSERV);
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

// Grouped int8 forward over `count` layers that share K and M (any scale grids).  QB200_ERR_NOT_SUPPORTED (no message)
// when the shape does not fit the kernel.
qb200_status gemv_i8_forward_many(const FwdArgs* f, uint32_t count, int y_dtype, int32_t* status, cudaStream_t st) {
    if (count == 0) return QB200_OK;
    if (count > (uint32_t)I8_MAX_LAYERS) return QB200_ERR_NOT_SUPPORTED;
    const uint32_t K = (uint32_t)f[0].in_dim, M = (uint32_t)f[0].m;
    if (K / 128 > 2 * REG_WARPS || M > 8) return QB200_ERR_NOT_SUPPORTED;
    uint64_t all_tiles = 0, all_rows = 0;
    for (uint32_t i = 0; i < count; i++) {
        all_tiles += (f[i].out_dim + 15) / 16;
        all_rows += f[i].out_dim;
    }
    const uint32_t rpi = gemv_rows_per_item(all_rows, all_tiles, 1, all_tiles >= 8 * 148);
    GemvBatchI8 b = {};
    uint32_t items = 0, srows_max = 1, tc_max = 1;
    for (uint32_t i = 0; i < count; i++) {
        const FwdArgs& a = f[i];
        GemvLayerI8& ly = b.layer[i];
        ly.codes = static_cast<const uint8_t*>(a.codes);
        ly.scales = a.scales;
        ly.bias = a.bias;
        ly.x = static_cast<const uint16_t*>(a.x);
        ly.y = a.y;
        ly.N = (uint32_t)a.out_dim;
        ly.rows_per_item = rpi;
        ly.item0 = items;
        ly.gr = (uint32_t)(a.gr > 0xFFFFFFFFull ? 0xFFFFFFFFull : a.gr);
        ly.gc = (uint32_t)(a.gc > 0xFFFFFFFFull ? 0xFFFFFFFFull : a.gc);
        ly.tc = (uint32_t)a.tc;
        ly.ldx = a.x_stride ? (uint32_t)a.x_stride : K;
        ly.kvalid = a.k_valid ? (uint32_t)a.k_valid : K;
        items += (ly.N + rpi - 1) / rpi;
        // scale rows an item of rpi rows can span, and whether every item's scale rows start on a 16-byte boundary
        const uint32_t span = ly.gr >= rpi ? 2 : (rpi + ly.gr - 1) / ly.gr + 1;
        srows_max = span > srows_max ? span : srows_max;
        tc_max = ly.tc > tc_max ? ly.tc : tc_max;
        if ((reinterpret_cast<uintptr_t>(ly.scales) & 15u) || (ly.tc & 3u)) b.async_scales = 1;
    }
    if ((items + 147) / 148 > REG_MAX_ITEMS) return QB200_ERR_NOT_SUPPORTED;
    b.status = status;
    b.count = count;
    b.total_items = items;
    b.M = M;
    b.K = K;
    b.srows_max = srows_max;
    b.red_cols = M <= 2 ? 2 : (M + 3) & ~3u;
    b.red_stride = async_red_stride(b.red_cols);
    const uint32_t ctas = items < 148 ? items : 148, per_cta = (items + ctas - 1) / ctas;
    uint32_t stages = per_cta < 2 ? 2 : (per_cta > 4 ? 4 : per_cta);
    while (stages > 2 && i8_smem_layout(K, b.red_stride, srows_max, tc_max, stages).total > 227u * 1024) stages--;
    b.stages = stages;
    const uint32_t smem = i8_smem_layout(K, b.red_stride, srows_max, tc_max, stages).total;
    if (smem > 227u * 1024) return QB200_ERR_NOT_SUPPORTED;
    if (M > 4) return y_dtype == QB200_F32 ? launch_gemv_i8<2, float>(b, smem, ctas, st) : launch_gemv_i8<2, uint16_t>(b, smem, ctas, st);
    return y_dtype == QB200_F32 ? launch_gemv_i8<1, float>(b, smem, ctas, st) : launch_gemv_i8<1, uint16_t>(b, smem, ctas, st);
}

qb200_status gemv_i4_forward(const FwdArgs& f, int y_dtype, int32_t* status, cudaStream_t st) {
    return gemv_i4_forward_many(&f, 1, y_dtype, status, st, nullptr);
}

}  // namespace qb
