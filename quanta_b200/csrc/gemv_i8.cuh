// Decode GEMV over int8 codes (M <= 8, K <= 4096): y[m, n] = sum_k x[m, k] * s(n, k) * q[n, k] with codes `[N, K]`
// (one byte each, crates/sci/quanta-array/src/quant.rs:27-30) and ANY scale grid whose tile width is a multiple of 32
// (32 x 32 blocks, 1 x 128 groups, per-row, per-tensor, ...).  Same pipeline as the int4 kernel (gemv_reg_async.cuh):
// persistent CTAs, a ring of bulk-copied stages, sixteen compute warps that own two 128-k column groups each and keep
// their activation fragments in registers, service warps that fold and store.  What differs:
//
//   - The operand.  A byte with its sign bit flipped is an unsigned 0..255 in the low byte of a 16-bit lane, and a
//     bf16 whose exponent field is 0 or 1 is linear in its bit pattern, so `(w & 0x00FF00FF) ^ 0x00800080` IS the
//     exact operand pair (q + 128) * 2^-133 for bytes 0 and 2 of a word, and the same on `w >> 8` for bytes 1 and 3:
//     three integer instructions per four codes.  The "+ 128" leaves as 128 * sum(x) per run of 32 columns.
//   - The scale may change every 32 columns, so the sixteen k-slots of one MMA must lie in one 32-column run: a lane
//     owns 8 consecutive bytes of every run (two MMAs per run), not 32 contiguous bytes of the group, and each run's
//     pair of MMAs starts a fresh accumulator that is scaled into the row's sum (`acc += s * (p - 128 sum x)`).
//   - Those 8-byte reads of four rows per half-warp would all hit the same banks if the rows lay K bytes apart (K is
//     a multiple of 128), so a stage keeps its rows K + 32 bytes apart and an item is one bulk copy PER ROW (4 KB for
//     K = 4096) instead of one per item.
//   - An item is a 16-row block; its scale rows (1 for 32-row tiles, 16 for per-row scales) are staged beside it.
#pragma once

namespace qb {

constexpr uint32_t I8_ROW_PAD = 32;  // bytes between the end of a staged row and the next one

struct GemvLayerI8 {
    const uint8_t* codes;   // [N, K] int8
    const float* scales;    // [ceil(N / gr), tc]
    const float* bias;      // [N] or null
    const uint16_t* x;      // bf16 [M, K], rows ldx elements apart
    void* y;                // [M, N] f32 or bf16
    uint32_t N, rows_per_item, item0;
    uint32_t gr, gc, tc;    // scale tile and the row length of the scale grid
    uint32_t ldx, kvalid;   // x's row stride; columns >= kvalid of x do not exist and read as zero (a multiple of 32)
};
constexpr int I8_MAX_LAYERS = 32;
struct GemvBatchI8 {
    GemvLayerI8 layer[I8_MAX_LAYERS];
    int32_t* status;
    uint32_t count, total_items, M, K, stages;
    uint32_t red_cols, red_stride;
    uint32_t srows_max;      // scale rows a stage holds room for
    uint32_t async_scales;   // some item's scale rows are not 16-byte aligned: 4-byte copies
};

struct I8Item {
    const uint16_t* x;
    void* y;
    const float* bias;
    const uint8_t* codes;
    const float* scales;   // first scale row of the item
    uint32_t row0, nrows, N, layer;
    uint32_t n_srows, pad;
};

struct I8Smem {
    uint32_t desc, red, scales, codes, total, stage_scales, stage_codes, slot_floats, row_stride;
};
__host__ __device__ inline I8Smem i8_smem_layout(uint32_t K, uint32_t red_stride, uint32_t srows_max, uint32_t tc_max, uint32_t stages) {
    I8Smem L;
    auto up = [](uint32_t v) { return (v + 127u) & ~127u; };
    L.desc = 128;
    L.red = L.desc + up(REG_MAX_ITEMS * (uint32_t)sizeof(I8Item));
    L.slot_floats = REG_WARPS * 16 * red_stride;
    L.scales = L.red + up(ASYNC_SLOTS * L.slot_floats * 4);
    L.stage_scales = up(srows_max * tc_max * 4);
    L.codes = L.scales + stages * L.stage_scales;
    L.row_stride = K + I8_ROW_PAD;
    L.stage_codes = up(16 * L.row_stride);
    L.total = L.codes + stages * L.stage_codes;
    return L;
}

#define GEMV_I8_OFFSET_X 1.2924697071141057e-26f  // 128 * 2^-93: the "+ 128" in units of the MMA partial sums

// Activation fragment of one 128-column group for batch row b: this lane's 8 consecutive columns of each of the four
// 32-column runs, ordered as the two MMAs of a run want them ({k0, k2}, {k1, k3}, {k4, k6}, {k5, k7}), scaled by 2^40;
// sums[j] receives the plain sum of the lane's 8 activations of run j.
__device__ __forceinline__ void load_fragment_i8(const uint16_t* __restrict__ x, uint32_t ldx, uint32_t kvalid, uint32_t b, uint32_t G,
                                                 uint32_t t, bool valid, uint4 (&frag)[4], float (&sums)[4], bool& out_of_domain) {
    uint32_t klo = X_SCALE_LO;
    const __nv_bfloat162 s40 = *reinterpret_cast<const __nv_bfloat162*>(&klo);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint4 v = make_uint4(0, 0, 0, 0);  // 8 consecutive bf16
        if (valid && G * 128 + j * 32 < kvalid) v = __ldg(reinterpret_cast<const uint4*>(x + (uint64_t)b * ldx + G * 128 + j * 32 + t * 8));
        const uint32_t xr[4] = {v.x, v.y, v.z, v.w};
        float sum = 0.0f;
        uint32_t top = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            sum += bf16_bits_to_f32(xr[i] & 0xFFFFu) + bf16_bits_to_f32(xr[i] >> 16);
            top = max(top, max(xr[i] & 0x7F80u, (xr[i] >> 16) & 0x7F80u));
        }
        if (top >= ((127u + 87u) << 7)) out_of_domain = true;
        sums[j] = sum;
        uint32_t o[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {  // words (k0 k1)(k2 k3) -> (k0 k2), (k1 k3)
            uint32_t even = __byte_perm(xr[2 * h], xr[2 * h + 1], 0x5410), odd = __byte_perm(xr[2 * h], xr[2 * h + 1], 0x7632);
            __nv_bfloat162 e2 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&even), s40);
            __nv_bfloat162 o2 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&odd), s40);
            o[2 * h] = *reinterpret_cast<uint32_t*>(&e2);
            o[2 * h + 1] = *reinterpret_cast<uint32_t*>(&o2);
        }
        frag[j] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__device__ __forceinline__ uint2 i8_lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

constexpr uint32_t I8_BYTES = 0x00FF00FFu, I8_SIGN = 0x00800080u;

template <int NSERV, typename YT>
__global__ void __launch_bounds__(REG_THREADS + 32 * NSERV, 1) k_gemv_i8_async(const __grid_constant__ GemvBatchI8 a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t groups = a.K >> 7, S = a.stages, BW = a.red_cols, RS = a.red_stride;
    uint32_t tc_max = 0;
    for (uint32_t l = 0; l < a.count; l++) tc_max = max(tc_max, a.layer[l].tc);
    const I8Smem L = i8_smem_layout(a.K, RS, a.srows_max, tc_max, S);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    uint64_t* done = bars + 8;
    uint64_t* vacant = bars + 8 + ASYNC_SLOTS;
    float* s_red = reinterpret_cast<float*>(smem + L.red);
    I8Item* s_desc = reinterpret_cast<I8Item*>(smem + L.desc);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t per_cta = a.total_items / gridDim.x, extra = a.total_items % gridDim.x;
    const uint32_t n_my = per_cta + (blockIdx.x < extra ? 1u : 0u);
    const uint32_t item_first = blockIdx.x * per_cta + min(blockIdx.x, extra);
    const bool async_scales = a.async_scales != 0;

    for (uint32_t j = tid; j < n_my; j += REG_THREADS + 32 * NSERV) {
        const uint32_t item = item_first + j;
        uint32_t l = 0;
        while (l + 1 < a.count && item >= a.layer[l + 1].item0) l++;
        const GemvLayerI8& ly = a.layer[l];
        I8Item d;
        d.row0 = (item - ly.item0) * ly.rows_per_item;
        d.nrows = min(ly.rows_per_item, ly.N - d.row0);
        d.N = ly.N;
        d.layer = l;
        d.x = ly.x;
        d.y = ly.y;
        d.bias = ly.bias;
        d.codes = ly.codes + (uint64_t)d.row0 * a.K;
        const uint32_t sr0 = d.row0 / ly.gr;
        d.scales = ly.scales + (uint64_t)sr0 * ly.tc;
        d.n_srows = (d.row0 + d.nrows - 1) / ly.gr - sr0 + 1;
        d.pad = 0;
        s_desc[j] = d;
    }
    // item j -> its stage: one bulk copy per row (lane r copies row r into the padded stage), one for the scale rows
    auto issue = [&](uint32_t j, uint32_t stage) {
        const I8Item& d = s_desc[j];
        const uint32_t sbytes = d.n_srows * a.layer[d.layer].tc * 4;
        if (lane == 0) mbar_expect_tx(&bars[stage], d.nrows * a.K + (async_scales ? 0 : sbytes));
        __syncwarp();
        if (lane < d.nrows)
            bulk_g2s(smem + L.codes + stage * L.stage_codes + lane * L.row_stride, d.codes + (uint64_t)lane * a.K, a.K, &bars[stage]);
        if (!async_scales) {
            if (lane == 16) bulk_g2s(smem + L.scales + stage * L.stage_scales, d.scales, sbytes, &bars[stage]);
        } else {
            const uint32_t sc = smem_u32(smem + L.scales + stage * L.stage_scales);
            for (uint32_t i = lane; i < sbytes / 4; i += 32)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sc + i * 4), "l"(d.scales + i) : "memory");
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars[stage])) : "memory");
        }
    };

    if (tid == 0) {
        for (uint32_t s = 0; s < S; s++) mbar_init(&bars[s], async_scales ? 1 + 32 : 1);
        for (uint32_t s = 0; s < ASYNC_SLOTS; s++) {
            mbar_init(&done[s], REG_WARPS);
            mbar_init(&vacant[s], NSERV);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    bool failed = false;
    if (warp >= REG_WARPS) {
        const uint32_t sw = warp - REG_WARPS;
        if (sw == 0)
            for (uint32_t j = 0; j < S && j < n_my; j++) issue(j, j);
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // ---- service warps: refill, fold (a row and four batch columns per 16-byte read), store ----
        const uint32_t vec = BW < 4 ? BW : 4, units = 16 * ((BW + 3) / 4);
        uint32_t st = 0;
        for (uint32_t j = 0; j < n_my; j++) {
            const I8Item& it = s_desc[j];
            const uint32_t slot = j % ASYNC_SLOTS;
            if (!mbar_wait_bounded(&done[slot], (j / ASYNC_SLOTS) & 1)) { failed = true; break; }
            if (sw == 0 && j + S < n_my) issue(j + S, st);
            for (uint32_t u = sw * 32 + lane; u < units; u += NSERV * 32) {
                const uint32_t r = u % 16, b0 = (u / 16) * 4;
                if (r >= it.nrows || b0 >= a.M) continue;
                const float* red = s_red + slot * L.slot_floats + r * RS + b0;
                float v[4];
                fold_sixteen(red, 16 * RS, vec, v);
                const uint32_t n = it.row0 + r;
                const float bias = it.bias ? it.bias[n] : 0.0f;
#pragma unroll
                for (uint32_t i = 0; i < 4; i++)
                    if (i < vec && b0 + i < a.M) store_y<YT>(static_cast<YT*>(it.y) + (uint64_t)(b0 + i) * it.N + n, fmaf(v[i], GEMV_UNSCALE, bias));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&vacant[slot]);
            if (++st == S) st = 0;
        }
    } else {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // ---- compute warps ----
        const bool v0 = warp < groups, v1 = warp + REG_WARPS < groups;
        const uint32_t Ga = v0 ? warp : 0, Gb = v1 ? warp + REG_WARPS : 0;
        uint4 fa[4], fb[4];      // activation fragments of the two groups (batch row g)
        float ka[4][2], kb[4][2];  // 128 * sum(x) per run for batch columns 2t, 2t + 1, in MMA units
        const uint16_t* cur_x = nullptr;
        const uint32_t sm0 = smem_u32(smem);
        const uint32_t codes0 = smem_u32(smem + L.codes) + g * L.row_stride + t * 8, scales0 = smem_u32(smem + L.scales);
        const uint32_t c8 = 8 * L.row_stride;
        const uint32_t red0 = smem_u32(s_red) + ((warp * 16 + g) * RS + 2 * t) * 4;
        const bool keeps = 2 * t < BW;
        uint32_t st = 0, parity = 0;
        for (uint32_t j = 0; j < n_my; j++) {
            if (!async_try_wait(sm0 + st * 8, parity) && !async_wait_bounded(sm0 + st * 8, parity)) { failed = true; break; }
            const uint32_t slot = j % ASYNC_SLOTS, vpar = ((j / ASYNC_SLOTS) & 1) ^ 1, vac = sm0 + 64 + (ASYNC_SLOTS + slot) * 8;
            if (j >= ASYNC_SLOTS && !async_try_wait(vac, vpar) && !async_wait_bounded(vac, vpar)) { failed = true; break; }
            const I8Item& it = s_desc[j];
            const GemvLayerI8& ly = a.layer[it.layer];
            if (it.x != cur_x) {  // uniform across the CTA: (re)load this warp's fragments and the runs' sums
                cur_x = it.x;
                bool ood = false;
                float sa[4], sb[4];
                load_fragment_i8(cur_x, ly.ldx, ly.kvalid, g, Ga, t, v0 && g < a.M, fa, sa, ood);
                load_fragment_i8(cur_x, ly.ldx, ly.kvalid, g, Gb, t, v1 && g < a.M, fb, sb, ood);
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    float s0 = sa[r], s1 = sb[r];
                    s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 1);
                    s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 2);
                    s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 1);
                    s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 2);
                    ka[r][0] = GEMV_I8_OFFSET_X * __shfl_sync(0xFFFFFFFFu, s0, 8 * t);      // lane 8t (+4) holds batch row 2t (+1)
                    ka[r][1] = GEMV_I8_OFFSET_X * __shfl_sync(0xFFFFFFFFu, s0, 8 * t + 4);
                    kb[r][0] = GEMV_I8_OFFSET_X * __shfl_sync(0xFFFFFFFFu, s1, 8 * t);
                    kb[r][1] = GEMV_I8_OFFSET_X * __shfl_sync(0xFFFFFFFFu, s1, 8 * t + 4);
                }
                if (ood) atomicExch(a.status, QB200_ERR_INVALID_PARAM);
            }
            // scale rows of this lane's two weight rows, relative to the item's first staged scale row
            const uint32_t row_last = it.row0 + it.nrows - 1;  // rows past the item read its last row's scales (their sums are not stored)
            const uint32_t row_lo = min(it.row0 + g, row_last), row_hi = min(it.row0 + g + 8, row_last), sr0 = it.row0 / ly.gr;
            const uint32_t srow_lo = scales0 + st * L.stage_scales + (row_lo / ly.gr - sr0) * ly.tc * 4;
            const uint32_t srow_hi = scales0 + st * L.stage_scales + (row_hi / ly.gr - sr0) * ly.tc * 4;
            const uint32_t cbase = codes0 + st * L.stage_codes;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#define QB_I8_GROUP(G, F, KC, VALID)                                                                                       \
    {                                                                                                                      \
        uint2 c0[4], c1[4];                                                                                                \
        float s_lo[4], s_hi[4];                                                                                            \
        _Pragma("unroll") for (int r = 0; r < 4; r++) {                                                                    \
            c0[r] = i8_lds64(cbase + (G) * 128 + r * 32);                                                                  \
            c1[r] = i8_lds64(cbase + c8 + (G) * 128 + r * 32);                                                             \
            const uint32_t si = (((G) * 128 + r * 32) / ly.gc) * 4;                                                        \
            s_lo[r] = (VALID) ? async_lds32(srow_lo + si) : 0.0f;                                                          \
            s_hi[r] = (VALID) ? async_lds32(srow_hi + si) : 0.0f;                                                          \
        }                                                                                                                  \
        _Pragma("unroll") for (int r = 0; r < 4; r++) {                                                                    \
            float p[4];                                                                                                    \
            {                                                                                                              \
                const uint32_t w0 = c0[r].x, w1 = c1[r].x;                                                                 \
                mma_bf16_first(p, lop3_and_xor(w0, I8_BYTES, I8_SIGN), lop3_and_xor(w1, I8_BYTES, I8_SIGN),                \
                               lop3_and_xor(w0 >> 8, I8_BYTES, I8_SIGN), lop3_and_xor(w1 >> 8, I8_BYTES, I8_SIGN), F[r].x, F[r].y); \
            }                                                                                                              \
            {                                                                                                              \
                const uint32_t w0 = c0[r].y, w1 = c1[r].y;                                                                 \
                mma_bf16(p, lop3_and_xor(w0, I8_BYTES, I8_SIGN), lop3_and_xor(w1, I8_BYTES, I8_SIGN),                      \
                         lop3_and_xor(w0 >> 8, I8_BYTES, I8_SIGN), lop3_and_xor(w1 >> 8, I8_BYTES, I8_SIGN), F[r].z, F[r].w); \
            }                                                                                                              \
            acc[0] = fmaf(s_lo[r], p[0] - KC[r][0], acc[0]);                                                               \
            acc[1] = fmaf(s_lo[r], p[1] - KC[r][1], acc[1]);                                                               \
            acc[2] = fmaf(s_hi[r], p[2] - KC[r][0], acc[2]);                                                               \
            acc[3] = fmaf(s_hi[r], p[3] - KC[r][1], acc[3]);                                                               \
        }                                                                                                                  \
    }
            QB_I8_GROUP(Ga, fa, ka, v0)
            QB_I8_GROUP(Gb, fb, kb, v1)
#undef QB_I8_GROUP
            if (keeps) {
                const uint32_t ra = red0 + slot * (L.slot_floats * 4);
                async_sts64(ra, acc[0], acc[1]);
                async_sts64(ra + 8 * RS * 4, acc[2], acc[3]);
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sm0 + 64 + slot * 8) : "memory");
            if (++st == S) {
                st = 0;
                parity ^= 1;
            }
        }
    }
    if (failed) {
        if (lane == 0) atomicExch(a.status, QB200_ERR_TIMEOUT);
        for (uint32_t s = 0; s < S; s++) mbar_wait_bounded(&bars[s], 0);
    }
}

}  // namespace qb
