// The kernel body of the register-resident decode GEMV (see gemv_reg.cuh).
#pragma once

namespace qb {

// OCC: CTAs per SM the register budget is sized for (2 lets the serial per-item phases of two
// CTAs overlap; the 16-column batch tile needs the full register file and runs with 1).
// RB: 16-row blocks per work item (2 halves the per-item bookkeeping per weight).
template <int NT, int RB, int OCC, typename YT>
__global__ void __launch_bounds__(REG_THREADS, OCC) k_gemv_i4_reg(const __grid_constant__ GemvBatch a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t BATCH = NT * 8;
    const uint32_t groups = a.K >> 7, row_bytes = a.K >> 1, S = a.stages;
    const RegSmem L = reg_smem_layout(a.K, NT, RB, S);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    float* s_red = reinterpret_cast<float*>(smem + L.red);
    RegItem* s_desc = reinterpret_cast<RegItem*>(smem + L.desc);     // one per item of this CTA

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    // a CTA takes a contiguous run of items: neighbours in a layer, so the activation fragments are reloaded
    // only where the run crosses into a layer with another input
    const uint32_t per_cta = a.total_items / gridDim.x, extra = a.total_items % gridDim.x;
    const uint32_t n_my = per_cta + (blockIdx.x < extra ? 1u : 0u);
    const uint32_t item_first = blockIdx.x * per_cta + min(blockIdx.x, extra);
    const bool async_scales = a.async_scales != 0;  // scales not 16-byte aligned: 4-byte async copies
    // this warp's two scale groups (the second may not exist for short K)
    const uint32_t G0 = warp, G1 = warp + REG_WARPS;
    const bool v0 = G0 < groups, v1 = G1 < groups;
    const uint32_t G0c = v0 ? G0 : 0, G1c = v1 ? G1 : 0;

    // Every item this CTA will process is described once, up front (thread i describes item i).
    for (uint32_t j = tid; j < n_my; j += REG_THREADS) {
        const uint32_t item = item_first + j;
        uint32_t l = 0;
        while (l + 1 < a.count && item >= a.layer[l + 1].item0) l++;
        const GemvLayer& ly = a.layer[l];
        RegItem d;
        d.row0 = (item - ly.item0) * ly.rows_per_item;
        d.nrows = min(ly.rows_per_item, ly.N - d.row0);
        d.N = ly.N;
        d.x = ly.x;
        d.y = ly.y;
        d.bias = ly.bias;
        d.codes = reinterpret_cast<const uint8_t*>(ly.codes) + (uint64_t)d.row0 * row_bytes;
        d.scales = ly.scales + (uint64_t)d.row0 * groups;
        s_desc[j] = d;
    }
    // Issues the copies of item j into its stage: ONE bulk copy for the codes and one for the
    // scales (unaligned scales: 4-byte async copies by the warp's lanes, counted on the barrier).
    // Called by one whole warp; the warps take turns so no warp is the slow one at every barrier.
    auto issue = [&](uint32_t j, uint32_t stage) {
        const RegItem& d = s_desc[j];
        if (lane == 0) {
            mbar_expect_tx(&bars[stage], d.nrows * row_bytes + (async_scales ? 0 : d.nrows * groups * 4));
            bulk_g2s(smem + L.codes + stage * L.stage_codes, d.codes, d.nrows * row_bytes, &bars[stage]);
            if (!async_scales) bulk_g2s(smem + L.scales + stage * L.stage_scales, d.scales, d.nrows * groups * 4, &bars[stage]);
        }
        if (async_scales) {
            const uint32_t sc = smem_u32(smem + L.scales + stage * L.stage_scales);
            for (uint32_t i = lane; i < d.nrows * groups; i += 32)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sc + i * 4), "l"(d.scales + i) : "memory");
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars[stage])) : "memory");
        }
    };

    if (tid == 0) {
        for (uint32_t s = 0; s < S; s++) mbar_init(&bars[s], async_scales ? 1 + 32 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0)
        for (uint32_t j = 0; j < S && j < n_my; j++) issue(j, j);
    // The codes and scales do not depend on the previous kernel; everything below may.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    uint4 fa[NT][4], fb[NT][4];  // activation fragments of groups G0 / G1
    float ka[NT][2], kb[NT][2];  // their "+ 8" corrections for batch columns 2t, 2t + 1, in MMA units
    const uint16_t* cur_x = nullptr;
    uint32_t st = 0, parity = 0, red_sel = 0;
    bool failed = false;

    for (uint32_t j = 0; j < n_my; j++) {
        if (!mbar_try_wait(&bars[st], parity) && !mbar_wait_bounded(&bars[st], parity)) failed = true;
        const RegItem& it = s_desc[j];
        if (it.x != cur_x && !failed) {  // uniform across the CTA: (re)load this warp's fragments
            cur_x = it.x;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint32_t b = g + 8 * nt;
                float s0 = load_fragment(cur_x, a.K, b, G0c, t, v0 && b < a.M, fa[nt]);
                float s1 = load_fragment(cur_x, a.K, b, G1c, t, v1 && b < a.M, fb[nt]);
                s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 1);
                s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 2);
                s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 1);
                s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 2);
                // lane 8t (+4) holds batch row 2t (+1)
                ka[nt][0] = GEMV_EIGHT_X * __shfl_sync(0xFFFFFFFFu, s0, 8 * t);
                ka[nt][1] = GEMV_EIGHT_X * __shfl_sync(0xFFFFFFFFu, s0, 8 * t + 4);
                kb[nt][0] = GEMV_EIGHT_X * __shfl_sync(0xFFFFFFFFu, s1, 8 * t);
                kb[nt][1] = GEMV_EIGHT_X * __shfl_sync(0xFFFFFFFFu, s1, 8 * t + 4);
            }
        }

        float* red = s_red + red_sel * (REG_WARPS * RB * 16 * BATCH);
#pragma unroll
        for (int rb = 0; rb < RB; rb++) {
        const uint8_t* codes = smem + L.codes + st * L.stage_codes + (rb * 16 + g) * row_bytes + t * 16;
        const float* sc = reinterpret_cast<const float*>(smem + L.scales + st * L.stage_scales) + (rb * 16 + g) * groups;
        float acc[NT][4];
        if (!failed) {
            const uint4 c0a = *reinterpret_cast<const uint4*>(codes + G0c * 64);
            const uint4 c1a = *reinterpret_cast<const uint4*>(codes + 8 * row_bytes + G0c * 64);
            const uint4 c0b = *reinterpret_cast<const uint4*>(codes + G1c * 64);
            const uint4 c1b = *reinterpret_cast<const uint4*>(codes + 8 * row_bytes + G1c * 64);
            const float s0a = sc[G0c], s1a = sc[8 * groups + G0c], s0b = v1 ? sc[G1c] : 0.0f,
                        s1b = v1 ? sc[8 * groups + G1c] : 0.0f;
            float pa[NT][4], pb[NT][4];  // one MMA chain per group (and batch tile)
#define QB_STEP(J, W0A, W1A, W0B, W1B, FIRST)                                                \
    {                                                                                        \
        {                                                                                    \
            QB_UNPACK(W0A, W1A)                                                              \
            _Pragma("unroll") for (int nt = 0; nt < NT; nt++) {                              \
                if (FIRST) mma_bf16_first(pa[nt], a0, a1, a2, a3, fa[nt][J].x, fa[nt][J].y); \
                else mma_bf16(pa[nt], a0, a1, a2, a3, fa[nt][J].x, fa[nt][J].y);             \
                mma_bf16(pa[nt], d0, d1, d2, d3, fa[nt][J].z, fa[nt][J].w);                  \
            }                                                                                \
        }                                                                                    \
        {                                                                                    \
            QB_UNPACK(W0B, W1B)                                                              \
            _Pragma("unroll") for (int nt = 0; nt < NT; nt++) {                              \
                if (FIRST) mma_bf16_first(pb[nt], a0, a1, a2, a3, fb[nt][J].x, fb[nt][J].y); \
                else mma_bf16(pb[nt], a0, a1, a2, a3, fb[nt][J].x, fb[nt][J].y);             \
                mma_bf16(pb[nt], d0, d1, d2, d3, fb[nt][J].z, fb[nt][J].w);                  \
            }                                                                                \
        }                                                                                    \
    }
            QB_STEP(0, c0a.x, c1a.x, c0b.x, c1b.x, true)
            QB_STEP(1, c0a.y, c1a.y, c0b.y, c1b.y, false)
            QB_STEP(2, c0a.z, c1a.z, c0b.z, c1b.z, false)
            QB_STEP(3, c0a.w, c1a.w, c0b.w, c1b.w, false)
#undef QB_STEP
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    // (p - 8 * sum x) is the group's sum of q * x in MMA units (2^-93); 2^93 is applied at the store
                    const float da = pa[nt][i] - ka[nt][i & 1], db = pb[nt][i] - kb[nt][i & 1];
                    acc[nt][i] = fmaf(i < 2 ? s0b : s1b, db, (i < 2 ? s0a : s1a) * da);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;
        }

        // fold the K slices of the warps through red[red_sel][warp][row][batch]
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float* base = red + (warp * RB * 16 + rb * 16) * BATCH + nt * 8;
            *reinterpret_cast<float2*>(base + g * BATCH + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<float2*>(base + (g + 8) * BATCH + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
        }
        }  // rb
        if (__syncthreads_or(failed ? 1 : 0)) {
            failed = true;
            break;
        }
        // the stage just consumed is free: refill it S items ahead (the warps take turns)
        if (j + S < n_my && warp == ((j + 1) & (REG_WARPS - 1))) issue(j + S, st);
        // threads 0 .. RB * 16 * BATCH - 1 each finish one (row, batch column)
        for (uint32_t e = tid; e < RB * 16 * BATCH; e += REG_THREADS) {
            const uint32_t r = e / BATCH, b = e % BATCH;
            if (r < it.nrows && b < a.M) {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < REG_WARPS; w++) v += red[(w * RB * 16 + r) * BATCH + b];
                v *= GEMV_UNSCALE;
                const uint32_t n = it.row0 + r;
                if (it.bias) v += it.bias[n];
                store_y<YT>(static_cast<YT*>(it.y) + (uint64_t)b * it.N + n, v);
            }
        }
        red_sel ^= 1;
        if (++st == S) {
            st = 0;
            parity ^= 1;
        }
    }
    if (failed) {
        // A copy never completed: record it, give copies still in flight a bounded chance to land, leave.
        if (tid == 0) atomicExch(a.status, QB200_ERR_TIMEOUT);
        for (uint32_t s = 0; s < S; s++) mbar_wait_bounded(&bars[s], 0);
    }
}

}  // namespace qb
