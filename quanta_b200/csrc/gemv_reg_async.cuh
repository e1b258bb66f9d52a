// Decode GEMV, register-resident activations (see gemv_reg.cuh), with the cross-warp fold and the
// refills taken off the compute warps: sixteen compute warps never wait for one another — each
// waits for its item's codes, runs its two scale groups, parks its partial sums in one of two
// shared-memory slots and arrives on the slot's barrier — and a seventeenth (service) warp waits
// for that barrier, refills the stage the item occupied, folds the sixteen partial sums per
// output and stores.  The kernel is bound by the latency of each warp's own chain (copy landed
// -> LDS -> unpack -> MMA chain -> store), so anything that a compute warp has to wait for
// besides its own data costs bandwidth; a CTA-wide barrier per item did.
#pragma once

namespace qb {

constexpr uint32_t ASYNC_THREADS = REG_THREADS + 32;

// shared-memory accesses and barrier polls on 32-bit shared addresses
__device__ __forceinline__ uint4 async_lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float async_lds32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void async_sts64(uint32_t a, float x, float y) {
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(a), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ bool async_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool async_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < GEMV_SPIN_LIMIT; i++)
        if (async_try_wait(bar, parity)) return true;
    return false;
}

template <int NT, int RB, typename YT>
__global__ void __launch_bounds__(ASYNC_THREADS, 1) k_gemv_i4_async(const __grid_constant__ GemvBatch a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t groups = a.K >> 7, row_bytes = a.K >> 1, S = a.stages;
    const uint32_t BW = a.red_cols;                 // batch columns kept per row of partial sums (>= M, even)
    const uint32_t SLOT = REG_WARPS * RB * 16 * BW;  // floats per slot of partial sums
    const RegSmem L = reg_smem_layout(a.K, NT, RB, S, BW);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [S] codes landed
    uint64_t* done = bars + 8;                           // [2] all compute warps have parked the item's partial sums
    uint64_t* vacant = bars + 10;                        // [2] the service warp has folded the slot
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
    // a compute warp's two scale groups (the second may not exist for short K)
    const uint32_t G0 = warp, G1 = warp + REG_WARPS;
    const bool v0 = G0 < groups, v1 = G1 < groups;
    const uint32_t G0c = v0 ? G0 : 0, G1c = v1 ? G1 : 0;

    // Every item this CTA will process is described once, up front (thread i describes item i).
    for (uint32_t j = tid; j < n_my; j += ASYNC_THREADS) {
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
    // Called by the whole service warp.
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
        for (uint32_t s = 0; s < 2; s++) {
            mbar_init(&done[s], REG_WARPS);
            mbar_init(&vacant[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == REG_WARPS)
        for (uint32_t j = 0; j < S && j < n_my; j++) issue(j, j);
    // The codes and scales do not depend on the previous kernel; everything below may.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    bool failed = false;
    if (warp == REG_WARPS) {
        // ---- service warp: refill, fold, store ----
        uint32_t st = 0;
        for (uint32_t j = 0; j < n_my; j++) {
            const uint32_t slot = j & 1;
            if (!mbar_wait_bounded(&done[slot], (j >> 1) & 1)) { failed = true; break; }
            if (j + S < n_my) issue(j + S, st);  // every compute warp has left the stage
            const RegItem& it = s_desc[j];
            const float* red = s_red + slot * SLOT;
            for (uint32_t r = lane; r < RB * 16; r += 32) {  // lane = output row: consecutive lanes, consecutive outputs
                if (r < it.nrows) {
                    const uint32_t n = it.row0 + r;
                    const float bias = it.bias ? it.bias[n] : 0.0f;
                    for (uint32_t b = 0; b < a.M; b++) {
                        float v = 0.0f;
#pragma unroll
                        for (int w = 0; w < REG_WARPS; w++) v += red[(w * RB * 16 + r) * BW + b];
                        YT* yp = static_cast<YT*>(it.y) + (uint64_t)b * it.N + n;
                        const float out = fmaf(v, GEMV_UNSCALE, bias);
                        if (a.n_peers == 0) {
                            store_y<YT>(yp, out);
                        } else {  // fused all-gather: the same element of every rank's buffer (peer memory over NVLink)
                            for (uint32_t p = 0; p < a.n_peers; p++)
                                store_y<YT>(reinterpret_cast<YT*>(reinterpret_cast<uint8_t*>(yp) + a.peer_delta[p]), out);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&vacant[slot]);
            if (++st == S) st = 0;
        }
        // Fused all-gather with the arrival barrier inside the launch: the CTA that finishes last tells every
        // peer "this rank's outputs of this step are written" and waits, bounded, for theirs, so the launch ends
        // when all ranks' outputs are here.  flags[p] is rank p's array {arrival of rank 0..7, step counter,
        // count of finished CTAs}.
        if (a.n_peers && a.peer_flags[0]) {
            __threadfence_system();  // this CTA's peer stores before its count
            uint32_t last = 0;
            uint64_t* mine = a.peer_flags[a.rank];
            if (lane == 0) last = atomicAdd(reinterpret_cast<unsigned int*>(mine + 9), 1u) == gridDim.x - 1 ? 1u : 0u;
            last = __shfl_sync(0xFFFFFFFFu, last, 0);
            if (last) {
                __threadfence_system();  // the other CTAs' stores (ordered before their counts) before the flags
                uint64_t step = 0;
                if (lane == 0) {
                    *reinterpret_cast<unsigned int*>(mine + 9) = 0;
                    step = mine[8] + 1;
                    mine[8] = step;
                }
                step = __shfl_sync(0xFFFFFFFFu, step, 0);
                if (lane < a.n_peers) {
                    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.peer_flags[lane] + a.rank), "l"(step) : "memory");
                    uint64_t v = 0;
                    uint32_t spins = 0;
                    for (;;) {
                        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine + lane) : "memory");
                        if (v >= step || ++spins >= (4u << 20)) break;
                        __nanosleep(200);
                    }
                    if (v < step) atomicExch(a.status, QB200_ERR_TIMEOUT);
                }
                __threadfence_system();
            }
        }
    } else {
        // ---- compute warps ----
        // The item loop works on 32-bit shared-memory addresses that are advanced, not recomputed:
        // every instruction here is paid 16 x 28 times per CTA and layer.
        uint4 fa[NT][4], fb[NT][4];  // activation fragments of groups G0 / G1
        float ka[NT][2], kb[NT][2];  // their "+ 8" corrections for batch columns 2t, 2t + 1, in MMA units
        const uint16_t* cur_x = nullptr;
        const uint32_t bar0 = smem_u32(bars), done0 = smem_u32(done), vacant0 = smem_u32(vacant);
        const uint32_t desc0 = smem_u32(s_desc);  // the item's activation pointer is the first field of its descriptor
        // offsets inside a stage of this lane's four 16-byte code loads and four scales (row g / g + 8, group G0 / G1)
        const uint32_t codes0 = smem_u32(smem + L.codes) + g * row_bytes + t * 16, scales0 = smem_u32(smem + L.scales) + g * groups * 4;
        const uint32_t oc0 = G0c * 64, oc1 = 8 * row_bytes + G0c * 64, oc2 = G1c * 64, oc3 = 8 * row_bytes + G1c * 64;
        const uint32_t os0 = G0c * 4, os1 = (8 * groups + G0c) * 4, os2 = G1c * 4, os3 = (8 * groups + G1c) * 4;
        const uint32_t rb_codes = 16 * row_bytes, rb_scales = 16 * groups * 4;
        // where this lane parks its partial sums inside a slot: row g (and g + 8) of row block rb, columns 2t, 2t + 1
        const uint32_t red0 = smem_u32(s_red) + ((warp * RB * 16 + g) * BW + 2 * t) * 4;
        const bool keeps = 2 * t < BW;  // NT == 1: columns past the batch are not kept
        uint32_t st = 0, parity = 0, stage_codes = codes0, stage_scales = scales0;
        for (uint32_t j = 0; j < n_my; j++) {
            if (!async_try_wait(bar0 + st * 8, parity) && !async_wait_bounded(bar0 + st * 8, parity)) { failed = true; break; }
            const uint32_t slot = j & 1, vpar = ((j >> 1) & 1) ^ 1;
            // the slot's previous item has long been folded: polled here so that its latency overlaps the loads
            if (j >= 2 && !async_try_wait(vacant0 + slot * 8, vpar) && !async_wait_bounded(vacant0 + slot * 8, vpar)) { failed = true; break; }
            const uint16_t* x_now;
            asm volatile("ld.shared.u64 %0, [%1];" : "=l"(x_now) : "r"(desc0 + j * (uint32_t)sizeof(RegItem)));
            if (x_now != cur_x) {  // uniform across the CTA: (re)load this warp's fragments
                cur_x = x_now;
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
            // every load of the item first
            uint4 c[RB][4];
            float sc[RB][4];
#pragma unroll
            for (int rb = 0; rb < RB; rb++) {
                const uint32_t cr = stage_codes + rb * rb_codes, sr = stage_scales + rb * rb_scales;
                c[rb][0] = async_lds128(cr + oc0);
                c[rb][1] = async_lds128(cr + oc1);
                c[rb][2] = async_lds128(cr + oc2);
                c[rb][3] = async_lds128(cr + oc3);
                sc[rb][0] = async_lds32(sr + os0);
                sc[rb][1] = async_lds32(sr + os1);
                sc[rb][2] = v1 ? async_lds32(sr + os2) : 0.0f;
                sc[rb][3] = v1 ? async_lds32(sr + os3) : 0.0f;
            }
            // 2 * RB independent MMA chains (row block x group), interleaved step by step
            float pa[RB][NT][4], pb[RB][NT][4];
#define QB_STEP(J, X, FIRST)                                                                         \
    _Pragma("unroll") for (int rb = 0; rb < RB; rb++) {                                              \
        {                                                                                            \
            QB_UNPACK(c[rb][0].X, c[rb][1].X)                                                        \
            _Pragma("unroll") for (int nt = 0; nt < NT; nt++) {                                      \
                if (FIRST) mma_bf16_first(pa[rb][nt], a0, a1, a2, a3, fa[nt][J].x, fa[nt][J].y);     \
                else mma_bf16(pa[rb][nt], a0, a1, a2, a3, fa[nt][J].x, fa[nt][J].y);                 \
                mma_bf16(pa[rb][nt], d0, d1, d2, d3, fa[nt][J].z, fa[nt][J].w);                      \
            }                                                                                        \
        }                                                                                            \
        {                                                                                            \
            QB_UNPACK(c[rb][2].X, c[rb][3].X)                                                        \
            _Pragma("unroll") for (int nt = 0; nt < NT; nt++) {                                      \
                if (FIRST) mma_bf16_first(pb[rb][nt], a0, a1, a2, a3, fb[nt][J].x, fb[nt][J].y);     \
                else mma_bf16(pb[rb][nt], a0, a1, a2, a3, fb[nt][J].x, fb[nt][J].y);                 \
                mma_bf16(pb[rb][nt], d0, d1, d2, d3, fb[nt][J].z, fb[nt][J].w);                      \
            }                                                                                        \
        }                                                                                            \
    }
            QB_STEP(0, x, true)
            QB_STEP(1, y, false)
            QB_STEP(2, z, false)
            QB_STEP(3, w, false)
#undef QB_STEP
            // park the partial sums in red[slot][warp][row][batch]: (p - 8 * sum x) is the group's sum of q * x in
            // MMA units (2^-93); 2^93 is applied at the store
            const uint32_t ra = red0 + slot * (SLOT * 4);
#pragma unroll
            for (int rb = 0; rb < RB; rb++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    float o[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float da = pa[rb][nt][i] - ka[nt][i & 1], db = pb[rb][nt][i] - kb[nt][i & 1];
                        o[i] = fmaf(sc[rb][i < 2 ? 2 : 3], db, sc[rb][i < 2 ? 0 : 1] * da);
                    }
                    if (nt == 0 ? keeps : nt * 8 + 2 * t < BW) {
                        async_sts64(ra + (rb * 16 * BW + nt * 8) * 4, o[0], o[1]);
                        async_sts64(ra + ((rb * 16 + 8) * BW + nt * 8) * 4, o[2], o[3]);
                    }
                }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(done0 + slot * 8) : "memory");  // releases the stage, publishes the sums
            stage_codes += L.stage_codes;
            stage_scales += L.stage_scales;
            if (++st == S) {
                st = 0;
                parity ^= 1;
                stage_codes = codes0;
                stage_scales = scales0;
            }
        }
    }
    if (failed) {
        // A wait ran out: record it, give copies still in flight a bounded chance to land, leave.
        if (lane == 0) atomicExch(a.status, QB200_ERR_TIMEOUT);
        for (uint32_t s = 0; s < S; s++) mbar_wait_bounded(&bars[s], 0);
    }
}

}  // namespace qb
