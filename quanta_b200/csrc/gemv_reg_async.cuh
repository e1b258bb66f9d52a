// Decode GEMV, register-resident activations (see gemv_reg.cuh), with the cross-warp fold and the
// refills taken off the compute warps: sixteen compute warps never wait for one another — each
// waits for its item's codes, runs its two scale groups, parks its partial sums in one of two
// shared-memory slots and arrives on the slot's barrier — and a seventeenth (service) warp waits
// for that barrier, refills the stage the item occupied, folds the sixteen partial sums per
// output and stores.  The kernel is bound by the latency of each warp's own chain (copy landed
// -> LDS -> unpack -> MMA chain -> store), so anything that a compute warp has to wait for
// besides its own data costs bandwidth; a CTA-wide barrier per item did.
//
// NT = 1 (batch <= 8): an item's RB row blocks are multiplied together (2 * RB interleaved MMA
// chains) and parked as one sub-item.  NT = 2 (batch <= 16): the activation fragments alone take
// half the register file, so a warp multiplies one 16-row block at a time (four chains: two
// groups x two batch tiles) and every row block is parked and folded as a sub-item of its own —
// which also keeps the slots of partial sums at 16 rows.
#pragma once

namespace qb {

// Threads per CTA: sixteen compute warps and the service warp.  With the 16-column batch tile the compute warps
// need more registers than an even split of the register file over 17 warps gives (registers are handed out per
// group of four warps, so 17 warps are budgeted as 20: 96 each), so that kernel is launched with a whole fifth
// warp group — three of its warps leave at once — which hands most of its registers to the compute warps.
constexpr uint32_t ASYNC_THREADS = REG_THREADS + 32, ASYNC_THREADS_WIDE = REG_THREADS + 128;
// The registers a warp group gains must have been given up by another group of the same CTA first (registers the
// CTA never held cannot be claimed; a request that cannot be met waits for ever).  640 threads start with 96 each.
constexpr uint32_t ASYNC_REGS_LAUNCH = 96, ASYNC_REGS_COMPUTE = 112, ASYNC_REGS_SERVICE = 32;
static_assert((ASYNC_REGS_LAUNCH - ASYNC_REGS_SERVICE) * 4 >= (ASYNC_REGS_COMPUTE - ASYNC_REGS_LAUNCH) * REG_WARPS,
              "the compute warps would wait for registers that nobody releases");
static_assert(ASYNC_THREADS_WIDE * ASYNC_REGS_LAUNCH <= 65536 && ASYNC_THREADS_WIDE * (ASYNC_REGS_LAUNCH + 8) > 65536,
              "the launch bound must make the compiler start every warp with ASYNC_REGS_LAUNCH registers");
#define QB_STR2(x) #x
#define QB_STR(x) QB_STR2(x)
// NSERV service warps share the fold of a sub-item (a single warp folding eight or more batch columns for sixteen
// partial sums each became the slowest stage of the pipeline).
__host__ __device__ constexpr uint32_t async_threads(int nt, int nserv) { return nt == 2 ? ASYNC_THREADS_WIDE : REG_THREADS + 32 * nserv; }

// Shared-memory carve-up of the service-warp kernel, identical on host and device.
// sub_rows: rows folded at a time; red_stride: floats between rows of a slot of partial sums.
constexpr uint32_t ASYNC_SLOTS = 2;  // slots of partial sums a CTA cycles through
struct AsyncSmem {
    uint32_t desc, red, scales, codes, total, stage_scales, stage_codes, slot_floats;
};
__host__ __device__ inline AsyncSmem async_smem_layout(uint32_t K, uint32_t rb, uint32_t sub_rows, uint32_t red_stride,
                                                       uint32_t stages) {
    AsyncSmem L;
    const uint32_t groups = K / 128;
    auto up = [](uint32_t v) { return (v + 127u) & ~127u; };
    L.desc = 128;  // barriers at 0: [S <= 8] codes landed, [2] slot parked, [2] slot folded
    L.red = L.desc + up(REG_MAX_ITEMS * (uint32_t)sizeof(RegItem));
    L.slot_floats = REG_WARPS * sub_rows * red_stride;
    L.scales = L.red + up(ASYNC_SLOTS * L.slot_floats * 4);
    L.stage_scales = up(rb * 16 * groups * 4);
    L.codes = L.scales + stages * L.stage_scales;
    L.stage_codes = up(rb * 16 * (K / 2));
    L.total = L.codes + stages * L.stage_codes;
    return L;
}
// Row stride of a slot for `cols` kept batch columns (2, 4 or a multiple of 4): the service warps read a row four
// columns at a time (16 bytes, lane = row), which is free of bank conflicts when the stride is an odd number of
// 16-byte units (padded by one unit where it would be even).
__host__ __device__ inline uint32_t async_red_stride(uint32_t cols) { return cols <= 2 ? cols : ((cols / 4) | 1u) * 4; }

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

// One unit of the service warps' fold: a row of a sub-item and up to four kept batch columns, summed over the sixteen
// compute warps' partial sums in warp order (`red` points at warp 0's row, the warps lie `warp_stride` floats apart).
__device__ __forceinline__ void fold_sixteen(const float* red, uint32_t warp_stride, uint32_t vec, float (&v)[4]) {
    v[0] = v[1] = v[2] = v[3] = 0.0f;
    if (vec == 4) {
#pragma unroll 4
        for (int w = 0; w < REG_WARPS; w++) {
            const float4 p = *reinterpret_cast<const float4*>(red + w * warp_stride);
            v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
        }
    } else {
#pragma unroll 4
        for (int w = 0; w < REG_WARPS; w++) {
            const float2 p = *reinterpret_cast<const float2*>(red + w * warp_stride);
            v[0] += p.x; v[1] += p.y;
        }
    }
}

// Barrier 2 over the CTA's `count` live threads (the warps that left early do not take part) with an OR of a predicate.
__device__ __forceinline__ uint32_t __syncthreads_or_live(bool pred, uint32_t count) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "bar.red.or.pred q, 2, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred), "r"(count)
        : "memory");
    return r;
}

template <int NT, int RB, int NSERV, typename YT>
__global__ void __launch_bounds__(async_threads(NT, NSERV), 1) k_gemv_i4_async(const __grid_constant__ GemvBatch a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int SUBS = NT == 2 ? RB : 1;  // sub-items (parked and folded separately) per item
    constexpr int RPS = RB / SUBS;          // row blocks per sub-item
    constexpr uint32_t SUB_ROWS = RPS * 16;
    const uint32_t groups = a.K >> 7, row_bytes = a.K >> 1, S = a.stages;
    const uint32_t BW = a.red_cols;             // batch columns kept per row of partial sums (>= M, even)
    const uint32_t RS = a.red_stride;           // floats between rows of a slot
    const AsyncSmem L = async_smem_layout(a.K, RB, SUB_ROWS, RS, S);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [S] codes landed
    uint64_t* done = bars + 8;                           // [slots] all compute warps have parked the sub-item's partial sums
    uint64_t* vacant = bars + 8 + ASYNC_SLOTS;           // [slots] the service warps have folded the slot
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

    // Every item this CTA will process is described once, up front (thread i describes item i).
    for (uint32_t j = tid; j < n_my; j += async_threads(NT, NSERV)) {
        const uint32_t item = item_first + j;
        uint32_t l = 0;
        while (l + 1 < a.count && item >= a.layer[l + 1].item0) l++;
        const GemvLayer& ly = a.layer[l];
        RegItem d;
        d.row0 = (item - ly.item0) * ly.rows_per_item;
        d.nrows = min(ly.rows_per_item, ly.N - d.row0);
        d.N = ly.N;
        d.layer = l;
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
        for (uint32_t s = 0; s < ASYNC_SLOTS; s++) {
            mbar_init(&done[s], REG_WARPS);
            mbar_init(&vacant[s], NSERV);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    bool failed = false;
    if (warp >= REG_WARPS) {
        // 20 warps were launched with 96 registers each: 16 x 112 + 4 x 32 is the same total.  The two roles
        // stay in separate branches to the end, so each is compiled for its own register budget.
        if constexpr (NT == 2) {
            asm volatile("setmaxnreg.dec.sync.aligned.u32 " QB_STR(32) ";");
            static_assert(ASYNC_REGS_SERVICE == 32, "keep the instruction's literal and the constant together");
        }
        const uint32_t sw = warp - REG_WARPS;  // service warp 0 also refills the stages
        if (sw >= NSERV) return;
        if (sw == 0)
            for (uint32_t j = 0; j < S && j < n_my; j++) issue(j, j);
        // The codes and scales do not depend on the previous kernel; everything below may.
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // pushed outputs carry the number of this exchange: one more than the count of exchanges this rank has
        // completed (bumped by the launch's last CTA; read after the previous grid is complete)
        uint32_t ll_flag = 0;
        if constexpr (sizeof(YT) == 8) {
            uint64_t done_count;
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(done_count) : "l"(a.peer_flags[a.rank] + 8) : "memory");
            ll_flag = (uint32_t)done_count + 1u;
            if (sw == 0 && lane == 0) *reinterpret_cast<volatile uint32_t*>(smem + 120) = ll_flag;  // for the validation at the end
        }
        // ---- service warps: refill, fold, store ----
        // A unit of the fold is one row of the sub-item and four batch columns (two when only two are kept): sixteen
        // 16-byte reads, one per compute warp, summed in warp order.  Units are dealt to the lanes row first, so a
        // store instruction writes runs of consecutive outputs.
        const uint32_t vec = BW < 4 ? BW : 4, units = SUB_ROWS * ((BW + 3) / 4);
        uint32_t st = 0, q = 0;
        for (uint32_t j = 0; j < n_my && !failed; j++) {
            const RegItem& it = s_desc[j];
#pragma unroll 1
            for (int s = 0; s < SUBS; s++, q++) {
                const uint32_t slot = q % ASYNC_SLOTS;
                if (!mbar_wait_bounded(&done[slot], (q / ASYNC_SLOTS) & 1)) { failed = true; break; }
                if (sw == 0 && s == SUBS - 1 && j + S < n_my) issue(j + S, st);  // every compute warp has left the stage
                for (uint32_t u = sw * 32 + lane; u < units; u += NSERV * 32) {
                    const uint32_t row_l = u % SUB_ROWS, b0 = (u / SUB_ROWS) * 4;
                    const uint32_t r = s * SUB_ROWS + row_l;  // row inside the item
                    if (r >= it.nrows || b0 >= a.M) continue;
                    const float* red = s_red + slot * L.slot_floats + row_l * RS + b0;
                    float v[4];
                    fold_sixteen(red, SUB_ROWS * RS, vec, v);
                    const uint32_t n = it.row0 + r;
                    const float bias = it.bias ? it.bias[n] : 0.0f;
#pragma unroll
                    for (uint32_t i = 0; i < 4; i++) {
                        const uint32_t b = b0 + i;
                        if (i < vec && b < a.M) {
                            YT* yp = static_cast<YT*>(it.y) + (uint64_t)b * it.N + n;
                            const float out = fmaf(v[i], GEMV_UNSCALE, bias);
                            if constexpr (sizeof(YT) == 8) {  // pushed: the same self-validating element into every rank's buffer
                                for (uint32_t p = 0; p < a.n_peers; p++)
                                    store_ll(reinterpret_cast<LLPair*>(reinterpret_cast<uint8_t*>(yp) + a.peer_delta[p]), out, ll_flag);
                            } else if (a.n_peers == 0) {
                                store_y<YT>(yp, out);
                            } else {  // fused exchange: the same element of every rank's buffer (peer memory over NVLink)
                                for (uint32_t p = 0; p < a.n_peers; p++)
                                    store_y<YT>(reinterpret_cast<YT*>(reinterpret_cast<uint8_t*>(yp) + a.peer_delta[p]), out);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&vacant[slot]);
            }
            if (++st == S) st = 0;
        }
        // Fused exchange with the arrival barrier inside the launch: the CTA that finishes last tells every
        // peer "this rank's outputs of this step are written" and waits, bounded, for theirs, so the launch ends
        // when all ranks' outputs are here.  flags[p] is rank p's array {arrival of rank 0..7, step counter,
        // count of finished CTAs}.
        // Ordering, with as few system-scope fences as it takes (one costs microseconds: it waits for the peers to
        // acknowledge every store in flight): each service warp fences its own peer stores once (sys scope) and
        // joins the CTA's other service warp; the CTA's count is a release / acquire at GPU scope, so the last CTA
        // has every CTA's fenced stores before it; its flag stores are releases at system scope and its polls
        // acquires, which is all the consumer of the gathered buffer needs — no fence follows.
        if constexpr (sizeof(YT) == 8) {
            // pushed outputs need no ordering; the launch's last CTA only records that this exchange is done
            if (NSERV > 1) asm volatile("bar.sync 1, %0;" ::"r"(NSERV * 32) : "memory");
            if (sw == 0 && lane == 0) {
                uint64_t* mine = a.peer_flags[a.rank];
                if (atomicAdd(reinterpret_cast<unsigned int*>(mine + 9), 1u) == gridDim.x - 1) {
                    *reinterpret_cast<unsigned int*>(mine + 9) = 0;
                    mine[8] = ll_flag;
                }
            }
        } else if (a.n_peers && a.peer_flags[0]) {
#ifdef QB200_TIMING
            uint64_t tf0, tf1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tf0));
#endif
            asm volatile("fence.acq_rel.sys;" ::: "memory");  // this warp's peer stores before the count
#ifdef QB200_TIMING
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tf1));
            if (blockIdx.x == 0 && sw == 0 && lane == 0) atomicAdd(reinterpret_cast<unsigned long long*>(a.peer_flags[a.rank] + 14), tf1 - tf0);
#endif
            // the other service warps' stores too: they join on a named barrier after their fences
            if (NSERV > 1) asm volatile("bar.sync 1, %0;" ::"r"(NSERV * 32) : "memory");
            uint32_t last = 0;
            uint64_t* mine = a.peer_flags[a.rank];
            if (sw == 0 && lane == 0) {
                uint32_t old;
                asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(mine + 9) : "memory");
                last = old == gridDim.x - 1 ? 1u : 0u;
            }
            last = __shfl_sync(0xFFFFFFFFu, last, 0);  // service warp 0 of the last CTA only
            if (last) {
#ifdef QB200_TIMING
                uint64_t tm0, tm1, tm2;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm0));
#endif
                uint64_t step = 0;
                if (lane == 0) {
                    *reinterpret_cast<unsigned int*>(mine + 9) = 0;
                    step = mine[8] + 1;
                    mine[8] = step;
                }
                step = __shfl_sync(0xFFFFFFFFu, step, 0);  // (the shuffle also carries lane 0's acquire to the lanes that publish)
                if (lane < a.n_peers) {
                    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.peer_flags[lane] + a.rank), "l"(step) : "memory");
#ifdef QB200_TIMING
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm1));
#endif
                    uint64_t v = 0;
                    uint32_t spins = 0;
                    for (;;) {
                        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine + lane) : "memory");
                        if (v >= step || ++spins >= a.peer_spin_limit) break;
                        __nanosleep(100);
                    }
#ifdef QB200_TIMING
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm2));
                    if (lane != a.rank) {  // the wait for a peer: ns from the count to the publish, from the publish to the arrival, polls
                        atomicAdd(reinterpret_cast<unsigned long long*>(mine + 10), tm1 - tm0);
                        atomicAdd(reinterpret_cast<unsigned long long*>(mine + 11), tm2 - tm1);
                        atomicAdd(reinterpret_cast<unsigned long long*>(mine + 12), 1ull);
                        atomicAdd(reinterpret_cast<unsigned long long*>(mine + 13), (unsigned long long)spins);
                    }
#endif
                    if (v < step) atomicExch(a.status, QB200_ERR_TIMEOUT);
                }
            }
        }
    } else {
        // ---- compute warps ----
        if constexpr (NT == 2) {
            asm volatile("setmaxnreg.inc.sync.aligned.u32 " QB_STR(112) ";");
            static_assert(ASYNC_REGS_COMPUTE == 112, "keep the instruction's literal and the constant together");
        }
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // a compute warp's two scale groups (the second may not exist for short K: it then re-reads the first
        // group's codes against zero activations and a zero scale)
        const bool v0 = warp < groups, v1 = warp + REG_WARPS < groups;
        const uint32_t G0c = v0 ? warp : 0;
        // The item loop works on 32-bit shared-memory addresses that are advanced, not recomputed:
        // every instruction here is paid 16 x 28 times per CTA and layer.
        uint4 fa[NT][4], fb[NT][4];  // activation fragments of the two groups
        float ka[NT][2], kb[NT][2];  // their "+ 8" corrections for batch columns 2t, 2t + 1, in MMA units
        const uint16_t* cur_x = nullptr;
        const uint32_t sm0 = smem_u32(smem);  // stage barriers at +0, done at +64, vacant at +80
        uint32_t dptr = smem_u32(s_desc);     // the item's activation pointer is the first field of its descriptor
        // this lane's code loads of a row block: rows g and g + 8 of groups G0 and G1, 16 bytes each; its four scales
        const uint32_t codes0 = smem_u32(smem + L.codes) + g * row_bytes + t * 16 + G0c * 64;
        const uint32_t scales0 = smem_u32(smem + L.scales) + (g * groups + G0c) * 4;
        const uint32_t c8 = 8 * row_bytes, s8 = 8 * groups * 4;
        const uint32_t cg1 = v1 ? REG_WARPS * 64 : 0, sg1 = v1 ? REG_WARPS * 4 : 0;
        // where this lane parks its partial sums inside a slot: row g (and g + 8) of a row block, columns 2t, 2t + 1
        const uint32_t red0 = smem_u32(s_red) + ((warp * SUB_ROWS + g) * RS + 2 * t) * 4;
        const bool keeps = 2 * t < BW;  // columns past the kept ones are not parked
        const bool keeps1 = 8 + 2 * t < BW;
        uint32_t st = 0, parity = 0, stage_codes = codes0, stage_scales = scales0, q = 0;
        for (uint32_t j = 0; j < n_my; j++, dptr += (uint32_t)sizeof(RegItem)) {
            if (!async_try_wait(sm0 + st * 8, parity) && !async_wait_bounded(sm0 + st * 8, parity)) { failed = true; break; }
            const uint16_t* x_now;
            asm volatile("ld.shared.u64 %0, [%1];" : "=l"(x_now) : "r"(dptr));
            if (x_now != cur_x) {  // uniform across the CTA: (re)load this warp's fragments
                cur_x = x_now;
                uint32_t li;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(li) : "r"(dptr + (uint32_t)offsetof(RegItem, layer)));
                const uint32_t ldx = a.layer[li].ldx, kvalid = a.layer[li].kvalid;  // columns past kvalid read as zero
                const uint32_t G1c = v1 ? warp + REG_WARPS : 0;
                bool ood = false;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint32_t b = g + 8 * nt;
                    float s0 = load_fragment(cur_x, ldx, b, G0c, t, v0 && b < a.M && G0c * 128 + t * 32 < kvalid, fa[nt], ood);
                    float s1 = load_fragment(cur_x, ldx, b, G1c, t, v1 && b < a.M && G1c * 128 + t * 32 < kvalid, fb[nt], ood);
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
                if (ood) atomicExch(a.status, QB200_ERR_INVALID_PARAM);  // reported by qb200_qlinear_check
            }
#pragma unroll
            for (int s = 0; s < SUBS; s++, q++) {
                const uint32_t slot = q % ASYNC_SLOTS, vpar = ((q / ASYNC_SLOTS) & 1) ^ 1;
                const uint32_t vac = sm0 + 64 + (ASYNC_SLOTS + slot) * 8;
                // The slot's previous sub-item has long been folded.  With 32-row sub-items the poll sits here, where its
                // latency overlaps the loads (measured: polling before the stores instead costs a single-row batch a
                // quarter of its bandwidth); with 16-row sub-items a warp may run one sub-item further ahead of the
                // fold if it polls only before it parks its sums (+ 7 % for a batch of 16).
                if (NT == 1 && q >= ASYNC_SLOTS && !async_try_wait(vac, vpar) && !async_wait_bounded(vac, vpar)) { failed = true; break; }
                // every load of the sub-item first
                uint4 c[RPS][4];
                float sc[RPS][4];
#pragma unroll
                for (int rb = 0; rb < RPS; rb++) {
                    const uint32_t cr = stage_codes + (s * RPS + rb) * 2 * c8, sr = stage_scales + (s * RPS + rb) * 2 * s8;
                    c[rb][0] = async_lds128(cr);
                    c[rb][1] = async_lds128(cr + c8);
                    c[rb][2] = async_lds128(cr + cg1);
                    c[rb][3] = async_lds128(cr + cg1 + c8);
                    sc[rb][0] = async_lds32(sr);
                    sc[rb][1] = async_lds32(sr + s8);
                    sc[rb][2] = v1 ? async_lds32(sr + sg1) : 0.0f;
                    sc[rb][3] = v1 ? async_lds32(sr + sg1 + s8) : 0.0f;
                }
                // 2 * RPS * NT independent MMA chains (row block x group x batch tile), interleaved step by step
                float pa[RPS][NT][4], pb[RPS][NT][4];
#define QB_STEP(J, X, FIRST)                                                                         \
    _Pragma("unroll") for (int rb = 0; rb < RPS; rb++) {                                             \
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
                const uint32_t ra = red0 + slot * (L.slot_floats * 4);
                if (NT == 2 && q >= ASYNC_SLOTS && !async_try_wait(vac, vpar) && !async_wait_bounded(vac, vpar)) { failed = true; break; }
#pragma unroll
                for (int rb = 0; rb < RPS; rb++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        float o[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const float da = pa[rb][nt][i] - ka[nt][i & 1], db = pb[rb][nt][i] - kb[nt][i & 1];
                            o[i] = fmaf(sc[rb][i < 2 ? 2 : 3], db, sc[rb][i < 2 ? 0 : 1] * da);
                        }
                        if (nt == 0 ? keeps : keeps1) {
                            async_sts64(ra + (rb * 16 * RS + nt * 8) * 4, o[0], o[1]);
                            async_sts64(ra + ((rb * 16 + 8) * RS + nt * 8) * 4, o[2], o[3]);
                        }
                    }
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sm0 + 64 + slot * 8) : "memory");  // publishes the sums; the last sub-item's arrival also releases the stage
            }
            if (failed) break;
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
    if constexpr (sizeof(YT) == 8) {
        // Pushed all-gather with the arrival checked in the launch: every rank runs the same items, so the rows this CTA
        // has just pushed are the rows its twin on every peer pushes into this rank's arena at about the same time.
        // All warps poll those elements (in the peers' slots of the own arena, `ll_slot_stride` bytes apart) until they
        // carry this exchange's number: when the launch ends, every rank's outputs are here — without a fence, a flag
        // or a second launch; the wait is one NVLink crossing after the twin's store.
        if (a.ll_slot_stride && __syncthreads_or_live(failed, REG_THREADS + 32 * NSERV) == 0) {
            const uint32_t flag = *reinterpret_cast<volatile uint32_t*>(smem + 120), nthreads = REG_THREADS + 32 * NSERV;
            const uint32_t others = a.n_peers - 1;
            // one flat index space over (item, peer, batch row, row) so that every thread polls at most a few elements
            constexpr uint32_t ROWS = RB * 16;
            const uint32_t per_item = ROWS * a.M * others, total = n_my * per_item;
            for (uint32_t e = tid; e < total && !failed; e += nthreads) {
                const uint32_t j = e / per_item, rem = e - j * per_item, pi = rem / (ROWS * a.M), rem2 = rem - pi * (ROWS * a.M);
                const uint32_t b = rem2 / ROWS, r = rem2 - b * ROWS;
                const RegItem& it = s_desc[j];
                if (r >= it.nrows) continue;
                const int64_t shift = ((int64_t)(pi + (pi >= a.rank ? 1u : 0u)) - (int64_t)a.rank) * (int64_t)a.ll_slot_stride;
                const uint8_t* p = reinterpret_cast<const uint8_t*>(static_cast<LLPair*>(it.y) + (uint64_t)b * it.N + it.row0 + r) + shift;
                uint32_t v0, v1, spins = 0;
                for (;;) {
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v0), "=r"(v1) : "l"(p) : "memory");
                    if (v1 == flag) break;
                    if (++spins >= a.peer_spin_limit || ((spins & 15u) == 0 && *reinterpret_cast<volatile int32_t*>(a.status) != 0)) {
                        atomicExch(a.status, QB200_ERR_TIMEOUT);
                        failed = true;
                        break;
                    }
                    __nanosleep(64);
                }
            }
            failed = false;  // recorded above; the copies of this launch have all landed
        }
    }
    if (failed) {
        // A wait ran out: record it, give copies still in flight a bounded chance to land, leave.
        if (lane == 0) atomicExch(a.status, QB200_ERR_TIMEOUT);
        for (uint32_t s = 0; s < S; s++) mbar_wait_bounded(&bars[s], 0);
    }
}

}  // namespace qb
