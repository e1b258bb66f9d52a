// The support ops of a decode step around the quantized linears (needed only to time the
// whole-model configuration; the hot path is the linears).  f32 arithmetic, bf16 storage for
// what feeds the next linear and for the KV cache.
//
// Reference semantics:
//   RMSNorm   rrms = 1 / sqrt(sum(x^2) / c + eps), out = x * rrms * gamma
//             (crates/ml/quanta-nn/src/norm.rs:192-225)
//   RoPE      rotate-half: out[j] = x[j] cos[j] -/+ x[j +/- d/2] sin[j], the table built in f64 on
//             the host (crates/sci/quanta-array/src/autograd/rope.rs:43-63, quanta-nn/src/rope.rs:23-58)
//   SDPA      online softmax over the keys, score = scale * (q . k), keys >= kv_len masked
//             (crates/ml/quanta-nn/src/kernel.rs:64-175)
//   SwiGLU    out = a * s * b, s = 1 / (1 + exp(min(-a, 30)))
//             (crates/ml/quanta-nn/src/activation.rs:145-162)
#include <cstdint>
#include <string>

#include "forward.hpp"
#include "quant_math.cuh"

namespace qb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// h += delta[0] + ... + delta[parts - 1] (arrays of n * c floats laid back to back; the partial outputs of a
// sliced linear), out = bf16(rmsnorm(h) * gamma).  One block of 1024 threads per row, four consecutive
// elements per thread and pass (the rows are short: latency, not bandwidth, is what this kernel has to hide).
__global__ void __launch_bounds__(1024) k_add_rmsnorm(float* __restrict__ h, const float* __restrict__ delta, uint32_t parts,
                                                      uint64_t part_stride, const float* __restrict__ gamma, uint32_t c, float eps,
                                                      uint16_t* __restrict__ out) {
    // launched with programmatic stream serialization: wait for the producer of the inputs, then let the
    // consumer start its own prologue (a decode GEMV prefetches its weights there) under this kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float s_part[32];
    const uint64_t base = (uint64_t)blockIdx.x * c;
    const bool vec = (c & 3u) == 0;  // rows start on 16-byte boundaries
    float sq = 0.0f;
    if (vec) {
        for (uint32_t i = threadIdx.x * 4; i < c; i += 4096) {
            float4 v = *reinterpret_cast<const float4*>(h + base + i);
            if (parts) {
                float4 d = *reinterpret_cast<const float4*>(delta + base + i);
                for (uint32_t p = 1; p < parts; p++) {
                    const float4 e = *reinterpret_cast<const float4*>(delta + p * part_stride + base + i);
                    d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
                }
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                *reinterpret_cast<float4*>(h + base + i) = v;
            }
            sq = fmaf(v.x, v.x, sq);
            sq = fmaf(v.y, v.y, sq);
            sq = fmaf(v.z, v.z, sq);
            sq = fmaf(v.w, v.w, sq);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < c; i += 1024) {
            float v = h[base + i];
            if (parts) {
                float d = delta[base + i];
                for (uint32_t p = 1; p < parts; p++) d += delta[p * part_stride + base + i];
                v += d;
                h[base + i] = v;
            }
            sq = fmaf(v, v, sq);
        }
    }
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sq;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 32; w++) tot += s_part[w];
    const float rrms = 1.0f / sqrtf(tot / (float)c + eps);
    // every thread re-reads what it wrote itself (same indices), so no further barrier is needed
    if (vec) {
        for (uint32_t i = threadIdx.x * 4; i < c; i += 4096) {
            const float4 v = *reinterpret_cast<const float4*>(h + base + i);
            const float4 g = *reinterpret_cast<const float4*>(gamma + i);
            uint2 o;
            o.x = f32_to_bf16_bits(v.x * rrms * g.x) | ((uint32_t)f32_to_bf16_bits(v.y * rrms * g.y) << 16);
            o.y = f32_to_bf16_bits(v.z * rrms * g.z) | ((uint32_t)f32_to_bf16_bits(v.w * rrms * g.w) << 16);
            *reinterpret_cast<uint2*>(out + base + i) = o;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < c; i += 1024) out[base + i] = f32_to_bf16_bits(h[base + i] * rrms * gamma[i]);
    }
}

// ---- consumers of pushed outputs (self-validating 8-byte elements: f32 bits + the number of the exchange) ----
// A rank's producer kernel has stored its part into every rank's buffer with plain 8-byte stores over NVLink; there
// is no barrier.  The consumer polls each element until its flag is the exchange it expects (state[8], the count of
// exchanges this rank itself has completed: every rank goes through the same sequence of exchanges).  Waits are
// bounded: a thread that runs out of polls records QB200_ERR_TIMEOUT in `status`, and every other thread gives up
// as soon as it sees that word set, so a rank that never delivers costs one wait, not one per element.

// Two consecutive elements (16 bytes, each half validated on its own); false when the polls ran out.
__device__ __forceinline__ bool pushed_load2(const uint4* p, uint32_t flag, uint32_t limit, int32_t* status, float& a, float& b) {
    uint4 v;
    for (uint32_t spins = 0;; spins++) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
        if (v.y == flag && v.w == flag) break;
        if (spins >= limit || ((spins & 15u) == 15u && *reinterpret_cast<volatile int32_t*>(status) != 0)) {
            atomicExch(status, QB200_ERR_TIMEOUT);
            a = b = 0.0f;
            return false;
        }
        __nanosleep(64);
    }
    a = __uint_as_float(v.x);
    b = __uint_as_float(v.z);
    return true;
}
__device__ __forceinline__ bool pushed_load1(const uint2* p, uint32_t flag, uint32_t limit, int32_t* status, float& a) {
    uint2 v;
    for (uint32_t spins = 0;; spins++) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
        if (v.y == flag) break;
        if (spins >= limit || ((spins & 15u) == 15u && *reinterpret_cast<volatile int32_t*>(status) != 0)) {
            atomicExch(status, QB200_ERR_TIMEOUT);
            a = 0.0f;
            return false;
        }
        __nanosleep(64);
    }
    a = __uint_as_float(v.x);
    return true;
}

// k_add_rmsnorm over pushed parts: h += part[0] + ... + part[parts - 1] in part order (the same order on every rank,
// so the residual stream stays bit-identical across ranks), out = bf16(rmsnorm(h) * gamma).
__global__ void __launch_bounds__(1024) k_add_rmsnorm_pushed(float* __restrict__ h, const uint2* __restrict__ pushed, uint32_t parts,
                                                             uint64_t part_stride, const uint64_t* __restrict__ state,
                                                             const float* __restrict__ gamma, uint32_t c, float eps,
                                                             uint16_t* __restrict__ out, uint32_t limit, int32_t* status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the local producer has bumped state[8]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float s_part[32];
    const uint32_t flag = (uint32_t)state[8];
    const uint64_t base = (uint64_t)blockIdx.x * c;
    const bool vec = (c & 3u) == 0;
    float sq = 0.0f;
    if (vec) {
        for (uint32_t i = threadIdx.x * 4; i < c; i += 4096) {
            float4 v = *reinterpret_cast<const float4*>(h + base + i);
            float4 d = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (uint32_t p = 0; p < parts; p++) {
                const uint4* q = reinterpret_cast<const uint4*>(pushed + p * part_stride + base + i);
                float e0, e1, e2, e3;
                pushed_load2(q, flag, limit, status, e0, e1);
                pushed_load2(q + 1, flag, limit, status, e2, e3);
                if (p == 0) d = make_float4(e0, e1, e2, e3);
                else { d.x += e0; d.y += e1; d.z += e2; d.w += e3; }
            }
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            *reinterpret_cast<float4*>(h + base + i) = v;
            sq = fmaf(v.x, v.x, sq);
            sq = fmaf(v.y, v.y, sq);
            sq = fmaf(v.z, v.z, sq);
            sq = fmaf(v.w, v.w, sq);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < c; i += 1024) {
            float v = h[base + i], d = 0.0f;
            for (uint32_t p = 0; p < parts; p++) {
                float e;
                pushed_load1(pushed + p * part_stride + base + i, flag, limit, status, e);
                d = p == 0 ? e : d + e;
            }
            v += d;
            h[base + i] = v;
            sq = fmaf(v, v, sq);
        }
    }
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sq;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 32; w++) tot += s_part[w];
    const float rrms = 1.0f / sqrtf(tot / (float)c + eps);
    if (vec) {
        for (uint32_t i = threadIdx.x * 4; i < c; i += 4096) {
            const float4 v = *reinterpret_cast<const float4*>(h + base + i);
            const float4 g = *reinterpret_cast<const float4*>(gamma + i);
            uint2 o;
            o.x = f32_to_bf16_bits(v.x * rrms * g.x) | ((uint32_t)f32_to_bf16_bits(v.y * rrms * g.y) << 16);
            o.y = f32_to_bf16_bits(v.z * rrms * g.z) | ((uint32_t)f32_to_bf16_bits(v.w * rrms * g.w) << 16);
            *reinterpret_cast<uint2*>(out + base + i) = o;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < c; i += 1024) out[base + i] = f32_to_bf16_bits(h[base + i] * rrms * gamma[i]);
    }
}

// Gathers column-sharded pushed outputs into a dense matrix: part r holds `rows` x w_r elements packed row by row,
// w_r = base + (r < extra ? 1 : 0) columns starting at column r * base + min(r, extra) of dst (rows `dst_stride` apart).
__global__ void __launch_bounds__(256) k_gather_pushed(const uint2* __restrict__ pushed, uint32_t parts, uint64_t part_stride,
                                                       uint32_t rows, uint32_t base, uint32_t extra, const uint64_t* __restrict__ state,
                                                       float* __restrict__ dst, uint64_t dst_stride, uint32_t limit, int32_t* status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t flag = (uint32_t)state[8];
    const uint32_t p = blockIdx.y, w = base + (p < extra ? 1u : 0u), lo = p * base + (p < extra ? p : extra);
    const uint64_t total = (uint64_t)rows * w;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        float v;
        pushed_load1(pushed + p * part_stride + i, flag, limit, status, v);
        dst[(i / w) * dst_stride + lo + (i % w)] = v;
    }
}

// q, k: rotate by the position's angles; q -> bf16 [b, heads, hd]; k, v -> the cache row `pos`.
__global__ void __launch_bounds__(128) k_rope_append(const float* __restrict__ q, const float* __restrict__ k,
                                                     const float* __restrict__ v, const float* __restrict__ cosv,
                                                     const float* __restrict__ sinv, uint32_t heads, uint32_t hd,
                                                     uint16_t* __restrict__ q_out, uint16_t* __restrict__ kcache,
                                                     uint16_t* __restrict__ vcache, uint32_t ctx_max, uint32_t pos) {
    // launched with programmatic stream serialization: wait for the producer of the inputs, then let the
    // consumer start its own prologue (a decode GEMV prefetches its weights there) under this kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t b = blockIdx.x / heads, hh = blockIdx.x % heads, half = hd >> 1;
    const uint64_t in = ((uint64_t)b * heads + hh) * hd;
    const uint64_t cache = (((uint64_t)b * ctx_max + pos) * heads + hh) * hd;
    for (uint32_t j = threadIdx.x; j < hd; j += blockDim.x) {
        const uint32_t partner = j < half ? j + half : j - half;
        const float pm = j < half ? -1.0f : 1.0f, c = cosv[j], s = sinv[j];
        const float qr = q[in + j] * c + pm * q[in + partner] * s;
        const float kr = k[in + j] * c + pm * k[in + partner] * s;
        q_out[in + j] = f32_to_bf16_bits(qr);
        kcache[cache + j] = f32_to_bf16_bits(kr);
        vcache[cache + j] = f32_to_bf16_bits(v[in + j]);
    }
}

// Decode attention, first pass: one block per (batch row, head, split of SDPA_SPLIT keys); a warp
// takes one key at a time (a key's hd bf16 are one coalesced read: lane l holds elements 4l..4l+3
// for hd = 128), keeps the online-softmax state (m, l) and its slice of the weighted V sum; the
// block's warps are merged and the split's (m, l, acc) go to scratch.
constexpr uint32_t SDPA_SPLIT = 128, SDPA_WARPS = 4;

__global__ void __launch_bounds__(SDPA_WARPS * 32) k_sdpa_decode_split(const uint16_t* __restrict__ q,
                                                                        const uint16_t* __restrict__ kcache,
                                                                        const uint16_t* __restrict__ vcache, uint32_t heads,
                                                                        uint32_t ctx_max, uint32_t kv_len, float scale,
                                                                        uint32_t splits, float* __restrict__ scratch) {
    // launched with programmatic stream serialization: wait for the producer of the inputs, then let the
    // consumer start its own prologue (a decode GEMV prefetches its weights there) under this kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr uint32_t HD = 128;
    __shared__ float s_m[SDPA_WARPS], s_l[SDPA_WARPS], s_acc[SDPA_WARPS][HD];
    const uint32_t split = blockIdx.x % splits, bh = blockIdx.x / splits, b = bh / heads, hh = bh % heads;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint2 qv = *reinterpret_cast<const uint2*>(q + ((uint64_t)b * heads + hh) * HD + lane * 4);
    const float q0 = bf16_bits_to_f32(qv.x & 0xFFFFu), q1 = bf16_bits_to_f32(qv.x >> 16);
    const float q2 = bf16_bits_to_f32(qv.y & 0xFFFFu), q3 = bf16_bits_to_f32(qv.y >> 16);
    float m = -3.0e38f, l = 0.0f, a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    const uint32_t k_end = min(kv_len, (split + 1) * SDPA_SPLIT);
    const uint64_t key_stride = (uint64_t)heads * HD;
    const uint64_t row0 = ((uint64_t)b * ctx_max * heads + hh) * HD + lane * 4;
    // four keys per iteration (keys kj, kj + W, kj + 2W, kj + 3W): eight independent 8-byte loads in flight per lane
    constexpr uint32_t U = 4;
    for (uint32_t kj = split * SDPA_SPLIT + warp; kj < k_end; kj += SDPA_WARPS * U) {
        uint2 kv[U], vv[U];
        bool ok[U];
#pragma unroll
        for (uint32_t u = 0; u < U; u++) {
            const uint32_t key = kj + u * SDPA_WARPS;
            ok[u] = key < k_end;
            const uint64_t row = row0 + (uint64_t)(ok[u] ? key : kj) * key_stride;
            kv[u] = *reinterpret_cast<const uint2*>(kcache + row);
            vv[u] = *reinterpret_cast<const uint2*>(vcache + row);
        }
        float sk[U];
#pragma unroll
        for (uint32_t u = 0; u < U; u++) {
            float dot = q0 * bf16_bits_to_f32(kv[u].x & 0xFFFFu);
            dot = fmaf(q1, bf16_bits_to_f32(kv[u].x >> 16), dot);
            dot = fmaf(q2, bf16_bits_to_f32(kv[u].y & 0xFFFFu), dot);
            dot = fmaf(q3, bf16_bits_to_f32(kv[u].y >> 16), dot);
            sk[u] = dot;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1)
#pragma unroll
            for (uint32_t u = 0; u < U; u++) sk[u] += __shfl_xor_sync(0xFFFFFFFFu, sk[u], o);
        float m_new = m;
#pragma unroll
        for (uint32_t u = 0; u < U; u++) {
            sk[u] = ok[u] ? scale * sk[u] : -3.0e38f;
            m_new = fmaxf(m_new, sk[u]);
        }
        const float ra = expf(m - m_new);
        l *= ra;
        a0 *= ra;
        a1 *= ra;
        a2 *= ra;
        a3 *= ra;
#pragma unroll
        for (uint32_t u = 0; u < U; u++) {
            const float rb = ok[u] ? expf(sk[u] - m_new) : 0.0f;
            l += rb;
            a0 = fmaf(rb, bf16_bits_to_f32(vv[u].x & 0xFFFFu), a0);
            a1 = fmaf(rb, bf16_bits_to_f32(vv[u].x >> 16), a1);
            a2 = fmaf(rb, bf16_bits_to_f32(vv[u].y & 0xFFFFu), a2);
            a3 = fmaf(rb, bf16_bits_to_f32(vv[u].y >> 16), a3);
        }
        m = m_new;
    }
    if (lane == 0) {
        s_m[warp] = m;
        s_l[warp] = l;
    }
    s_acc[warp][lane * 4] = a0;
    s_acc[warp][lane * 4 + 1] = a1;
    s_acc[warp][lane * 4 + 2] = a2;
    s_acc[warp][lane * 4 + 3] = a3;
    __syncthreads();
    if (threadIdx.x < HD) {  // merge the warps: thread = one of the hd outputs
        float M = s_m[0];
#pragma unroll
        for (int w = 1; w < (int)SDPA_WARPS; w++) M = fmaxf(M, s_m[w]);
        float L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < (int)SDPA_WARPS; w++) {
            const float r = expf(s_m[w] - M);
            L = fmaf(s_l[w], r, L);
            A = fmaf(s_acc[w][threadIdx.x], r, A);
        }
        float* o = scratch + ((uint64_t)bh * splits + split) * (HD + 2);
        o[2 + threadIdx.x] = A;
        if (threadIdx.x == 0) {
            o[0] = M;
            o[1] = L;
        }
    }
}

// Second pass: merge the splits of one (batch row, head); out = acc / l as bf16.
__global__ void __launch_bounds__(128) k_sdpa_decode_merge(const float* __restrict__ scratch, uint32_t splits,
                                                           uint16_t* __restrict__ out) {
    // launched with programmatic stream serialization: wait for the producer of the inputs, then let the
    // consumer start its own prologue (a decode GEMV prefetches its weights there) under this kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr uint32_t HD = 128;
    const uint32_t bh = blockIdx.x;
    const float* s = scratch + (uint64_t)bh * splits * (HD + 2);
    float M = -3.0e38f;
    for (uint32_t i = 0; i < splits; i++) M = fmaxf(M, s[i * (HD + 2)]);
    float L = 0.0f, A = 0.0f;
    for (uint32_t i = 0; i < splits; i++) {
        const float r = expf(s[i * (HD + 2)] - M);
        L = fmaf(s[i * (HD + 2) + 1], r, L);
        A = fmaf(s[i * (HD + 2) + 2 + threadIdx.x], r, A);
    }
    out[(uint64_t)bh * HD + threadIdx.x] = f32_to_bf16_bits(A / L);
}

// out = silu(gate) * up as bf16, written in column slices: slice s holds columns
// [start_s, start_s + width_s) of every row back to back ([n, width_s] each), so that a linear
// whose input width exceeds the decode kernel's limit can run as one grouped launch over
// contiguous inputs.
struct SliceSpec {
    uint32_t count;
    uint32_t start[8], width[8], stride[8];  // stride: row pitch of the slice's block (>= width; the rest is not written)
    uint64_t offset[8];  // element offset of the slice's [n, width] block in `out`
};
__global__ void __launch_bounds__(256) k_swiglu_sliced(const float* __restrict__ gate, const float* __restrict__ up,
                                                       uint32_t n, uint32_t h, SliceSpec sp, uint16_t* __restrict__ out) {
    // launched with programmatic stream serialization: wait for the producer of the inputs, then let the
    // consumer start its own prologue (a decode GEMV prefetches its weights there) under this kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (uint64_t)n * h) return;
    const uint32_t row = (uint32_t)(i / h), col = (uint32_t)(i % h);
    const float a = gate[i], b = up[i];
    const float s = 1.0f / (1.0f + expf(fminf(-a, 30.0f)));
    uint32_t sl = 0;
    while (sl + 1 < sp.count && col >= sp.start[sl + 1]) sl++;
    out[sp.offset[sl] + (uint64_t)row * sp.stride[sl] + (col - sp.start[sl])] = f32_to_bf16_bits(a * s * b);
}

// y[i] = sum of `count` arrays (the partial outputs of a sliced linear).
__global__ void __launch_bounds__(256) k_sum_arrays(const float* __restrict__ parts, uint32_t count, uint64_t n,
                                                    float* __restrict__ y) {
    // launched with programmatic stream serialization: wait for the producer of the inputs, then let the
    // consumer start its own prologue (a decode GEMV prefetches its weights there) under this kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float v = parts[i];
    for (uint32_t p = 1; p < count; p++) v += parts[(uint64_t)p * n + i];
    y[i] = v;
}

}  // namespace qb

namespace qb {

// Every kernel of this file is launched with programmatic stream serialization (see the kernels' first lines).
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), uint32_t grid, uint32_t block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace qb

using qb::fail;

extern "C" {

qb200_status qb200_add_rmsnorm(float* h, const float* delta, uint32_t delta_parts, const float* gamma, uint64_t n, uint64_t c,
                               float eps, uint16_t* out_bf16, void* stream) {
    if (!h || !gamma || !out_bf16 || (delta_parts && !delta)) return fail(QB200_ERR_INVALID_PARAM, "qb200_add_rmsnorm: null pointer");
    if (n == 0 || c == 0 || c > 0x7FFFFFFFull || n > 0x7FFFFFFFull) return fail(QB200_ERR_INVALID_PARAM, "qb200_add_rmsnorm: bad shape");
    QB_CUDA_TRY(qb::launch_pdl(qb::k_add_rmsnorm, (uint32_t)n, 1024, static_cast<cudaStream_t>(stream), h, delta, delta ? delta_parts : 0, n * c, gamma, (uint32_t)c, eps,
                                                                                   out_bf16));
    return QB200_OK;
}

qb200_status qb200_add_rmsnorm_pushed(float* h, const void* pushed, uint32_t parts, const uint64_t* state_own, const float* gamma,
                                      uint64_t n, uint64_t c, float eps, uint16_t* out_bf16, int32_t* status_dev, void* stream) {
    if (!h || !gamma || !out_bf16 || !pushed || !state_own || !status_dev || parts == 0)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_add_rmsnorm_pushed: null pointer or no parts");
    if (n == 0 || c == 0 || c > 0x7FFFFFFFull || n > 0x7FFFFFFFull) return fail(QB200_ERR_INVALID_PARAM, "qb200_add_rmsnorm_pushed: bad shape");
    if (reinterpret_cast<uintptr_t>(pushed) & 15u) return fail(QB200_ERR_INVALID_PARAM, "qb200_add_rmsnorm_pushed: the pushed buffer must be 16-byte aligned");
    QB_CUDA_TRY(qb::launch_pdl(qb::k_add_rmsnorm_pushed, (uint32_t)n, 1024, static_cast<cudaStream_t>(stream), h, static_cast<const uint2*>(pushed),
                               parts, n * c, state_own, gamma, (uint32_t)c, eps, out_bf16, qb::peer_spin_limit(), status_dev));
    return QB200_OK;
}

qb200_status qb200_gather_pushed(const void* pushed, uint32_t parts, uint64_t part_stride, uint32_t rows, uint64_t cols,
                                 const uint64_t* state_own, float* dst, uint64_t dst_stride, int32_t* status_dev, void* stream) {
    if (!pushed || !state_own || !dst || !status_dev || parts == 0 || rows == 0 || cols < parts || cols > 0x7FFFFFFFull || dst_stride < cols)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_gather_pushed: null pointer or bad shape");
    const uint32_t base = (uint32_t)(cols / parts), extra = (uint32_t)(cols % parts);
    const uint64_t widest = (uint64_t)rows * (base + (extra ? 1 : 0));
    if (part_stride < widest) return fail(QB200_ERR_INVALID_PARAM, "qb200_gather_pushed: parts overlap (part_stride below rows x widest shard)");
    const uint32_t bx = (uint32_t)((widest + 255) / 256 > 64 ? 64 : (widest + 255) / 256);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(bx, parts);
    cfg.blockDim = dim3(256);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QB_CUDA_TRY(cudaLaunchKernelEx(&cfg, qb::k_gather_pushed, static_cast<const uint2*>(pushed), parts, part_stride, rows, base, extra, state_own,
                                   dst, dst_stride, qb::peer_spin_limit(), status_dev));
    return QB200_OK;
}

qb200_status qb200_rope_append(const float* q, const float* k, const float* v, const float* cos_row, const float* sin_row,
                               uint32_t b, uint32_t heads, uint32_t hd, uint16_t* q_out, uint16_t* kcache, uint16_t* vcache,
                               uint32_t ctx_max, uint32_t pos, void* stream) {
    if (!q || !k || !v || !cos_row || !sin_row || !q_out || !kcache || !vcache)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_rope_append: null pointer");
    if (hd == 0 || (hd & 1) || pos >= ctx_max || b == 0 || heads == 0)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_rope_append: head dim must be even and the position inside the cache");
    QB_CUDA_TRY(qb::launch_pdl(qb::k_rope_append, b * heads, 128, static_cast<cudaStream_t>(stream), q, k, v, cos_row, sin_row, heads, hd, q_out, kcache,
                                                                                vcache, ctx_max, pos));
    return QB200_OK;
}

uint64_t qb200_sdpa_decode_scratch_floats(uint32_t b, uint32_t heads, uint32_t kv_len) {
    const uint64_t splits = (kv_len + qb::SDPA_SPLIT - 1) / qb::SDPA_SPLIT;
    return (uint64_t)b * heads * splits * (128 + 2);
}

qb200_status qb200_sdpa_decode(const uint16_t* q, const uint16_t* kcache, const uint16_t* vcache, uint32_t b, uint32_t heads,
                               uint32_t hd, uint32_t ctx_max, uint32_t kv_len, float scale, float* scratch, uint16_t* out,
                               void* stream) {
    if (!q || !kcache || !vcache || !scratch || !out) return fail(QB200_ERR_INVALID_PARAM, "qb200_sdpa_decode: null pointer");
    if (hd != 128) return fail(QB200_ERR_NOT_SUPPORTED, "qb200_sdpa_decode: head dim 128 only, got " + std::to_string(hd));
    if (kv_len == 0 || kv_len > ctx_max || b == 0 || heads == 0) return fail(QB200_ERR_INVALID_PARAM, "qb200_sdpa_decode: bad lengths");
    const uint32_t splits = (kv_len + qb::SDPA_SPLIT - 1) / qb::SDPA_SPLIT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    QB_CUDA_TRY(qb::launch_pdl(qb::k_sdpa_decode_split, b * heads * splits, qb::SDPA_WARPS * 32, st, q, kcache, vcache, heads, ctx_max, kv_len, scale, splits,
                                                                               scratch));
    QB_CUDA_TRY(qb::launch_pdl(qb::k_sdpa_decode_merge, b * heads, 128, st, scratch, splits, out));
    return QB200_OK;
}

qb200_status qb200_swiglu_sliced(const float* gate, const float* up, uint64_t n, uint64_t h, const uint32_t* slice_widths,
                                 uint32_t slices, uint32_t pad_to, uint16_t* out, void* stream) {
    if (!gate || !up || !out || !slice_widths) return fail(QB200_ERR_INVALID_PARAM, "qb200_swiglu_sliced: null pointer");
    if (slices == 0 || slices > 8 || n == 0 || h == 0 || n * h > 0x7FFFFFFFFFull)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_swiglu_sliced: 1..8 slices");
    qb::SliceSpec sp = {};
    sp.count = slices;
    uint64_t start = 0;
    for (uint32_t s = 0; s < slices; s++) {
        if (pad_to && slice_widths[s] > pad_to) return fail(QB200_ERR_INVALID_PARAM, "qb200_swiglu_sliced: a slice is wider than pad_to");
        sp.start[s] = (uint32_t)start;
        sp.width[s] = slice_widths[s];
        sp.stride[s] = pad_to ? pad_to : slice_widths[s];
        sp.offset[s] = pad_to ? n * pad_to * s : n * start;
        start += slice_widths[s];
    }
    if (start != h) return fail(QB200_ERR_INVALID_PARAM, "qb200_swiglu_sliced: the slice widths must add up to the hidden width");
    QB_CUDA_TRY(qb::launch_pdl(qb::k_swiglu_sliced, (uint32_t)((n * h + 255) / 256), 256, static_cast<cudaStream_t>(stream), gate, up, (uint32_t)n, (uint32_t)h,
                                                                                                        sp, out));
    return QB200_OK;
}

qb200_status qb200_sum_arrays(const float* parts, uint32_t count, uint64_t n, float* y, void* stream) {
    if (!parts || !y || count == 0) return fail(QB200_ERR_INVALID_PARAM, "qb200_sum_arrays: null pointer");
    if (n == 0) return QB200_OK;
    QB_CUDA_TRY(qb::launch_pdl(qb::k_sum_arrays, (uint32_t)((n + 255) / 256), 256, static_cast<cudaStream_t>(stream), parts, count, n, y));
    return QB200_OK;
}

}  // extern "C"
