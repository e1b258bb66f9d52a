// QuantizedLinear forward, generic kernels: every dtype, every scale grid, both
// weight orientations, f32 or bf16 activations.  The f32 weight is never
// materialised: codes are unpacked and scaled in registers and accumulated in
// f32 (the reference dequantizes the whole matrix to f32 and then runs an f32
// GEMM, crates/ml/quanta-nn/src/quant.rs:903-918).
//
//   rows kernel  (OUT_IN, W `[out, in]`): one warp per output feature, lanes
//                stride over 8-code chunks of K, shuffle reduction.
//   cols kernel  (IN_OUT, W `[in, out]`, the reference's Linear orientation):
//                each thread owns 8 adjacent output features and streams down
//                K (coalesced along N); K is split across warps and, for small
//                N, across CTAs — partial sums go to a scratch buffer and a
//                second kernel folds them, adds the bias and casts.
#include <atomic>
#include <cstdint>
#include <string>

#include "forward.hpp"
#include "qlinear_handle.hpp"
#include "quant_math.cuh"

namespace qb {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<uint16_t>(uint16_t v) { return bf16_bits_to_f32(v); }

template <typename T>
__device__ __forceinline__ void store_out(T* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<uint16_t>(uint16_t* p, float v) { *p = f32_to_bf16_bits(v); }

template <int BITS>
__device__ __forceinline__ int code_at(const void* codes, uint64_t row, uint64_t col, uint64_t cols, uint64_t wpr) {
    if constexpr (BITS == 4)
        return int4_unpack(static_cast<const uint32_t*>(codes)[row * wpr + (col >> 3)], (uint32_t)(col & 7));
    else
        return (int)static_cast<const int8_t*>(codes)[row * cols + col];
}

// ---- OUT_IN: warp per output feature ---------------------------------------

template <int BITS, typename XT, typename YT, int MT>
__global__ void __launch_bounds__(256) k_forward_rows(FwdArgs a) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t n = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= a.out_dim) return;  // whole warp exits together
    const uint64_t K = a.in_dim, wpr = (K + 7) >> 3, tc = a.tc;
    const XT* x = static_cast<const XT*>(a.x);
    const uint64_t srow = (n / a.gr) * tc;
    const bool chunk_scale = (a.gc & 7u) == 0;
    // Aligned case (K % 8 == 0, one scale per chunk, 16-byte aligned activations, 8-byte aligned int8 codes, 32-bit
    // sizes): codes and activations come in 8- and 16-byte loads, four chunks of codes in flight per lane, indices
    // in 32 bits.  The arithmetic and its order are those of the general loop below, so the results are the same bits.
    const bool vec = chunk_scale && (K & 7u) == 0 && K < (1ull << 32) && a.gc < (1ull << 32) &&
                     (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.codes) & 7u) == 0;
    if (vec) {
        const uint32_t K32 = (uint32_t)K, gc32 = (uint32_t)a.gc, cpr = K32 >> 3;
        const float* srow_p = a.scales + srow;
        for (uint64_t m0 = (uint64_t)blockIdx.y * MT; m0 < a.m; m0 += (uint64_t)gridDim.y * MT) {
            float acc[MT];
#pragma unroll
            for (int i = 0; i < MT; i++) acc[i] = 0.0f;
            for (uint32_t c0 = lane; c0 < cpr; c0 += 128) {
                uint2 cw[4];
#pragma unroll
                for (uint32_t u = 0; u < 4; u++) {
                    const uint32_t ch = c0 + 32 * u;
                    cw[u] = make_uint2(0u, 0u);
                    if (ch < cpr) {
                        if constexpr (BITS == 4) cw[u].x = __ldg(static_cast<const uint32_t*>(a.codes) + n * cpr + ch);
                        else cw[u] = __ldg(reinterpret_cast<const uint2*>(static_cast<const int8_t*>(a.codes) + n * K + ((uint64_t)ch << 3)));
                    }
                }
#pragma unroll
                for (uint32_t u = 0; u < 4; u++) {
                    const uint32_t ch = c0 + 32 * u;
                    if (ch >= cpr) break;
                    const uint32_t k0 = ch << 3;
                    const float s = __ldg(srow_p + k0 / gc32);
                    float wv[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        int q;
                        if constexpr (BITS == 4) q = int4_unpack(cw[u].x, j);
                        else q = (int)(int8_t)(((j < 4 ? cw[u].x : cw[u].y) >> (8 * (j & 3))) & 0xFFu);
                        wv[j] = s * (float)q;
                    }
#pragma unroll
                    for (int i = 0; i < MT; i++) {
                        if (m0 + i < a.m) {
                            float xf[8];
                            if constexpr (sizeof(XT) == 2) {
                                const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (m0 + i) * K + k0));
                                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    xf[2 * j] = bf16_bits_to_f32(xw[j] & 0xFFFFu);
                                    xf[2 * j + 1] = bf16_bits_to_f32(xw[j] >> 16);
                                }
                            } else {
                                const float4* xp = reinterpret_cast<const float4*>(x + (m0 + i) * K + k0);
                                const float4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                                xf[0] = x0.x; xf[1] = x0.y; xf[2] = x0.z; xf[3] = x0.w;
                                xf[4] = x1.x; xf[5] = x1.y; xf[6] = x1.z; xf[7] = x1.w;
                            }
#pragma unroll
                            for (int j = 0; j < 8; j++) acc[i] = fmaf(xf[j], wv[j], acc[i]);
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < MT; i++) {
                float v = acc[i];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                if (lane == 0 && m0 + i < a.m) {
                    if (a.bias) v += a.bias[n];
                    store_out<YT>(static_cast<YT*>(a.y) + (m0 + i) * a.out_dim + n, v);
                }
            }
        }
        return;
    }
    for (uint64_t m0 = (uint64_t)blockIdx.y * MT; m0 < a.m; m0 += (uint64_t)gridDim.y * MT) {
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; i++) acc[i] = 0.0f;
        for (uint64_t ch = lane; ch < wpr; ch += 32) {
            const uint64_t k0 = ch << 3;
            int q[8];
            if constexpr (BITS == 4) {
                uint32_t word = __ldg(static_cast<const uint32_t*>(a.codes) + n * wpr + ch);
#pragma unroll
                for (int j = 0; j < 8; j++) q[j] = int4_unpack(word, j);
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    q[j] = (k0 + j < K) ? (int)__ldg(static_cast<const int8_t*>(a.codes) + n * K + k0 + j) : 0;
            }
            float wv[8];
            if (chunk_scale) {
                float s = __ldg(a.scales + srow + k0 / a.gc);
#pragma unroll
                for (int j = 0; j < 8; j++) wv[j] = s * (float)q[j];
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint64_t k = k0 + j;
                    wv[j] = k < K ? __ldg(a.scales + srow + k / a.gc) * (float)q[j] : 0.0f;
                }
            }
#pragma unroll
            for (int i = 0; i < MT; i++) {
                if (m0 + i < a.m) {
                    const XT* xr = x + (m0 + i) * K + k0;
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        if (k0 + j < K) acc[i] = fmaf(to_f32<XT>(xr[j]), wv[j], acc[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MT; i++) {
            float v = acc[i];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0 && m0 + i < a.m) {
                if (a.bias) v += a.bias[n];
                store_out<YT>(static_cast<YT*>(a.y) + (m0 + i) * a.out_dim + n, v);
            }
        }
    }
}

// ---- IN_OUT: thread per 8 output features, streaming down K ------------------

constexpr int COLS_WARPS = 8;
constexpr int COLS_MT = 4;

// grid: x = column blocks of 256, y = K slices, z = m tiles of COLS_MT.
// Writes y directly when gridDim.y == 1, else f32 partials `[slice, m, out]`.
template <int BITS, typename XT, typename YT>
__global__ void __launch_bounds__(32 * COLS_WARPS) k_forward_cols(FwdArgs a, float* __restrict__ partial) {
    __shared__ float red[COLS_WARPS][COLS_MT][256 + 8];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint64_t N = a.out_dim, K = a.in_dim, wpr = (N + 7) >> 3, tc = a.tc;
    const uint64_t n0 = ((uint64_t)blockIdx.x * 32 + lane) << 3;
    const uint64_t m0 = (uint64_t)blockIdx.z * COLS_MT;
    const uint64_t kper = (K + gridDim.y - 1) / gridDim.y;
    const uint64_t kbeg = (uint64_t)blockIdx.y * kper, kend = min(K, kbeg + kper);
    const XT* x = static_cast<const XT*>(a.x);
    const bool chunk_scale = (a.gc & 7u) == 0;

    float acc[COLS_MT][8];
#pragma unroll
    for (int i = 0; i < COLS_MT; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

    if (n0 < N) {
        for (uint64_t k = kbeg + warp; k < kend; k += COLS_WARPS) {
            int q[8];
            if constexpr (BITS == 4) {
                uint32_t word = __ldg(static_cast<const uint32_t*>(a.codes) + k * wpr + (n0 >> 3));
#pragma unroll
                for (int j = 0; j < 8; j++) q[j] = int4_unpack(word, j);
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    q[j] = (n0 + j < N) ? (int)__ldg(static_cast<const int8_t*>(a.codes) + k * N + n0 + j) : 0;
            }
            const uint64_t srow = (k / a.gr) * tc;
            float wv[8];
            if (chunk_scale) {
                float s = __ldg(a.scales + srow + n0 / a.gc);
#pragma unroll
                for (int j = 0; j < 8; j++) wv[j] = s * (float)q[j];
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    wv[j] = (n0 + j < N) ? __ldg(a.scales + srow + (n0 + j) / a.gc) * (float)q[j] : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < COLS_MT; i++) {
                if (m0 + i < a.m) {
                    float xv = to_f32<XT>(__ldg(x + (m0 + i) * K + k));
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[i][j] = fmaf(xv, wv[j], acc[i][j]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < COLS_MT; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) red[warp][i][lane * 8 + j] = acc[i][j];
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < COLS_MT * 256; e += blockDim.x) {
        const uint32_t i = e >> 8, c = e & 255u;
        const uint64_t n = (uint64_t)blockIdx.x * 256 + c;
        if (n >= N || m0 + i >= a.m) continue;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < COLS_WARPS; w++) v += red[w][i][c];
        if (gridDim.y == 1) {
            if (a.bias) v += a.bias[n];
            store_out<YT>(static_cast<YT*>(a.y) + (m0 + i) * N + n, v);
        } else {
            partial[((uint64_t)blockIdx.y * a.m + (m0 + i)) * N + n] = v;
        }
    }
}

template <typename YT>
__global__ void k_fold_partials(const float* __restrict__ partial, uint32_t slices, uint64_t m, uint64_t N,
                                const float* __restrict__ bias, YT* __restrict__ y) {
    const uint64_t total = m * N;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        float v = 0.0f;
        for (uint32_t s = 0; s < slices; s++) v += partial[(uint64_t)s * total + i];
        if (bias) v += bias[i % N];
        store_out<YT>(y + i, v);
    }
}

// ---- launchers ----------------------------------------------------------------

template <int BITS, typename XT, typename YT>
static qb200_status launch_rows(const FwdArgs& a, cudaStream_t st) {
    const uint32_t warps = 8;
    dim3 grid((uint32_t)div_ceil(a.out_dim, warps), 1);
    if (a.m <= 1) k_forward_rows<BITS, XT, YT, 1><<<grid, warps * 32, 0, st>>>(a);
    else if (a.m <= 2) k_forward_rows<BITS, XT, YT, 2><<<grid, warps * 32, 0, st>>>(a);
    else if (a.m <= 4) k_forward_rows<BITS, XT, YT, 4><<<grid, warps * 32, 0, st>>>(a);
    else {
        grid.y = (uint32_t)(div_ceil(a.m, 8) > 64 ? 64 : div_ceil(a.m, 8));
        k_forward_rows<BITS, XT, YT, 8><<<grid, warps * 32, 0, st>>>(a);
    }
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

uint32_t forward_cols_slices(uint64_t in_dim, uint64_t out_dim, uint64_t m) {
    const uint64_t ctas = div_ceil(out_dim, 256) * div_ceil(m, COLS_MT);
    uint64_t s = 1;
    while (ctas * s < 296 && in_dim / (s * 2) >= 64 && s < 64) s *= 2;
    return (uint32_t)s;
}

template <int BITS, typename XT, typename YT>
static qb200_status launch_cols(const FwdArgs& a, float* scratch, uint32_t slices, cudaStream_t st) {
    dim3 grid((uint32_t)div_ceil(a.out_dim, 256), slices, (uint32_t)div_ceil(a.m, COLS_MT));
    if (grid.z > 65535) return fail(QB200_ERR_INVALID_PARAM, "forward: m too large for the column kernel");
    k_forward_cols<BITS, XT, YT><<<grid, 32 * COLS_WARPS, 0, st>>>(a, scratch);
    QB_CUDA_TRY(cudaGetLastError());
    if (slices > 1) {
        uint64_t total = a.m * a.out_dim;
        uint32_t blocks = (uint32_t)(div_ceil(total, 256) > 148 * 16 ? 148 * 16 : div_ceil(total, 256));
        k_fold_partials<YT><<<blocks, 256, 0, st>>>(scratch, slices, a.m, a.out_dim, a.bias, static_cast<YT*>(a.y));
        QB_CUDA_TRY(cudaGetLastError());
    }
    return QB200_OK;
}

template <int BITS, typename XT>
static qb200_status by_out(const FwdArgs& a, int y_dtype, bool rows, float* scratch, uint32_t slices, cudaStream_t st) {
    if (y_dtype == QB200_F32)
        return rows ? launch_rows<BITS, XT, float>(a, st) : launch_cols<BITS, XT, float>(a, scratch, slices, st);
    return rows ? launch_rows<BITS, XT, uint16_t>(a, st) : launch_cols<BITS, XT, uint16_t>(a, scratch, slices, st);
}

qb200_status forward_generic(const FwdArgs& a, uint32_t bits, int x_dtype, int y_dtype, bool rows_kernel,
                             float* scratch, uint32_t slices, cudaStream_t st) {
    if (bits == 4) {
        return x_dtype == QB200_F32 ? by_out<4, float>(a, y_dtype, rows_kernel, scratch, slices, st)
                                    : by_out<4, uint16_t>(a, y_dtype, rows_kernel, scratch, slices, st);
    }
    return x_dtype == QB200_F32 ? by_out<8, float>(a, y_dtype, rows_kernel, scratch, slices, st)
                                : by_out<8, uint16_t>(a, y_dtype, rows_kernel, scratch, slices, st);
}

// ---- f32 activations on the bf16 kernels ----------------------------------------------------------------------------
// An f32 has 24 significant bits: its top 8 (a truncation to bf16), the top 8 of what is left, and the rest are three
// bf16 values whose sum is the f32 exactly.  The bf16 kernels multiply each part exactly and accumulate in f32, so the
// three partial outputs added up are the exact-product, f32-accumulated result for the f32 activation.

__global__ void __launch_bounds__(256) k_split_f32(const float* __restrict__ x, uint64_t mk, uint16_t* __restrict__ xs) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < mk; i += (uint64_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        const uint32_t b0 = __float_as_uint(v) & 0xFFFF0000u;
        const float r1 = v - __uint_as_float(b0);  // exact: the low 16 bits of the significand
        const uint32_t b1 = __float_as_uint(r1) & 0xFFFF0000u;
        const float r2 = r1 - __uint_as_float(b1);  // exact: at most 8 significant bits
        xs[i] = (uint16_t)(b0 >> 16);
        xs[mk + i] = (uint16_t)(b1 >> 16);
        xs[2 * mk + i] = f32_to_bf16_bits(r2);
    }
}

template <typename YT>
__global__ void __launch_bounds__(256) k_fold_split(const float* __restrict__ ys, uint64_t mn, uint32_t n, const float* __restrict__ bias,
                                                    YT* __restrict__ y) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < mn; i += (uint64_t)gridDim.x * blockDim.x) {
        float v = (ys[i] + ys[mn + i]) + ys[2 * mn + i];
        if (bias) v += bias[i % n];
        if constexpr (sizeof(YT) == 4) y[i] = v;
        else y[i] = f32_to_bf16_bits(v);
    }
}

qb200_status split_f32_activations(const float* x, uint64_t m, uint64_t k, void* xs, cudaStream_t st) {
    const uint64_t mk = m * k;
    const uint32_t blocks = (uint32_t)((mk + 255) / 256 > 1184 ? 1184 : (mk + 255) / 256);
    k_split_f32<<<blocks, 256, 0, st>>>(x, mk, static_cast<uint16_t*>(xs));
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

qb200_status fold_split_outputs(const float* ys, uint64_t m, uint64_t n, const float* bias, void* y, int y_dtype, cudaStream_t st) {
    const uint64_t mn = m * n;
    const uint32_t blocks = (uint32_t)((mn + 255) / 256 > 1184 ? 1184 : (mn + 255) / 256);
    if (y_dtype == QB200_F32) k_fold_split<float><<<blocks, 256, 0, st>>>(ys, mn, (uint32_t)n, bias, static_cast<float*>(y));
    else k_fold_split<uint16_t><<<blocks, 256, 0, st>>>(ys, mn, (uint32_t)n, bias, static_cast<uint16_t*>(y));
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

}  // namespace qb

// ---- forward without any allocation ------------------------------------------------------------
// Some callers may not allocate device memory at all: latency-critical code where cudaMalloc's
// implicit synchronisation is not acceptable, real-time serving loops with a fixed memory
// budget, and hosts that pre-register every device buffer with another runtime.  For them the split-K partial sums of the column kernel live in a fixed
// array inside the library image instead of a cudaMalloc'd buffer.  Every GPU that loads the
// library holds these 2 MiB until the process exits.

namespace qb {
constexpr uint64_t STATIC_SCRATCH_FLOATS = 1ull << 19;  // 2 MiB: slices * m * out_dim must fit
}
static __device__ __align__(256) float g_static_partials[qb::STATIC_SCRATCH_FLOATS];

extern "C" qb200_status qb200_qlinear_forward_static(qb200_qlinear* ql, const void* x_dev, int32_t x_dtype, uint64_t m,
                                                     void* y_dev, int32_t y_dtype, void* stream) {
    using qb::fail;
    if (!ql) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_static: null handle");
    if (!x_dev || !y_dev) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_static: null device pointer");
    if ((x_dtype != QB200_F32 && x_dtype != QB200_BF16) || (y_dtype != QB200_F32 && y_dtype != QB200_BF16))
        return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_static: activations are f32 or bf16");
    if (ql->layout != QB200_IN_OUT)
        return fail(QB200_ERR_NOT_SUPPORTED,
                    "qb200_qlinear_forward_static serves [in, out] weights (the column kernel); an [out, in] "
                    "handle needs no scratch: call qb200_qlinear_forward");
    if (m == 0) return QB200_OK;
    const uint32_t slices = qb::forward_cols_slices(ql->in_dim, ql->out_dim, m);
    const uint64_t need = slices > 1 ? (uint64_t)slices * m * ql->out_dim : 0;
    if (need > qb::STATIC_SCRATCH_FLOATS)
        return fail(QB200_ERR_INVALID_PARAM,
                    "qb200_qlinear_forward_static: " + std::to_string(slices) + " K slices x m = " + std::to_string(m) +
                        " x out = " + std::to_string(ql->out_dim) + " needs " + std::to_string(need) +
                        " partial sums, the built-in scratch holds " + std::to_string(qb::STATIC_SCRATCH_FLOATS) +
                        " (2 MiB); lower m or call qb200_qlinear_forward");
    // The array's name is a host-side stand-in here, not a device address: look the address up once
    // per device, with that device current.  Every GPU has its own copy of the array, so the address must be
    // the one of the GPU that holds the handle's buffers and runs the kernels: the call is refused when another
    // device is current.  Threads may race to fill an entry; they all store the same address.
    static std::atomic<float*> scratch_of_device[64] = {};
    int dev = 0;
    QB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_static: device index out of range");
    if (ql->device >= 0 && dev != ql->device)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_static: the handle's buffers live on device " +
                                                 std::to_string(ql->device) + " but device " + std::to_string(dev) +
                                                 " is current; make the handle's device current before the call");
    float* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
    if (!scratch) {
        QB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_static_partials));
        scratch_of_device[dev].store(scratch, std::memory_order_release);
    }
    qb::FwdArgs a;
    a.codes = ql->codes;
    a.scales = ql->scales;
    a.bias = ql->bias;
    a.x = x_dev;
    a.y = y_dev;
    a.m = m;
    a.in_dim = ql->in_dim;
    a.out_dim = ql->out_dim;
    a.gr = ql->gr;
    a.gc = ql->gc;
    a.tc = ql->tc;
    // Nothing needs clearing: the column kernel writes every partial sum the fold kernel reads.
    ql->last_kernel = "generic_cols";
    return qb::forward_generic(a, ql->bits, x_dtype, y_dtype, false, scratch, slices, static_cast<cudaStream_t>(stream));
}
