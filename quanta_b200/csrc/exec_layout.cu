// Execution layouts of a QuantizedLinear handle, built once at creation.
//
// The fast int4 kernels read K-contiguous rows: codes `[out, in / 8]` with a 1 x 128 scale grid, at most 4096
// inputs per launch.  These stored layouts do not have that shape as they are:
//   - the reference's own `[in, out]` weight with Group{axis: 0, size: 128} (QuantizedLinear::new takes
//     `w: [in, out]`, crates/ml/quanta-nn/src/quant.rs:853-862): the nibbles run along `out`.  A transposed copy
//     of codes and scales is a pure permutation — every dequantized weight s * q keeps its bits;
//   - inputs wider than 4096 (a feed-forward down projection): the decode kernel keeps the activation
//     fragments of at most 32 scale groups in registers, so the weight is cut into column runs of whole scale
//     groups, every run padded with zero codes and zero scales to one width and stored with contiguous rows
//     (an item of the decode kernel is ONE bulk copy).  A decode call is one grouped launch over the runs —
//     each reads its window of the activations in place — and a fold of their f32 partial outputs.
// Both are copies (+ 0.5 byte per weight each, + the scales): the stored buffers stay what accessors, writers
// and the tcgen05 GEMM's tensor maps over `[out, in]` codes see.
//   - a third int4 copy is scales only: a grid whose scale is constant over whole 128-column runs (tile widths that
//     are multiples of 128, per-row and per-tensor scales, after the transposition where there is one) is spelt out
//     per run as `[out][in / 128]`, after which the layer IS a 1 x 128 layer for every kernel.
//
// The int8 kernels read `[out, in]` bytes with a grid whose tile width is a whole number of 16-column steps: an
// `[in, out]` int8 weight whose tile HEIGHT is such a number (32 x 32 blocks, Group{axis: 0, size: 128}, per-column
// scales) gets a transposed copy of codes and scale grid as well (+ 1 byte per weight), and an int8 weight with more
// than 4096 inputs whose tiles are 32, 64 or 128 columns wide gets column slices like the int4 ones.
#include <cstdint>
#include <string>

#include "forward.hpp"
#include "qlinear_handle.hpp"
#include "quant_math.cuh"

namespace qb {

constexpr uint32_t SLICE_LIMIT = 4096;  // inputs the decode kernel serves per launch (two scale groups per warp)
constexpr uint32_t SLICE_MAX = 8;

// dst[n][kw] packs q(k = 8 kw + i, n), i = 0..7, low nibble first; src word (k, n >> 3) holds q(k, n) in nibble n & 7.
// Threads run along n: the eight reads of a thread are shared by its seven neighbours (one word serves eight n).
__global__ void __launch_bounds__(256) k_transpose_i4(const uint32_t* __restrict__ src, uint32_t in_dim, uint32_t out_dim,
                                                      uint32_t src_words, uint32_t* __restrict__ dst) {
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x, kw = blockIdx.y;
    if (n >= out_dim) return;
    const uint32_t sh = 4 * (n & 7);
    uint32_t w = 0;
#pragma unroll
    for (uint32_t i = 0; i < 8; i++) {
        const uint32_t k = 8 * kw + i;
        if (k < in_dim) w |= ((src[(uint64_t)k * src_words + (n >> 3)] >> sh) & 0xFu) << (4 * i);
    }
    dst[(uint64_t)n * (in_dim / 8) + kw] = w;
}

// dst[n][k] = src[k][n] over bytes, through a 64 x 64 tile in shared memory (both sides coalesced).
__global__ void __launch_bounds__(256) k_transpose_i8(const uint8_t* __restrict__ src, uint32_t in_dim, uint32_t out_dim,
                                                      uint8_t* __restrict__ dst) {
    __shared__ uint8_t tile[64][65];
    const uint32_t n0 = blockIdx.x * 64, k0 = blockIdx.y * 64, tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    for (uint32_t i = ty; i < 64; i += 4)
        if (k0 + i < in_dim && n0 + tx < out_dim) tile[i][tx] = src[(uint64_t)(k0 + i) * out_dim + n0 + tx];
    __syncthreads();
    for (uint32_t i = ty; i < 64; i += 4)
        if (n0 + i < out_dim && k0 + tx < in_dim) dst[(uint64_t)(n0 + i) * in_dim + k0 + tx] = tile[tx][i];
}

// dst[n][g] = src[g][n]
__global__ void __launch_bounds__(256) k_transpose_f32(const float* __restrict__ src, uint32_t rows, uint32_t cols,
                                                       float* __restrict__ dst) {
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c < cols) dst[(uint64_t)c * rows + r] = src[(uint64_t)r * cols + c];
}

// dst[n][g] = src[n / gr][(128 g) / gc]: a grid whose scale is constant over whole 128-column runs, as a 1 x 128 grid.
__global__ void __launch_bounds__(256) k_expand_scales(const float* __restrict__ src, uint32_t src_tc, uint32_t gr, uint64_t gc, uint32_t N,
                                                       uint32_t groups, float* __restrict__ dst) {
    const uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (i >= (uint64_t)N * groups) return;
    const uint32_t n = (uint32_t)(i / groups), g = (uint32_t)(i % groups);
    dst[i] = src[(uint64_t)(n / gr) * src_tc + (uint32_t)((uint64_t)g * 128 / gc)];
}

// y[i] = sum_s parts[s][i] (+ bias[i % N]): the slices' partial outputs, summed in slice order.
template <typename YT>
__global__ void __launch_bounds__(256) k_fold_slices(const float* __restrict__ parts, uint32_t slices, uint64_t mn, uint32_t N,
                                                     const float* __restrict__ bias, YT* __restrict__ y) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < mn; i += (uint64_t)gridDim.x * blockDim.x) {
        float v = 0.0f;
        for (uint32_t s = 0; s < slices; s++) v += parts[s * mn + i];
        if (bias) v += bias[i % N];
        if constexpr (sizeof(YT) == 4) y[i] = v;
        else y[i] = f32_to_bf16_bits(v);
    }
}

void free_exec_layout(qb200_qlinear* ql) {
    if (ql->t_codes) cudaFree(ql->t_codes);
    if (ql->t_scales) cudaFree(ql->t_scales);
    if (ql->x_scales) cudaFree(ql->x_scales);
    ql->x_scales = nullptr;
    if (ql->slice_codes) cudaFree(ql->slice_codes);
    if (ql->slice_scales) cudaFree(ql->slice_scales);
    if (ql->slice_partials) cudaFree(ql->slice_partials);
    ql->t_codes = ql->slice_codes = nullptr;
    ql->t_scales = ql->slice_scales = ql->slice_partials = nullptr;
    ql->n_slices = 0;
}

qb200_status build_exec_layout(qb200_qlinear* ql) {
    if (ql->bits == 8) {
        if (ql->in_dim == 0 || ql->out_dim == 0 || ql->in_dim > 0x7FFFFFFFull || ql->out_dim > 0x7FFFFFFFull) return QB200_OK;
        const uint32_t K = (uint32_t)ql->in_dim, N = (uint32_t)ql->out_dim;
        if (ql->layout == QB200_IN_OUT) {
            if (ql->gr < ql->in_dim && ql->gr % 16 != 0) return QB200_OK;  // the tile height becomes the tile width
            const uint64_t tr = (ql->in_dim + ql->gr - 1) / ql->gr;  // the stored grid is [tr, tc]; the copy's [tc, tr]
            if (tr > 0x7FFFFFFFull || ql->tc > 0x7FFFFFFFull || (K + 63) / 64 > 65535u || tr > 65535u) return QB200_OK;
            QB_CUDA_TRY(cudaMalloc(&ql->t_codes, (uint64_t)N * K));
            QB_CUDA_TRY(cudaMalloc(&ql->t_scales, tr * ql->tc * 4));
            k_transpose_i8<<<dim3((N + 63) / 64, (K + 63) / 64), 256>>>(static_cast<const uint8_t*>(ql->codes), K, N,
                                                                         static_cast<uint8_t*>(ql->t_codes));
            QB_CUDA_TRY(cudaGetLastError());
            k_transpose_f32<<<dim3(((uint32_t)ql->tc + 255) / 256, (uint32_t)tr), 256>>>(ql->scales, (uint32_t)tr, (uint32_t)ql->tc, ql->t_scales);
            QB_CUDA_TRY(cudaGetLastError());
            ql->t_gr = ql->gc;
            ql->t_gc = ql->gr;
            ql->t_tc = tr;
        }
        // inputs wider than the int8 decode kernel keeps in registers: column slices of whole 128-column runs, like the
        // int4 ones (+ 1 byte per weight), for grids whose tile width divides 128
        const uint32_t gc = (uint32_t)(ql->fast_gc() > 0xFFFFFFFFull ? 0 : ql->fast_gc()), gr = (uint32_t)(ql->fast_gr() > 0xFFFFFFFFull ? 0 : ql->fast_gr());
        if (K > SLICE_LIMIT && K % 128 == 0 && K <= SLICE_LIMIT * SLICE_MAX && gr != 0 && (gc == 32 || gc == 64 || gc == 128)) {
            const uint32_t groups = K / 128, n = (K + SLICE_LIMIT - 1) / SLICE_LIMIT, base = groups / n, extra = groups % n;
            const uint32_t tr = (N + gr - 1) / gr, tc = (uint32_t)ql->fast_tc();
            uint32_t widest = 0, c0 = 0;
            for (uint32_t s = 0; s < n; s++) {
                ql->slice_col0[s] = c0;
                ql->slice_width[s] = (base + (s < extra ? 1u : 0u)) * 128;
                c0 += ql->slice_width[s];
                widest = widest > ql->slice_width[s] ? widest : ql->slice_width[s];
            }
            const uint32_t pad = (widest + 511) / 512 * 512;  // rows of scales that are whole 16-byte units
            const uint64_t cbytes = (uint64_t)n * N * pad, sbytes = (uint64_t)n * tr * (pad / gc) * 4;
            QB_CUDA_TRY(cudaMalloc(&ql->slice_codes, cbytes));
            QB_CUDA_TRY(cudaMalloc(&ql->slice_scales, sbytes));
            QB_CUDA_TRY(cudaMalloc(&ql->slice_partials, (uint64_t)n * 16 * N * 4));
            QB_CUDA_TRY(cudaMemset(ql->slice_codes, 0, cbytes));
            QB_CUDA_TRY(cudaMemset(ql->slice_scales, 0, sbytes));
            const uint8_t* codes = static_cast<const uint8_t*>(ql->fast_codes());
            const float* scales = ql->fast_scales();
            for (uint32_t s = 0; s < n; s++) {
                QB_CUDA_TRY(cudaMemcpy2D(static_cast<uint8_t*>(ql->slice_codes) + (uint64_t)s * N * pad, pad, codes + ql->slice_col0[s], K,
                                         ql->slice_width[s], N, cudaMemcpyDeviceToDevice));
                QB_CUDA_TRY(cudaMemcpy2D(ql->slice_scales + (uint64_t)s * tr * (pad / gc), (pad / gc) * 4, scales + ql->slice_col0[s] / gc,
                                         (uint64_t)tc * 4, (ql->slice_width[s] / gc) * 4, tr, cudaMemcpyDeviceToDevice));
            }
            ql->n_slices = n;
            ql->slice_pad = pad;
        }
        QB_CUDA_TRY(cudaDeviceSynchronize());
        return QB200_OK;
    }
    if (ql->bits != 4 || ql->in_dim % 128 != 0 || ql->in_dim == 0 || ql->out_dim == 0 || ql->out_dim > 0x7FFFFFFFull ||
        ql->in_dim > (uint64_t)SLICE_LIMIT * SLICE_MAX)
        return QB200_OK;
    const uint32_t K = (uint32_t)ql->in_dim, N = (uint32_t)ql->out_dim, groups = K / 128;
    if (ql->layout == QB200_IN_OUT) {
        // the transposed copy's tiles are the stored tiles turned: a tile HEIGHT of whole 16-row steps that divides the
        // inputs (or spans them) becomes a tile width the kernels take.  Group{axis: 0, size: 128} is the documented grid.
        if (ql->gr < K && (ql->gr % 16 != 0 || K % ql->gr != 0)) return QB200_OK;
        const uint64_t tr = (K + ql->gr - 1) / ql->gr;
        if (tr > 65535u || ql->tc > 0x7FFFFFFFull) return QB200_OK;
        QB_CUDA_TRY(cudaMalloc(&ql->t_codes, (uint64_t)N * (K / 8) * 4));
        QB_CUDA_TRY(cudaMalloc(&ql->t_scales, tr * ql->tc * 4));
        k_transpose_i4<<<dim3((N + 255) / 256, K / 8), 256>>>(static_cast<const uint32_t*>(ql->codes), K, N, (N + 7) / 8,
                                                               static_cast<uint32_t*>(ql->t_codes));
        QB_CUDA_TRY(cudaGetLastError());
        k_transpose_f32<<<dim3(((uint32_t)ql->tc + 255) / 256, (uint32_t)tr), 256>>>(ql->scales, (uint32_t)tr, (uint32_t)ql->tc, ql->t_scales);
        QB_CUDA_TRY(cudaGetLastError());
        ql->t_gr = ql->gc;
        ql->t_gc = ql->gr;
        ql->t_tc = tr;
    }
    if (ql->fast_gr() != 1 || ql->fast_gc() != 128) {
        // a scale that is constant over whole 128-column runs (tile widths that are multiples of 128, per-row and
        // per-tensor scales): spelt out per run, the grid is 1 x 128 and every kernel of that grid serves it
        const uint64_t vgr = ql->fast_gr(), vgc = ql->fast_gc();
        if (vgr == 0 || vgr > 0x7FFFFFFFull || (vgc < K && vgc % 128 != 0)) {
            QB_CUDA_TRY(cudaDeviceSynchronize());
            return QB200_OK;  // other grids: the prefill kernel's general issuer, the generic kernels
        }
        float* xs = nullptr;
        QB_CUDA_TRY(cudaMalloc(&xs, (uint64_t)N * groups * 4));
        const uint64_t total = (uint64_t)N * groups;
        k_expand_scales<<<(uint32_t)((total + 255) / 256), 256>>>(ql->fast_scales(), (uint32_t)ql->fast_tc(), (uint32_t)vgr, vgc, N, groups, xs);
        QB_CUDA_TRY(cudaGetLastError());
        QB_CUDA_TRY(cudaDeviceSynchronize());
        ql->x_scales = xs;  // from here on the view is 1 x 128
    }
    if (K > SLICE_LIMIT) {
        const uint32_t n = (K + SLICE_LIMIT - 1) / SLICE_LIMIT, base = groups / n, extra = groups % n;
        uint32_t widest = 0, c0 = 0;
        for (uint32_t s = 0; s < n; s++) {
            ql->slice_col0[s] = c0;
            ql->slice_width[s] = (base + (s < extra ? 1u : 0u)) * 128;
            c0 += ql->slice_width[s];
            widest = widest > ql->slice_width[s] ? widest : ql->slice_width[s];
        }
        const uint32_t pad = (widest + 511) / 512 * 512;  // rows of scales that are whole 16-byte units
        const uint64_t cbytes = (uint64_t)n * N * (pad / 2), sbytes = (uint64_t)n * N * (pad / 128) * 4;
        QB_CUDA_TRY(cudaMalloc(&ql->slice_codes, cbytes));
        QB_CUDA_TRY(cudaMalloc(&ql->slice_scales, sbytes));
        QB_CUDA_TRY(cudaMalloc(&ql->slice_partials, (uint64_t)n * 16 * N * 4));
        QB_CUDA_TRY(cudaMemset(ql->slice_codes, 0, cbytes));
        QB_CUDA_TRY(cudaMemset(ql->slice_scales, 0, sbytes));
        const uint8_t* codes = static_cast<const uint8_t*>(ql->fast_codes());
        const float* scales = ql->fast_scales();
        for (uint32_t s = 0; s < n; s++) {
            QB_CUDA_TRY(cudaMemcpy2D(static_cast<uint8_t*>(ql->slice_codes) + (uint64_t)s * N * (pad / 2), pad / 2,
                                     codes + ql->slice_col0[s] / 2, K / 2, ql->slice_width[s] / 2, N, cudaMemcpyDeviceToDevice));
            QB_CUDA_TRY(cudaMemcpy2D(ql->slice_scales + (uint64_t)s * N * (pad / 128), (pad / 128) * 4,
                                     scales + ql->slice_col0[s] / 128, groups * 4, (ql->slice_width[s] / 128) * 4, N,
                                     cudaMemcpyDeviceToDevice));
        }
        ql->n_slices = n;
        ql->slice_pad = pad;
    }
    QB_CUDA_TRY(cudaDeviceSynchronize());
    return QB200_OK;
}

qb200_status forward_sliced(qb200_qlinear* ql, const void* x, uint64_t m, void* y, int y_dtype, cudaStream_t st) {
    const uint32_t n = ql->n_slices, pad = ql->slice_pad, N = (uint32_t)ql->out_dim;
    const bool i8 = ql->bits == 8;
    const uint32_t gr = i8 ? (uint32_t)ql->fast_gr() : 1, gc = i8 ? (uint32_t)ql->fast_gc() : 128, tr = (N + gr - 1) / gr;
    const uint64_t slice_code_bytes = i8 ? (uint64_t)N * pad : (uint64_t)N * (pad / 2);
    // the int8 kernel keeps eight batch rows in registers: a batch of 9..16 is two launches over the slices
    for (uint64_t r0 = 0; r0 < m; r0 += i8 ? 8 : 16) {
        const uint64_t mr = i8 && m - r0 > 8 ? 8 : m - r0;
        FwdArgs a[SLICE_MAX];
        for (uint32_t s = 0; s < n; s++) {
            a[s].codes = static_cast<const uint8_t*>(ql->slice_codes) + s * slice_code_bytes;
            a[s].scales = ql->slice_scales + (uint64_t)s * tr * (pad / gc);
            a[s].bias = nullptr;  // added once, by the fold
            a[s].x = static_cast<const uint16_t*>(x) + r0 * ql->in_dim + ql->slice_col0[s];
            a[s].y = ql->slice_partials + ((uint64_t)s * m + r0) * N;
            a[s].m = mr;
            a[s].in_dim = pad;
            a[s].out_dim = N;
            a[s].gr = gr;
            a[s].gc = gc;
            a[s].tc = pad / gc;
            a[s].x_stride = ql->in_dim;
            a[s].k_valid = ql->slice_width[s];
        }
        const qb200_status r = i8 ? gemv_i8_forward_many(a, n, QB200_F32, ql->status, st) : gemv_i4_forward_many(a, n, QB200_F32, ql->status, st);
        if (r) return r;
    }
    const uint64_t mn = m * N;
    const uint32_t blocks = (uint32_t)((mn + 255) / 256 > 592 ? 592 : (mn + 255) / 256);
    if (y_dtype == QB200_F32)
        k_fold_slices<float><<<blocks, 256, 0, st>>>(ql->slice_partials, n, mn, N, ql->bias, static_cast<float*>(y));
    else
        k_fold_slices<uint16_t><<<blocks, 256, 0, st>>>(ql->slice_partials, n, mn, N, ql->bias, static_cast<uint16_t*>(y));
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

}  // namespace qb
