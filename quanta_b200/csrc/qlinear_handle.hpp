// The QuantizedLinear handle behind the C ABI (internal to the library).
#pragma once
#include <cstdint>

#include <cuda_runtime.h>

#include "common.hpp"

struct qb200_qlinear {
    const void* codes = nullptr;
    const float* scales = nullptr;
    const float* bias = nullptr;
    uint64_t rows = 0, cols = 0, gr = 0, gc = 0, tc = 0;
    uint32_t bits = 0;
    int32_t layout = QB200_IN_OUT;
    int device = -1;  // the device that holds the codes (-1: unknown)
    uint64_t in_dim = 0, out_dim = 0;
    // split-K partial sums of the column kernel (grow-only)
    float* scratch = nullptr;
    uint64_t scratch_bytes = 0;
    // device staging for the host-buffer entry point (grow-only)
    void* x_stage = nullptr;
    void* y_stage = nullptr;
    uint64_t x_stage_bytes = 0, y_stage_bytes = 0;
    cudaStream_t host_stream = nullptr;
    // f32 activations on the bf16 kernels: the three bf16 parts of x, [3 m, in_dim], and their outputs, [3 m, out_dim] f32
    // (grow-only; apart from `scratch`, which the inner call may grow)
    void* split_stage = nullptr;
    uint64_t split_stage_bytes = 0;
    // Execution layout, built once at creation where the stored layout does not feed the fast kernels as it is
    // (copies: the stored codes and scales stay the record that accessors and writers see).
    //   t_codes / t_scales: an `[in, out]` matrix transposed to `[out, in]` — int4 with Group{axis: 0, size: 128} to a
    //     1 x 128 grid, int8 with tiles of whole 16-row steps to the transposed grid (t_gr x t_gc tiles, t_tc scales
    //     per row; a permutation of the codes and of the scales);
    //   slices: inputs wider than the decode kernel keeps in registers (4096) cut into `n_slices` column runs of whole
    //     scale groups, each padded with zero codes and zero scales to `slice_pad` columns, rows contiguous.
    //   x_scales: an int4 grid whose scale is constant over whole 128-column runs (tile widths that are multiples of 128,
    //     per-row and per-tensor scales) spelt out as a 1 x 128 grid `[out_dim][in_dim / 128]`, so that the 1 x 128
    //     kernels serve it: the same scale multiplies the same codes.
    void* t_codes = nullptr;
    float* t_scales = nullptr;
    uint64_t t_gr = 0, t_gc = 0, t_tc = 0;
    float* x_scales = nullptr;
    void* slice_codes = nullptr;     // [n_slices][out_dim][slice_pad / 8] u32 (int8: [n_slices][out_dim][slice_pad] bytes)
    float* slice_scales = nullptr;   // [n_slices][out_dim][slice_pad / 128] (int8: [n_slices][ceil(out_dim / gr)][slice_pad / gc])
    float* slice_partials = nullptr; // [n_slices][16][out_dim] f32: the slices' partial outputs of one decode call
    uint32_t n_slices = 0, slice_pad = 0;
    uint32_t slice_col0[8] = {}, slice_width[8] = {};
    int32_t* status = nullptr;  // device word written by kernels whose bounded waits ran out
    const char* last_kernel = "";

    // what the fast kernels read: the transposed copy when there is one, else the stored buffers
    bool fast_view() const { return t_codes != nullptr || layout == QB200_OUT_IN; }
    const void* fast_codes() const { return t_codes ? t_codes : codes; }
    const float* fast_scales() const { return x_scales ? x_scales : t_codes ? t_scales : scales; }
    uint64_t fast_gr() const { return x_scales ? 1 : t_codes ? t_gr : gr; }
    uint64_t fast_gc() const { return x_scales ? 128 : t_codes ? t_gc : gc; }
    uint64_t fast_tc() const { return x_scales ? in_dim / 128 : t_codes ? t_tc : tc; }
};

namespace qb {
// exec_layout.cu
qb200_status build_exec_layout(qb200_qlinear* ql);
void free_exec_layout(qb200_qlinear* ql);
#ifdef __CUDACC__
// decode forward (m <= 16, bf16 x) of a handle with column slices: one grouped launch over the slices, then the fold
qb200_status forward_sliced(qb200_qlinear* ql, const void* x, uint64_t m, void* y, int y_dtype, cudaStream_t st);
#endif
}  // namespace qb
