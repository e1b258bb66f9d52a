// Internal interface between the QuantizedLinear handle and its kernels.
#pragma once
#include <cstdint>

#include "common.hpp"

namespace qb {

// One forward call: y[m, out] = x[m, in] @ deq(w) (+ bias).
struct FwdArgs {
    const void* codes;    // int8 [rows, cols] or u32 [rows, ceil(cols/8)]
    const float* scales;  // [ceil(rows/gr), tc]
    const float* bias;    // [out_dim] or null
    const void* x;        // [m, in_dim]
    void* y;              // [m, out_dim]
    uint64_t m, in_dim, out_dim;
    uint64_t gr, gc, tc;  // tile and scale-grid row length (ceil(cols/gc))
    // decode GEMV only: x may be a column window of a wider activation matrix — rows `x_stride` elements apart
    // (0: in_dim), of which only the first `k_valid` columns exist (0: in_dim; the rest read as zero)
    uint64_t x_stride = 0, k_valid = 0;
};

#ifdef __CUDACC__
// Generic kernels (forward_generic.cu).  rows_kernel: OUT_IN orientation.
qb200_status forward_generic(const FwdArgs& a, uint32_t bits, int x_dtype, int y_dtype, bool rows_kernel,
                             float* scratch, uint32_t slices, cudaStream_t st);
#endif
// Decode GEMV on the tensor pipe (gemv_decode.cu): int4, 1x128 grid, OUT_IN, bf16 x, m <= 16, in_dim <= 4096.
bool gemv_i4_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* scales, const void* x);
// Fused all-gather: byte offsets from this rank's output buffer to every rank's copy of it (as mapped in
// this process; the own entry is 0).  A kernel given a PeerSpec stores each output to all of them.
struct PeerSpec {
    uint32_t world = 0;
    int64_t delta[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // with flags, the launch also runs the arrival barrier (its last CTA signals every peer and waits for theirs):
    // flags[p] is rank p's barrier state (16 u64, zero-initialised) as mapped here
    uint64_t* flags[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    uint32_t rank = 0;
    // pushed outputs only: when non-zero, rank p's slot of an arena lies (p - rank) * slot_stride bytes from the own
    // slot and the launch polls its twins' elements in the own arena before it ends (an all-gather complete at launch end)
    uint64_t slot_stride = 0;
};
// Internal output type of the decode GEMV beside QB200_F32 / QB200_BF16: pushed self-validating elements (8 bytes:
// f32 bits + exchange number) for every rank; flags[rank] is then this rank's own state array and no barrier runs.
constexpr int QB_Y_PUSHED = 100;
// Polls of a peer's arrival flag (about 0.25 us each) before a barrier gives up with QB200_ERR_TIMEOUT (peers.cu).
uint32_t peer_spin_limit();
#ifdef __CUDACC__
// QB200_ERR_NOT_SUPPORTED (no message) when no launch plan fits the shape.
qb200_status gemv_i4_forward(const FwdArgs& a, int y_dtype, int32_t* status, cudaStream_t st);
// One persistent launch over several layers that share K and m (x and y per layer).
// With `peers`, only launch plans whose kernel can store to peer buffers are taken (else NOT_SUPPORTED).
qb200_status gemv_i4_forward_many(const FwdArgs* a, uint32_t count, int y_dtype, int32_t* status, cudaStream_t st,
                                  const PeerSpec* peers = nullptr);
#endif
// Decode GEMV over int8 codes (gemv_i8.cuh): OUT_IN, bf16 x, m <= 8, in_dim <= 4096, any grid whose tile width is a multiple of 32.
bool gemv_i8_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim, uint64_t m,
                      int x_dtype, const void* codes, const void* x);
#ifdef __CUDACC__
qb200_status gemv_i8_forward_many(const FwdArgs* a, uint32_t count, int y_dtype, int32_t* status, cudaStream_t st);
#endif
// Prefill GEMM on tcgen05 (gemm_prefill.cu): int4, OUT_IN, bf16 x; the 1x128 grid at every m (asked after the decode GEMV),
// other grids whose tile width is a multiple of 16 that divides in_dim (or covers the row) from m = 9.
bool gemm_i4_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* x);
uint64_t gemm_i4_scratch_bytes(uint64_t m, uint64_t in_dim, uint64_t out_dim, uint64_t gr, uint64_t gc, const void* bias);
#ifdef __CUDACC__
qb200_status gemm_i4_forward(const FwdArgs& a, int y_dtype, void* scratch, int32_t* status, cudaStream_t st);
#endif
// The same kernel over int8 codes: OUT_IN, bf16 x, in_dim a multiple of 64, any grid whose tile width is a multiple of
// 16 that divides in_dim (or covers the row), from m = 5; asked after the int8 decode GEMV.
bool gemm_i8_eligible(uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, uint64_t in_dim, uint64_t out_dim,
                      uint64_t m, int x_dtype, const void* codes, const void* x);
uint64_t gemm_i8_scratch_bytes(uint64_t m, uint64_t in_dim, uint64_t out_dim, uint64_t gc, const void* bias);
#ifdef __CUDACC__
qb200_status gemm_i8_forward(const FwdArgs& a, int y_dtype, void* scratch, int32_t* status, cudaStream_t st);
#endif
#ifdef __CUDACC__
// f32 activations on the bf16 kernels (forward_generic.cu).  split: x [m, k] f32 -> xs [3 m, k] bf16 with
// x = xs[i] + xs[m + i] + xs[2 m + i] exactly (two truncations and the remainder); fold: y[i] = (ys[i] + ys[m + i]) + ys[2 m + i]
// (+ bias), ys [3 m, n] f32.
qb200_status split_f32_activations(const float* x, uint64_t m, uint64_t k, void* xs, cudaStream_t st);
qb200_status fold_split_outputs(const float* ys, uint64_t m, uint64_t n, const float* bias, void* y, int y_dtype, cudaStream_t st);
#endif
// K slices the column kernel splits into (1 = no scratch needed).
uint32_t forward_cols_slices(uint64_t in_dim, uint64_t out_dim, uint64_t m);

}  // namespace qb
