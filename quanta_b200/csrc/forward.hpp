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
};

#ifdef __CUDACC__
// Generic kernels (forward_generic.cu).  rows_kernel: OUT_IN orientation.
qb200_status forward_generic(const FwdArgs& a, uint32_t bits, int x_dtype, int y_dtype, bool rows_kernel,
                             float* scratch, uint32_t slices, cudaStream_t st);
#endif
// K slices the column kernel splits into (1 = no scratch needed).
uint32_t forward_cols_slices(uint64_t in_dim, uint64_t out_dim, uint64_t m);

}  // namespace qb
