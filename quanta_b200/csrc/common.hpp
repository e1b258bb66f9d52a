// Shared host-side plumbing of the qb200 library: status codes, the per-thread
// error message and CUDA error mapping.
#pragma once
#include <cstdint>
#include <string>

#include "../../include/qb200.h"

namespace qb {

// Records `msg` as the calling thread's last error and returns `code`.
qb200_status fail(qb200_status code, const std::string& msg);
void clear_error();

inline uint64_t div_ceil(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

// Rust-style `[a, b]` list formatting used by the reference's messages.
std::string fmt_shape(const uint64_t* dims, size_t n);

}  // namespace qb

#ifdef __CUDACC__
#include <cuda_runtime.h>
#define QB_CUDA_TRY(expr)                                                                  \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return qb::fail(QB200_ERR_CUDA, std::string("CUDA error in " #expr ": ") +     \
                                                cudaGetErrorString(_e));                   \
    } while (0)
#endif
