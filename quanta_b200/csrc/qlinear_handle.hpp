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
    uint64_t in_dim = 0, out_dim = 0;
    // split-K partial sums of the column kernel (grow-only)
    float* scratch = nullptr;
    uint64_t scratch_bytes = 0;
    // device staging for the host-buffer entry point (grow-only)
    void* x_stage = nullptr;
    void* y_stage = nullptr;
    uint64_t x_stage_bytes = 0, y_stage_bytes = 0;
    cudaStream_t host_stream = nullptr;
    int32_t* status = nullptr;  // device word written by kernels whose bounded waits ran out
    const char* last_kernel = "";
};
