// Tensor parallelism behind the C ABI: shard arithmetic, a communicator over NCCL, and the sharded forwards whose
// exchange is a library collective — the path for every shape the fused kernels do not take (prefill batches, int8
// layers, inputs wider than the decode kernel's) and for hosts without peer access between their GPUs.  The
// reference has no multi-GPU code (crates/ml/quanta-nn/PARITY.md:76-79).
//
// NCCL is not linked: libnccl.so.2 is opened at run time (the process usually has one loaded already), and only
// its public C API is used (ncclGetUniqueId, ncclCommInitRank, ncclAllGather, ncclAllReduce, ncclCommDestroy).
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>

#include "forward.hpp"
#include "qlinear_handle.hpp"
#include "quant_math.cuh"

namespace qb {

// the slice of NCCL's public API this file calls (nccl.h: ncclResult_t is an int, 0 = success; ncclUniqueId is 128 bytes)
struct NcclId {
    char internal[128];
};
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(void** comm, int nranks, NcclId id, int rank) = nullptr;
    int (*CommDestroy)(void* comm) = nullptr;
    int (*AllGather)(const void* send, void* recv, size_t count, int dtype, void* comm, cudaStream_t st) = nullptr;
    int (*AllReduce)(const void* send, void* recv, size_t count, int dtype, int op, void* comm, cudaStream_t st) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string error;
};
constexpr int NCCL_FLOAT32 = 7, NCCL_UINT8 = 1, NCCL_SUM = 0;  // ncclDataType_t / ncclRedOp_t values of nccl.h

static NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.lib) break;
        }
        if (!api.lib) {
            api.error = std::string("libnccl.so.2 could not be opened (") + (dlerror() ? dlerror() : "no detail") + ")";
            return;
        }
        auto sym = [&](const char* name) {
            void* p = dlsym(api.lib, name);
            if (!p && api.error.empty()) api.error = std::string("libnccl has no symbol ") + name;
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    });
    return api;
}

static qb200_status nccl_fail(const char* what, int rc) {
    NcclApi& n = nccl();
    return fail(QB200_ERR_NCCL, std::string(what) + ": " + (n.GetErrorString ? n.GetErrorString(rc) : "NCCL error") + " (" + std::to_string(rc) + ")");
}

// [world][m][per] gathered shards -> [m][out_total]; shard r holds columns [r * per, min((r + 1) * per, out_total)).
template <typename T>
__global__ void __launch_bounds__(256) k_unpad_gathered(const T* __restrict__ src, uint64_t m, uint64_t per, uint64_t out_total,
                                                        T* __restrict__ dst) {
    const uint64_t total = m * out_total;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / out_total, col = i % out_total, r = col / per;
        dst[i] = src[(r * m + row) * per + (col - r * per)];
    }
}

}  // namespace qb

struct qb200_tp {
    void* comm = nullptr;
    uint32_t rank = 0, world = 1;
    int device = 0;
    void* stage = nullptr;  // [world + 1][m][n_max] of the output type: the local shard padded, then the gathered shards
    uint64_t stage_bytes = 0;
    int32_t* status = nullptr;
};

using qb::fail;

extern "C" {

qb200_status qb200_shard_rows(uint64_t rows, uint64_t gr, uint32_t world, uint32_t rank, uint64_t* lo, uint64_t* hi) {
    if (!lo || !hi || world == 0 || rank >= world || gr == 0)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_shard_rows: rank " + std::to_string(rank) + " outside a world of " + std::to_string(world) +
                                                 ", or a zero tile height");
    uint64_t per = qb::div_ceil(rows, world);
    per = qb::div_ceil(per, gr) * gr;  // no scale tile straddles a boundary
    const uint64_t a = rank * per < rows ? rank * per : rows;
    *lo = a;
    *hi = a + per < rows ? a + per : rows;
    return QB200_OK;
}

qb200_status qb200_shard_cols(uint64_t cols, uint64_t gc, uint32_t bits, uint32_t world, uint32_t rank, uint64_t* lo, uint64_t* hi) {
    if (gc == 0 || (bits != 4 && bits != 8)) return fail(QB200_ERR_INVALID_PARAM, "qb200_shard_cols: zero tile width or bits not 4 / 8");
    uint64_t mult = gc;
    if (bits == 4 && gc % 8 != 0) {  // whole packed words as well as whole tiles: lcm(gc, 8)
        uint64_t a = gc, b = 8;
        while (b) {
            const uint64_t t = a % b;
            a = b;
            b = t;
        }
        mult = gc / a * 8;
    }
    return qb200_shard_rows(cols, mult, world, rank, lo, hi);
}

qb200_status qb200_tp_unique_id(uint8_t* id128) {
    if (!id128) return fail(QB200_ERR_INVALID_PARAM, "qb200_tp_unique_id: null output");
    qb::NcclApi& n = qb::nccl();
    if (!n.error.empty()) return fail(QB200_ERR_NCCL, "qb200_tp_unique_id: " + n.error);
    qb::NcclId id;
    if (int rc = n.GetUniqueId(&id)) return qb::nccl_fail("ncclGetUniqueId", rc);
    std::memcpy(id128, &id, 128);
    return QB200_OK;
}

qb200_status qb200_tp_create(uint32_t rank, uint32_t world, const uint8_t* id128, qb200_tp** out) {
    if (!out) return fail(QB200_ERR_INVALID_PARAM, "qb200_tp_create: null output pointer");
    *out = nullptr;
    if (world == 0 || rank >= world) return fail(QB200_ERR_INVALID_PARAM, "qb200_tp_create: rank " + std::to_string(rank) + " outside a world of " + std::to_string(world));
    if (world > 1 && !id128) return fail(QB200_ERR_INVALID_PARAM, "qb200_tp_create: a world of more than one rank needs the unique id of rank 0");
    auto* tp = new qb200_tp();
    tp->rank = rank;
    tp->world = world;
    if (cudaGetDevice(&tp->device) != cudaSuccess || cudaMalloc(&tp->status, sizeof(int32_t)) != cudaSuccess ||
        cudaMemset(tp->status, 0, sizeof(int32_t)) != cudaSuccess) {
        cudaGetLastError();
        delete tp;
        return fail(QB200_ERR_CUDA, "qb200_tp_create: no usable CUDA device (this library has no CPU path)");
    }
    if (world > 1) {
        qb::NcclApi& n = qb::nccl();
        if (!n.error.empty()) {
            cudaFree(tp->status);
            delete tp;
            return fail(QB200_ERR_NCCL, "qb200_tp_create: " + n.error);
        }
        qb::NcclId id;
        std::memcpy(&id, id128, 128);
        if (int rc = n.CommInitRank(&tp->comm, (int)world, id, (int)rank)) {
            cudaFree(tp->status);
            delete tp;
            return qb::nccl_fail("ncclCommInitRank", rc);
        }
    }
    *out = tp;
    return QB200_OK;
}

void qb200_tp_destroy(qb200_tp* tp) {
    if (!tp) return;
    if (tp->comm) qb::nccl().CommDestroy(tp->comm);
    if (tp->stage) cudaFree(tp->stage);
    if (tp->status) cudaFree(tp->status);
    delete tp;
}

uint32_t qb200_tp_rank(const qb200_tp* tp) { return tp ? tp->rank : 0; }
uint32_t qb200_tp_world(const qb200_tp* tp) { return tp ? tp->world : 0; }

qb200_status qb200_qlinear_forward_tp(qb200_tp* tp, qb200_qlinear* shard, int32_t mode, uint64_t full_dim, uint64_t granule,
                                      const void* x_dev, int32_t x_dtype, uint64_t m, void* y_dev, int32_t y_dtype, void* stream) {
    if (!tp) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_tp: null communicator");
    if (!x_dev || !y_dev) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_tp: null device pointer");
    if (mode != QB200_TP_COLUMN && mode != QB200_TP_ROW) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_tp: unknown mode");
    if (m == 0) return QB200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    qb::NcclApi& n = qb::nccl();
    if (mode == QB200_TP_ROW) {
        // every rank multiplies its slice of the input features; the partial outputs are summed (f32, in place)
        if (y_dtype != QB200_F32) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_tp: the row-parallel sum is f32");
        if (shard) {
            if (shard->out_dim != full_dim)
                return fail(QB200_ERR_LENGTH, "qb200_qlinear_forward_tp: a row-parallel shard has all " + std::to_string(full_dim) +
                                                  " outputs, this one has " + std::to_string(shard->out_dim));
            if (qb200_status s = qb200_qlinear_forward(shard, x_dev, x_dtype, m, y_dev, QB200_F32, stream)) return s;
        } else {
            QB_CUDA_TRY(cudaMemsetAsync(y_dev, 0, m * full_dim * sizeof(float), st));  // a rank without columns adds zeros
        }
        if (tp->world > 1)
            if (int rc = n.AllReduce(y_dev, y_dev, m * full_dim, qb::NCCL_FLOAT32, qb::NCCL_SUM, tp->comm, st)) return qb::nccl_fail("ncclAllReduce", rc);
        return QB200_OK;
    }
    // column-parallel: rank r owns the rows qb200_shard_rows(full_dim, granule, world, r) of the [out, in] weight (equal
    // blocks of whole scale tiles; trailing ranks may be short or empty) and the shards' outputs are gathered along
    // the feature axis
    const uint64_t esz = y_dtype == QB200_F32 ? 4 : 2;
    if (y_dtype != QB200_F32 && y_dtype != QB200_BF16) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_tp: outputs are f32 or bf16");
    uint64_t lo = 0, hi = 0;
    if (qb200_status s = qb200_shard_rows(full_dim, granule ? granule : 1, tp->world, tp->rank, &lo, &hi)) return s;
    uint64_t lo0 = 0, n_max = 0;
    qb200_shard_rows(full_dim, granule ? granule : 1, tp->world, 0, &lo0, &n_max);  // the block size: rank 0's shard
    const uint64_t w_mine = hi - lo;
    if ((shard ? shard->out_dim : 0) != w_mine)
        return fail(QB200_ERR_LENGTH, "qb200_qlinear_forward_tp: rank " + std::to_string(tp->rank) + " of " + std::to_string(tp->world) + " owns " +
                                          std::to_string(w_mine) + " of " + std::to_string(full_dim) + " outputs, the shard has " +
                                          std::to_string(shard ? shard->out_dim : 0));
    if (tp->world == 1) return qb200_qlinear_forward(shard, x_dev, x_dtype, m, y_dev, y_dtype, stream);
    const uint64_t slot = m * n_max * esz, need = (tp->world + 1) * slot;
    if (tp->stage_bytes < need) {  // grows on demand: run the largest shape once before capturing into a CUDA graph
        if (tp->stage) QB_CUDA_TRY(cudaFree(tp->stage));
        tp->stage = nullptr;
        tp->stage_bytes = 0;
        QB_CUDA_TRY(cudaMalloc(&tp->stage, need));
        tp->stage_bytes = need;
    }
    uint8_t* mine = static_cast<uint8_t*>(tp->stage);
    uint8_t* all = mine + slot;
    if (w_mine != n_max || !shard) QB_CUDA_TRY(cudaMemsetAsync(mine, 0, slot, st));
    if (shard) {
        if (w_mine == n_max) {
            if (qb200_status s = qb200_qlinear_forward(shard, x_dev, x_dtype, m, mine, y_dtype, stream)) return s;
        } else {  // a narrower shard: forward into the tail of the gather area, then pad its rows to n_max
            uint8_t* tmp = all;  // overwritten by the gather afterwards
            if (qb200_status s = qb200_qlinear_forward(shard, x_dev, x_dtype, m, tmp, y_dtype, stream)) return s;
            QB_CUDA_TRY(cudaMemcpy2DAsync(mine, n_max * esz, tmp, w_mine * esz, w_mine * esz, m, cudaMemcpyDeviceToDevice, st));
        }
    }
    if (int rc = n.AllGather(mine, all, slot, qb::NCCL_UINT8, tp->comm, st)) return qb::nccl_fail("ncclAllGather", rc);
    const uint64_t total = m * full_dim;
    const uint32_t blocks = (uint32_t)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256);
    if (esz == 4)
        qb::k_unpad_gathered<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(all), m, n_max, full_dim, static_cast<float*>(y_dev));
    else
        qb::k_unpad_gathered<uint16_t><<<blocks, 256, 0, st>>>(reinterpret_cast<const uint16_t*>(all), m, n_max, full_dim,
                                                               static_cast<uint16_t*>(y_dev));
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

qb200_status qb200_tp_status(qb200_tp* tp, qb200_qlinear* shard, void* stream) {
    if (!tp) return fail(QB200_ERR_INVALID_PARAM, "qb200_tp_status: null communicator");
    if (shard) return qb200_qlinear_check(shard, stream);
    QB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return QB200_OK;
}

}  // extern "C"
