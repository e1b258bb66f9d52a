// Peer buffers and the arrival barrier of the fused all-gather.
//
// Column-sharded layers need every rank's outputs on every rank.  Instead of a collective after
// the kernel, the decode kernel's service warp stores each output straight into every rank's
// gather buffer (peer memory over NVLink; plain stores, no multicast), and one small kernel
// afterwards tells the peers "my outputs of step s are written" and waits, bounded, for theirs.
// The buffers are ordinary cudaMalloc allocations shared between the node's processes with CUDA
// IPC handles, which the caller exchanges through its own process group.
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>

#include "forward.hpp"

namespace qb {

// polls of ~0.25 us each before a barrier gives up with QB200_ERR_TIMEOUT: about a second by default
static std::atomic<uint32_t> g_peer_spin_limit{0};
uint32_t peer_spin_limit() {
    uint32_t v = g_peer_spin_limit.load(std::memory_order_relaxed);
    if (v == 0) {  // first use: the environment may set the limit (QB200_SPIN_LIMIT, in polls), else 4 Mi
        const char* e = getenv("QB200_SPIN_LIMIT");
        const unsigned long long n = e ? strtoull(e, nullptr, 10) : 0;
        v = n >= 1 && n <= 0xFFFFFFFFull ? (uint32_t)n : 4u << 20;
        g_peer_spin_limit.store(v, std::memory_order_relaxed);
    }
    return v;
}

struct PeerFlags {
    uint64_t* flags[8];  // flags[p]: rank p's array {arrival of rank 0, ..., arrival of rank 7, own step counter}
};

// One launch per step and rank.  The step number lives in device memory (slot 8 of the own flag
// array), so a CUDA graph that replays this launch still counts.
__global__ void k_peer_signal_wait(PeerFlags f, uint32_t world, uint32_t rank, uint32_t spin_limit, int32_t* status) {
    __shared__ uint64_t s_step;
    if (threadIdx.x == 0) {
        s_step = f.flags[rank][8] + 1;
        f.flags[rank][8] = s_step;
    }
    __syncthreads();
    const uint64_t step = s_step;
    const uint32_t p = threadIdx.x;
    // the kernel before this one wrote this rank's outputs into every peer's buffer: order those stores
    // before the arrival flags at system scope
    __threadfence_system();
    if (p < world) {
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(f.flags[p] + rank), "l"(step) : "memory");
        const uint64_t* mine = f.flags[rank] + p;
        uint64_t v = 0;
        uint32_t spins = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
            if (v >= step || ++spins >= spin_limit) break;
            __nanosleep(200);
        }
        if (v < step) atomicExch(status, QB200_ERR_TIMEOUT);
    }
    __threadfence_system();
}

}  // namespace qb

using qb::fail;

extern "C" {

qb200_status qb200_peer_alloc(uint64_t bytes, void** dev_ptr, uint8_t* handle64) {
    if (!dev_ptr || !handle64 || bytes == 0) return fail(QB200_ERR_INVALID_PARAM, "qb200_peer_alloc: null argument or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64 bytes");
    void* p = nullptr;
    QB_CUDA_TRY(cudaMalloc(&p, bytes));
    QB_CUDA_TRY(cudaMemset(p, 0, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(QB200_ERR_CUDA, std::string("qb200_peer_alloc: cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    }
    std::memcpy(handle64, &h, 64);
    *dev_ptr = p;
    return QB200_OK;
}

qb200_status qb200_peer_open(const uint8_t* handle64, void** dev_ptr) {
    if (!dev_ptr || !handle64) return fail(QB200_ERR_INVALID_PARAM, "qb200_peer_open: null argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    void* p = nullptr;
    QB_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *dev_ptr = p;
    return QB200_OK;
}

qb200_status qb200_peer_close(void* dev_ptr) {
    if (dev_ptr) QB_CUDA_TRY(cudaIpcCloseMemHandle(dev_ptr));
    return QB200_OK;
}

qb200_status qb200_peer_free(void* dev_ptr) {
    if (dev_ptr) QB_CUDA_TRY(cudaFree(dev_ptr));
    return QB200_OK;
}

qb200_status qb200_peer_set_spin_limit(uint32_t polls) {
    if (polls == 0) return fail(QB200_ERR_INVALID_PARAM, "qb200_peer_set_spin_limit: the limit must be positive");
    qb::g_peer_spin_limit.store(polls, std::memory_order_relaxed);
    return QB200_OK;
}

qb200_status qb200_peer_signal_wait(uint64_t* const* flag_arrays, uint32_t world, uint32_t rank, int32_t* status_dev,
                                    void* stream) {
    if (!flag_arrays || !status_dev || world == 0 || world > 8 || rank >= world)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_peer_signal_wait: bad world / rank or null argument");
    qb::PeerFlags f = {};
    for (uint32_t p = 0; p < world; p++) {
        if (!flag_arrays[p]) return fail(QB200_ERR_INVALID_PARAM, "qb200_peer_signal_wait: null flag array");
        f.flags[p] = flag_arrays[p];
    }
    qb::k_peer_signal_wait<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, qb::peer_spin_limit(), status_dev);
    QB_CUDA_TRY(cudaGetLastError());
    return QB200_OK;
}

}  // extern "C"
