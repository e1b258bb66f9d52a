// The QuantizedLinear handle: validation at construction (the reference's
// QuantizedLinear::new, crates/ml/quanta-nn/src/quant.rs:853-862) and kernel
// selection per forward (the body of Layer::apply, quant.rs:903-918).
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "forward.hpp"

#include "qlinear_handle.hpp"

using qb::fail;

namespace {

uint64_t dtype_size(int32_t dt) { return dt == QB200_F32 ? 4 : 2; }

// Base and size of the CUDA host allocation (cudaHostAlloc / cudaHostRegister) that holds p, from the driver.
bool host_range(const void* p, void** base, size_t* size) {
    typedef CUresult (*Fn)(void*, CUpointer_attribute, CUdeviceptr);
    static Fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &f, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<Fn>(f);
    }
    if (!fn) return false;
    CUdeviceptr start = 0;
    size_t sz = 0;
    if (fn(&start, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS ||
        fn(&sz, CU_POINTER_ATTRIBUTE_RANGE_SIZE, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS || !start || !sz)
        return false;
    *base = reinterpret_cast<void*>(start);
    *size = sz;
    return true;
}

// Grow-only scratch.  Growing frees and allocates, which synchronises the device and is illegal while `capturing` (the
// stream the forward was given) records a CUDA graph: that case is refused with a message instead of breaking the capture.
qb200_status grow(void** p, uint64_t* have, uint64_t need, cudaStream_t capturing = nullptr) {
    if (*have >= need) return QB200_OK;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(capturing, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone)
        return fail(QB200_ERR_INVALID_PARAM, "QuantizedLinear: this forward needs " + std::to_string(need) +
                                                 " bytes of scratch that are not allocated yet, and its stream is recording a CUDA graph; "
                                                 "run the same shape once before the capture");
    cudaGetLastError();
    if (*p) QB_CUDA_TRY(cudaFree(*p));
    *p = nullptr;
    *have = 0;
    QB_CUDA_TRY(cudaMalloc(p, need));
    *have = need;
    return QB200_OK;
}

// The forward's arguments over what the fast kernels read (the transposed copy of an [in, out] weight when
// there is one, else the stored buffers).
qb::FwdArgs fast_args(const qb200_qlinear* q, const void* x, void* y, uint64_t m) {
    qb::FwdArgs a;
    a.codes = q->fast_codes();
    a.scales = q->fast_scales();
    a.bias = q->bias;
    a.x = x;
    a.y = y;
    a.m = m;
    a.in_dim = q->in_dim;
    a.out_dim = q->out_dim;
    a.gr = q->fast_gr();
    a.gc = q->fast_gc();
    a.tc = q->fast_tc();
    return a;
}

// The forward's arguments over the stored buffers.
qb::FwdArgs stored_args(const qb200_qlinear* q, const void* x, void* y, uint64_t m) {
    qb::FwdArgs a;
    a.codes = q->codes;
    a.scales = q->scales;
    a.bias = q->bias;
    a.x = x;
    a.y = y;
    a.m = m;
    a.in_dim = q->in_dim;
    a.out_dim = q->out_dim;
    a.gr = q->gr;
    a.gc = q->gc;
    a.tc = q->tc;
    return a;
}

bool decode_i8_eligible(const qb200_qlinear* q, uint64_t m, int x_dtype, const void* x) {
    return q->fast_view() && qb::gemv_i8_eligible(q->bits, q->fast_gr(), q->fast_gc(), QB200_OUT_IN, q->in_dim, q->out_dim, m, x_dtype,
                                                  q->fast_codes(), x);
}

bool decode_eligible(const qb200_qlinear* q, uint64_t m, int x_dtype, const void* x) {
    return q->fast_view() && qb::gemv_i4_eligible(q->bits, q->fast_gr(), q->fast_gc(), QB200_OUT_IN, q->in_dim, q->out_dim, m,
                                                  x_dtype, q->fast_codes(), q->fast_scales(), x);
}

// Whether a forward of m bf16 rows (at a 16-byte aligned address) would take one of the fast kernels.
bool bf16_fast(const qb200_qlinear* q, uint64_t m) {
    const void* aligned = reinterpret_cast<const void*>(uintptr_t(256));  // only its alignment is looked at
    if (decode_eligible(q, m, QB200_BF16, aligned) || decode_i8_eligible(q, m, QB200_BF16, aligned)) return true;
    if (m > 8 && m <= 16 && decode_i8_eligible(q, 8, QB200_BF16, aligned)) return true;
    if (q->n_slices && m <= 16) return true;
    if (!q->fast_view()) return false;
    return qb::gemm_i4_eligible(q->bits, q->fast_gr(), q->fast_gc(), QB200_OUT_IN, q->in_dim, q->out_dim, m, QB200_BF16, q->fast_codes(), aligned) ||
           qb::gemm_i8_eligible(q->bits, q->fast_gr(), q->fast_gc(), QB200_OUT_IN, q->in_dim, q->out_dim, m, QB200_BF16, q->fast_codes(), aligned);
}

}  // namespace

extern "C" {

qb200_status qb200_qlinear_create(const void* codes_dev, const float* scales_dev, uint64_t rows, uint64_t cols,
                                  uint32_t bits, uint64_t gr, uint64_t gc, int32_t layout, const float* bias_dev,
                                  uint64_t bias_len, qb200_qlinear** out) {
    if (!out) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_create: null output pointer");
    *out = nullptr;
    uint64_t tr, tc, cbytes;
    if (qb200_status s = qb200_codes_bytes(rows, cols, bits, &cbytes)) return s;
    if (qb200_status s = qb200_scales_count(rows, cols, gr, gc, &tr, &tc)) return s;
    if (layout != QB200_IN_OUT && layout != QB200_OUT_IN)
        return fail(QB200_ERR_INVALID_PARAM, "QuantizedLinear: unknown weight layout " + std::to_string(layout));
    if (!codes_dev || !scales_dev) return fail(QB200_ERR_INVALID_PARAM, "QuantizedLinear: null codes or scales pointer");
    const uint64_t in_dim = layout == QB200_IN_OUT ? rows : cols;
    const uint64_t out_dim = layout == QB200_IN_OUT ? cols : rows;
    if (bias_dev && bias_len != out_dim)
        return fail(QB200_ERR_INVALID_PARAM, "QuantizedLinear: bias shape [" + std::to_string(bias_len) +
                                                 "], weight [in, " + std::to_string(out_dim) + "] wants [" +
                                                 std::to_string(out_dim) + "]");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        return fail(QB200_ERR_CUDA, "QuantizedLinear: no CUDA device is available (this library has no CPU path)");
    }
    auto* ql = new qb200_qlinear();
    {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, codes_dev) == cudaSuccess && at.type == cudaMemoryTypeDevice) ql->device = at.device;
        else cudaGetLastError();
    }
    ql->codes = codes_dev;
    ql->scales = scales_dev;
    ql->bias = bias_dev;
    ql->rows = rows;
    ql->cols = cols;
    ql->gr = gr;
    ql->gc = gc;
    ql->tc = tc;
    ql->bits = bits;
    ql->layout = layout;
    ql->in_dim = in_dim;
    ql->out_dim = out_dim;
    if (cudaMalloc(&ql->status, sizeof(int32_t)) != cudaSuccess || cudaMemset(ql->status, 0, sizeof(int32_t)) != cudaSuccess) {
        cudaGetLastError();
        delete ql;
        return fail(QB200_ERR_CUDA, "QuantizedLinear: could not allocate the device status word");
    }
    if (qb200_status s = qb::build_exec_layout(ql)) {  // transposed / sliced copies for the fast int4 kernels
        qb200_qlinear_destroy(ql);
        return s;
    }
    *out = ql;
    return QB200_OK;
}

void qb200_qlinear_destroy(qb200_qlinear* ql) {
    if (!ql) return;
    qb::free_exec_layout(ql);
    if (ql->status) cudaFree(ql->status);
    if (ql->scratch) cudaFree(ql->scratch);
    if (ql->x_stage) cudaFree(ql->x_stage);
    if (ql->y_stage) cudaFree(ql->y_stage);
    if (ql->split_stage) cudaFree(ql->split_stage);
    if (ql->host_stream) cudaStreamDestroy(ql->host_stream);
    delete ql;
}

uint64_t qb200_qlinear_in_dim(const qb200_qlinear* ql) { return ql ? ql->in_dim : 0; }
uint64_t qb200_qlinear_out_dim(const qb200_qlinear* ql) { return ql ? ql->out_dim : 0; }
const char* qb200_qlinear_last_kernel(const qb200_qlinear* ql) { return ql ? ql->last_kernel : ""; }

qb200_status qb200_qlinear_forward(qb200_qlinear* ql, const void* x_dev, int32_t x_dtype, uint64_t m, void* y_dev,
                                   int32_t y_dtype, void* stream) {
    if (!ql) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward: null handle");
    if (!x_dev || !y_dev) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward: null device pointer");
    if ((x_dtype != QB200_F32 && x_dtype != QB200_BF16) || (y_dtype != QB200_F32 && y_dtype != QB200_BF16))
        return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward: activations are f32 or bf16");
    if (m == 0) return QB200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static const bool split_f32 = [] { const char* e = getenv("QB200_F32_SPLIT"); return !(e && e[0] == '0'); }();
    // (small layers at small batches stay on the generic kernel: one launch of a few microseconds beats the split's three;
    // measured, one layer per launch: [1024, 1024] at 8 rows 9 us generic against 15 us split, [4096, 4096] at one row a
    // tie at 10 us, at 8 rows 58 us against 20 us)
    if (x_dtype == QB200_F32 && split_f32 && m <= 0x7FFFFFFFull / 3 && m * ql->in_dim * ql->out_dim >= (1ull << 24) && bf16_fast(ql, 3 * m)) {
        // f32 activations (the reference's own dtype) on the bf16 kernels: x is the exact sum of three bf16 parts, the
        // kernels' products are exact, so three times the rows and one fold give the exact-product result
        const uint64_t xs_bytes = (3 * m * ql->in_dim * 2 + 255) & ~uint64_t(255);
        if (qb200_status s = grow(&ql->split_stage, &ql->split_stage_bytes, xs_bytes + 3 * m * ql->out_dim * 4, st)) return s;
        float* ys = reinterpret_cast<float*>(static_cast<uint8_t*>(ql->split_stage) + xs_bytes);
        if (qb200_status s = qb::split_f32_activations(static_cast<const float*>(x_dev), m, ql->in_dim, ql->split_stage, st)) return s;
        const float* bias = ql->bias;
        ql->bias = nullptr;  // added once, by the fold
        const qb200_status s = qb200_qlinear_forward(ql, ql->split_stage, QB200_BF16, 3 * m, ys, QB200_F32, stream);
        ql->bias = bias;
        if (s) return s;
        return qb::fold_split_outputs(ys, m, ql->out_dim, bias, y_dev, y_dtype, st);
    }
    if (decode_eligible(ql, m, x_dtype, x_dev)) {
        qb200_status s = qb::gemv_i4_forward(fast_args(ql, x_dev, y_dev, m), y_dtype, ql->status, st);
        if (s != QB200_ERR_NOT_SUPPORTED) {
            ql->last_kernel = "gemv_mma";
            return s;
        }
    }
    if (decode_i8_eligible(ql, m, x_dtype, x_dev)) {
        const qb::FwdArgs a8 = fast_args(ql, x_dev, y_dev, m);
        qb200_status s = qb::gemv_i8_forward_many(&a8, 1, y_dtype, ql->status, st);
        if (s != QB200_ERR_NOT_SUPPORTED) {
            ql->last_kernel = "gemv_mma_i8";
            return s;
        }
    } else if (m > 8 && m <= 16 && decode_i8_eligible(ql, 8, x_dtype, x_dev)) {
        // the int8 decode kernel keeps eight batch rows in registers: a batch of 9..16 runs as two launches (the second
        // pass over a layer that fits L2 re-reads it from there)
        const uint64_t ysz = y_dtype == QB200_F32 ? 4 : 2;
        qb::FwdArgs lo = fast_args(ql, x_dev, y_dev, 8);
        qb::FwdArgs hi = fast_args(ql, static_cast<const uint16_t*>(x_dev) + 8 * ql->in_dim,
                                     static_cast<uint8_t*>(y_dev) + 8 * ql->out_dim * ysz, m - 8);
        qb200_status s = qb::gemv_i8_forward_many(&lo, 1, y_dtype, ql->status, st);
        if (s == QB200_OK) s = qb::gemv_i8_forward_many(&hi, 1, y_dtype, ql->status, st);
        if (s != QB200_ERR_NOT_SUPPORTED) {
            ql->last_kernel = "gemv_mma_i8_x2";
            return s;
        }
    }
    if (ql->n_slices && m <= 16 && x_dtype == QB200_BF16 && (reinterpret_cast<uintptr_t>(x_dev) & 15u) == 0) {
        qb200_status s = qb::forward_sliced(ql, x_dev, m, y_dev, y_dtype, st);
        if (s != QB200_ERR_NOT_SUPPORTED) {
            ql->last_kernel = ql->bits == 8 ? "gemv_mma_i8_sliced" : "gemv_mma_sliced";
            return s;
        }
    }
    if (ql->fast_view() && qb::gemm_i4_eligible(ql->bits, ql->fast_gr(), ql->fast_gc(), QB200_OUT_IN, ql->in_dim, ql->out_dim, m,
                                                x_dtype, ql->fast_codes(), x_dev)) {
        // outputs with few tiles split the K loop over the idle SM pairs: partial tiles in the handle's scratch
        const uint64_t need = qb::gemm_i4_scratch_bytes(m, ql->in_dim, ql->out_dim, ql->fast_gr(), ql->fast_gc(), ql->bias);
        if (need) {
            void* p = ql->scratch;
            qb200_status s = grow(&p, &ql->scratch_bytes, need, st);
            ql->scratch = static_cast<float*>(p);
            if (s) return s;
        }
        ql->last_kernel = "gemm_tcgen05";
        return qb::gemm_i4_forward(fast_args(ql, x_dev, y_dev, m), y_dtype, need ? ql->scratch : nullptr, ql->status, st);
    }
    if (ql->fast_view() && qb::gemm_i8_eligible(ql->bits, ql->fast_gr(), ql->fast_gc(), QB200_OUT_IN, ql->in_dim, ql->out_dim, m,
                                                x_dtype, ql->fast_codes(), x_dev)) {
        const uint64_t need = qb::gemm_i8_scratch_bytes(m, ql->in_dim, ql->out_dim, ql->fast_gc(), ql->bias);
        if (need) {
            void* p = ql->scratch;
            qb200_status s = grow(&p, &ql->scratch_bytes, need, st);
            ql->scratch = static_cast<float*>(p);
            if (s) return s;
        }
        ql->last_kernel = "gemm_tcgen05_i8";
        return qb::gemm_i8_forward(fast_args(ql, x_dev, y_dev, m), y_dtype, need ? ql->scratch : nullptr, ql->status, st);
    }
    const qb::FwdArgs a = stored_args(ql, x_dev, y_dev, m);
    if (ql->layout == QB200_OUT_IN) {
        ql->last_kernel = "generic_rows";
        return qb::forward_generic(a, ql->bits, x_dtype, y_dtype, true, nullptr, 1, st);
    }
    const uint32_t slices = qb::forward_cols_slices(ql->in_dim, ql->out_dim, m);
    if (slices > 1) {
        void* p = ql->scratch;
        qb200_status s = grow(&p, &ql->scratch_bytes, (uint64_t)slices * m * ql->out_dim * sizeof(float), st);
        ql->scratch = static_cast<float*>(p);
        if (s) return s;
    }
    ql->last_kernel = "generic_cols";
    return qb::forward_generic(a, ql->bits, x_dtype, y_dtype, false, ql->scratch, slices, st);
}

qb200_status qb200_qlinear_forward_many(qb200_qlinear* const* layers, uint32_t count, const void* const* x_dev,
                                        int32_t x_dtype, uint64_t m, void* const* y_dev, int32_t y_dtype,
                                        void* stream) {
    if (count == 0 || m == 0) return QB200_OK;
    if (!layers || !x_dev || !y_dev) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many: null argument");
    for (uint32_t i = 0; i < count; i++)
        if (!layers[i] || !x_dev[i] || !y_dev[i])
            return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many: null entry " + std::to_string(i));
    // One persistent launch when every layer takes the decode GEMV and they share the input width.
    bool grouped = count > 1 && (y_dtype == QB200_F32 || y_dtype == QB200_BF16);
    for (uint32_t i = 0; i < count && grouped; i++)
        grouped = layers[i]->in_dim == layers[0]->in_dim && decode_eligible(layers[i], m, x_dtype, x_dev[i]);
    if (grouped) {
        std::vector<qb::FwdArgs> args(count);
        for (uint32_t i = 0; i < count; i++) args[i] = fast_args(layers[i], x_dev[i], y_dev[i], m);
        qb200_status s = qb::gemv_i4_forward_many(args.data(), count, y_dtype, layers[0]->status,
                                                  static_cast<cudaStream_t>(stream));
        if (s != QB200_ERR_NOT_SUPPORTED) {
            for (uint32_t i = 0; i < count; i++) layers[i]->last_kernel = "gemv_mma_grouped";
            return s;
        }
    }
    bool grouped8 = count > 1 && count <= 32 && (y_dtype == QB200_F32 || y_dtype == QB200_BF16);
    for (uint32_t i = 0; i < count && grouped8; i++)
        grouped8 = layers[i]->in_dim == layers[0]->in_dim && decode_i8_eligible(layers[i], m, x_dtype, x_dev[i]);
    if (grouped8) {  // int8 layers that share the input width: one persistent launch as well
        std::vector<qb::FwdArgs> args(count);
        for (uint32_t i = 0; i < count; i++) args[i] = fast_args(layers[i], x_dev[i], y_dev[i], m);
        qb200_status s = qb::gemv_i8_forward_many(args.data(), count, y_dtype, layers[0]->status, static_cast<cudaStream_t>(stream));
        if (s != QB200_ERR_NOT_SUPPORTED) {
            for (uint32_t i = 0; i < count; i++) layers[i]->last_kernel = "gemv_mma_i8_grouped";
            return s;
        }
    }
    for (uint32_t i = 0; i < count; i++)
        if (qb200_status s = qb200_qlinear_forward(layers[i], x_dev[i], x_dtype, m, y_dev[i], y_dtype, stream)) return s;
    return QB200_OK;
}

qb200_status qb200_qlinear_forward_many_gather(qb200_qlinear* const* layers, uint32_t count, const void* const* x_dev,
                                               int32_t x_dtype, uint64_t m, void* const* y_own, int32_t y_dtype,
                                               void* const* gather_bases, uint64_t* const* flag_arrays, uint32_t world,
                                               uint32_t rank, void* stream) {
    if (count == 0 || m == 0) return QB200_OK;
    if (!layers || !x_dev || !y_own || !gather_bases || world == 0 || world > 8 || rank >= world)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_gather: null argument or bad world / rank");
    for (uint32_t p = 0; p < world; p++)
        if (!gather_bases[p]) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_gather: null gather buffer");
    std::vector<qb::FwdArgs> args(count);
    for (uint32_t i = 0; i < count; i++) {
        const qb200_qlinear* q = layers[i];
        if (!q || !x_dev[i] || !y_own[i])
            return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_gather: null entry " + std::to_string(i));
        if (q->in_dim != layers[0]->in_dim || !decode_eligible(q, m, x_dtype, x_dev[i]))
            return fail(QB200_ERR_NOT_SUPPORTED, "qb200_qlinear_forward_many_gather: layer " + std::to_string(i) +
                                                     " does not take the decode kernel (int4, 1x128, [out, in], bf16 x, m <= 16, in <= 4096)");
        args[i] = fast_args(q, x_dev[i], y_own[i], m);
    }
    qb::PeerSpec peers;
    peers.world = world;
    peers.rank = rank;
    if (flag_arrays)
        for (uint32_t p = 0; p < world; p++) {
            if (!flag_arrays[p]) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_gather: null flag array");
            peers.flags[p] = flag_arrays[p];
        }
    for (uint32_t p = 0; p < world; p++)
        peers.delta[p] = static_cast<int64_t>(reinterpret_cast<intptr_t>(gather_bases[p]) - reinterpret_cast<intptr_t>(gather_bases[rank]));
    qb200_status s = qb::gemv_i4_forward_many(args.data(), count, y_dtype, layers[0]->status, static_cast<cudaStream_t>(stream), &peers);
    if (s == QB200_ERR_NOT_SUPPORTED)
        return fail(QB200_ERR_NOT_SUPPORTED, "qb200_qlinear_forward_many_gather: no launch plan with peer stores fits this shape (m <= 16, K <= 4096)");
    if (s == QB200_OK)
        for (uint32_t i = 0; i < count; i++) layers[i]->last_kernel = "gemv_mma_grouped_gather";
    return s;
}

qb200_status qb200_qlinear_forward_many_push(qb200_qlinear* const* layers, uint32_t count, const void* const* x_dev, int32_t x_dtype,
                                             uint64_t m, void* const* slot_own, void* const* arena_bases, uint32_t world, uint32_t rank,
                                             uint64_t* state_own, uint64_t slot_stride, void* stream) {
    if (count == 0 || m == 0) return QB200_OK;
    if (!layers || !x_dev || !slot_own || !arena_bases || !state_own || world == 0 || world > 8 || rank >= world)
        return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_push: null argument or bad world / rank");
    std::vector<qb::FwdArgs> args(count);
    for (uint32_t i = 0; i < count; i++) {
        const qb200_qlinear* q = layers[i];
        if (!q || !x_dev[i] || !slot_own[i] || (reinterpret_cast<uintptr_t>(slot_own[i]) & 7u))
            return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_push: null or misaligned entry " + std::to_string(i));
        if (q->in_dim != layers[0]->in_dim || !decode_eligible(q, m, x_dtype, x_dev[i]))
            return fail(QB200_ERR_NOT_SUPPORTED, "qb200_qlinear_forward_many_push: layer " + std::to_string(i) +
                                                     " does not take the decode kernel (int4, 1x128, [out, in], bf16 x, m <= 16, in <= 4096)");
        args[i] = fast_args(q, x_dev[i], slot_own[i], m);
    }
    qb::PeerSpec peers;
    peers.world = world;
    peers.rank = rank;
    for (uint32_t p = 0; p < world; p++) {
        if (!arena_bases[p]) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_push: null arena");
        peers.delta[p] = static_cast<int64_t>(reinterpret_cast<intptr_t>(arena_bases[p]) - reinterpret_cast<intptr_t>(arena_bases[rank]));
    }
    peers.flags[rank] = state_own;
    if (slot_stride & 7u) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_push: slot_stride must be a multiple of 8 bytes");
    peers.slot_stride = world > 1 ? slot_stride : 0;
    qb200_status s = qb::gemv_i4_forward_many(args.data(), count, qb::QB_Y_PUSHED, layers[0]->status, static_cast<cudaStream_t>(stream), &peers);
    if (s == QB200_ERR_NOT_SUPPORTED)
        return fail(QB200_ERR_NOT_SUPPORTED, "qb200_qlinear_forward_many_push: the layers do not fit ONE launch of the decode kernel");
    if (s == QB200_OK)
        for (uint32_t i = 0; i < count; i++) layers[i]->last_kernel = "gemv_mma_grouped_push";
    return s;
}

qb200_status qb200_qlinear_forward_many_host(qb200_qlinear* const* layers, uint32_t count, const void* const* x_host,
                                             int32_t x_dtype, uint64_t m, void* const* y_host, int32_t y_dtype) {
    if (count == 0 || m == 0) return QB200_OK;
    if (!layers || !x_host || !y_host) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_host: null argument");
    qb200_qlinear* lead = layers[0];
    if (!lead) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_host: null entry 0");
    // every distinct input is copied once; outputs are packed back to back in one staging buffer
    std::vector<uint64_t> x_off(count), y_off(count);
    std::vector<const void*> uniq;
    std::vector<uint64_t> uniq_off;
    uint64_t xb = 0, yb = 0;
    for (uint32_t i = 0; i < count; i++) {
        if (!layers[i] || !x_host[i] || !y_host[i])
            return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_many_host: null entry " + std::to_string(i));
        size_t k = 0;
        while (k < uniq.size() && uniq[k] != x_host[i]) k++;
        if (k == uniq.size()) {
            uniq.push_back(x_host[i]);
            uniq_off.push_back(xb);
            xb += (m * layers[i]->in_dim * dtype_size(x_dtype) + 255) & ~uint64_t(255);
        }
        x_off[i] = uniq_off[k];
        y_off[i] = yb;
        yb += (m * layers[i]->out_dim * dtype_size(y_dtype) + 255) & ~uint64_t(255);
    }
    if (qb200_status s = grow(&lead->x_stage, &lead->x_stage_bytes, xb)) return s;
    if (qb200_status s = grow(&lead->y_stage, &lead->y_stage_bytes, yb)) return s;
    if (!lead->host_stream) QB_CUDA_TRY(cudaStreamCreateWithFlags(&lead->host_stream, cudaStreamNonBlocking));
    cudaStream_t st = lead->host_stream;
    for (size_t k = 0; k < uniq.size(); k++) {
        uint64_t in_dim = 0;
        for (uint32_t i = 0; i < count; i++)
            if (x_host[i] == uniq[k]) in_dim = layers[i]->in_dim;
        QB_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(lead->x_stage) + uniq_off[k], uniq[k],
                                    m * in_dim * dtype_size(x_dtype), cudaMemcpyHostToDevice, st));
    }
    std::vector<const void*> xd(count);
    std::vector<void*> yd(count);
    // Outputs in pinned, device-mapped host memory are written by the kernels themselves (the stores cross PCIe
    // while the launch is still streaming weights), which takes the device-to-host copy off the end of the call.
    // Only calls that the dispatcher sends to the decode kernels qualify (they store with plain instructions; the
    // tcgen05 GEMM's TMA stores and split-K workspace keep the staging path): the same test the dispatcher applies.
    bool direct = true;
    for (uint32_t i = 0; i < count && direct; i++)
        direct = decode_eligible(layers[i], m, x_dtype, lead->x_stage) || decode_i8_eligible(layers[i], m, x_dtype, lead->x_stage) ||
                 (layers[i]->n_slices && m <= 16 && x_dtype == QB200_BF16);
    // one query per host allocation: outputs inside the range of an allocation already seen reuse its mapping
    const uint8_t *range_lo = nullptr, *range_hi = nullptr, *range_dev = nullptr;
    for (uint32_t i = 0; i < count && direct; i++) {
        const uint8_t* p = static_cast<const uint8_t*>(y_host[i]);
        const uint64_t bytes = m * layers[i]->out_dim * dtype_size(y_dtype);
        if (range_lo && p >= range_lo && p + bytes <= range_hi) {
            yd[i] = const_cast<uint8_t*>(range_dev + (p - range_lo));
            continue;
        }
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, p) != cudaSuccess || at.type != cudaMemoryTypeHost || !at.devicePointer) {
            cudaGetLastError();
            direct = false;
            break;
        }
        yd[i] = at.devicePointer;
        void* base = nullptr;
        size_t size = 0;
        range_lo = nullptr;
        if (host_range(p, &base, &size)) {  // without range information from the driver every pointer is queried
            if (p + bytes > static_cast<const uint8_t*>(base) + size) {
                direct = false;  // the output runs past the end of its allocation
                break;
            }
            range_lo = static_cast<const uint8_t*>(base);
            range_hi = range_lo + size;
            range_dev = static_cast<const uint8_t*>(at.devicePointer) - (p - range_lo);
        }
    }
    for (uint32_t i = 0; i < count; i++) {
        xd[i] = static_cast<uint8_t*>(lead->x_stage) + x_off[i];
        if (!direct) yd[i] = static_cast<uint8_t*>(lead->y_stage) + y_off[i];
    }
    if (qb200_status s = qb200_qlinear_forward_many(layers, count, xd.data(), x_dtype, m, yd.data(), y_dtype, st)) return s;
    if (direct) {
        QB_CUDA_TRY(cudaStreamSynchronize(st));
        return QB200_OK;
    }
    // outputs that are neighbours both on the host and in the staging buffer leave in one copy
    for (uint32_t i = 0; i < count;) {
        uint64_t bytes = m * layers[i]->out_dim * dtype_size(y_dtype);
        uint32_t j = i + 1;
        while (j < count && static_cast<uint8_t*>(y_host[i]) + bytes == y_host[j] && y_off[i] + bytes == y_off[j]) {
            bytes += m * layers[j]->out_dim * dtype_size(y_dtype);
            j++;
        }
        QB_CUDA_TRY(cudaMemcpyAsync(y_host[i], yd[i], bytes, cudaMemcpyDeviceToHost, st));
        i = j;
    }
    QB_CUDA_TRY(cudaStreamSynchronize(st));
    return QB200_OK;
}

qb200_status qb200_qlinear_check(qb200_qlinear* ql, void* stream) {
    if (!ql) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_check: null handle");
    int32_t st = 0;
    QB_CUDA_TRY(cudaMemcpyAsync(&st, ql->status, sizeof st, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    QB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    if (st != 0) {  // reported once: the word is cleared so that the handle stays usable
        QB_CUDA_TRY(cudaMemsetAsync(ql->status, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream)));
        QB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    }
    if (st == QB200_ERR_TIMEOUT)
        return fail(QB200_ERR_TIMEOUT, "QuantizedLinear: a device-side wait ran out of polls (an async copy never completed, or a peer rank never arrived at the barrier)");
    if (st == QB200_ERR_INVALID_PARAM)
        return fail(QB200_ERR_INVALID_PARAM, "QuantizedLinear: an activation given to the decode kernel is not finite or lies outside its "
                                             "domain |x| < 2^87; the outputs of that call are not valid");
    if (st != 0) return fail(QB200_ERR_CUDA, "QuantizedLinear: device status " + std::to_string(st));
    return QB200_OK;
}

qb200_status qb200_qlinear_forward_host(qb200_qlinear* ql, const void* x_host, int32_t x_dtype, uint64_t m,
                                        void* y_host, int32_t y_dtype) {
    if (!ql) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_host: null handle");
    if (!x_host || !y_host) return fail(QB200_ERR_INVALID_PARAM, "qb200_qlinear_forward_host: null host pointer");
    if (m == 0) return QB200_OK;
    const uint64_t xb = m * ql->in_dim * dtype_size(x_dtype), yb = m * ql->out_dim * dtype_size(y_dtype);
    if (qb200_status s = grow(&ql->x_stage, &ql->x_stage_bytes, xb)) return s;
    if (qb200_status s = grow(&ql->y_stage, &ql->y_stage_bytes, yb)) return s;
    if (!ql->host_stream) QB_CUDA_TRY(cudaStreamCreateWithFlags(&ql->host_stream, cudaStreamNonBlocking));
    QB_CUDA_TRY(cudaMemcpyAsync(ql->x_stage, x_host, xb, cudaMemcpyHostToDevice, ql->host_stream));
    // a decode-shaped call with its output in pinned, device-mapped memory: the kernel stores there itself
    void* y_direct = nullptr;
    if (decode_eligible(ql, m, x_dtype, ql->x_stage) || decode_i8_eligible(ql, m, x_dtype, ql->x_stage) ||
        (ql->n_slices && m <= 16 && x_dtype == QB200_BF16)) {
        cudaPointerAttributes at;
        void* base = nullptr;
        size_t size = 0;
        if (cudaPointerGetAttributes(&at, y_host) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer &&
            host_range(y_host, &base, &size) && static_cast<uint8_t*>(y_host) + yb <= static_cast<uint8_t*>(base) + size)
            y_direct = at.devicePointer;
        else
            cudaGetLastError();
    }
    if (qb200_status s = qb200_qlinear_forward(ql, ql->x_stage, x_dtype, m, y_direct ? y_direct : ql->y_stage, y_dtype, ql->host_stream))
        return s;
    if (!y_direct) QB_CUDA_TRY(cudaMemcpyAsync(y_host, ql->y_stage, yb, cudaMemcpyDeviceToHost, ql->host_stream));
    QB_CUDA_TRY(cudaStreamSynchronize(ql->host_stream));
    return QB200_OK;
}

}  // extern "C"
