// qb200.hpp — C++ host-side mirror of quanta's quantized-inference API over the C ABI (qb200.h).
//
// The reference is a Rust library (`quanta::sci::quant`, `quanta::nn::quant`); this header gives
// the same vocabulary to a compiled host: QuantDtype, Granularity, QuantizedMatrix
// (quantize / from_parts / dequantize / accessors, crates/sci/quanta-array/src/quant.rs:60-637),
// QuantizedLinear (new_ / forward, crates/ml/quanta-nn/src/quant.rs:830-919), QuantLeaf,
// save_named / load_named (quant.rs:279-390, 676-729).  DeviceArray<T> stands in for the
// reference's device `Array<T>`: it owns a cudaMalloc'd buffer and a shape.  Errors are thrown as
// qb200::Error carrying the status code and the library's message (the reference returns
// Result<_, ArrayError>; messages keep its substrings).  Header-only; link libqb200 and cudart.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "qb200.h"

namespace qb200 {

class Error : public std::runtime_error {
public:
    Error(int code, const std::string& msg) : std::runtime_error(msg), code_(code) {}
    int code() const { return code_; }
    // Name of the reference arm: Rank / Granularity / Grid / Format / NotSupported / Scale / ...
    const char* kind() const {
        static const char* names[] = {"Ok", "Rank", "Granularity", "Grid", "Format", "NotSupported", "Scale",
                                      "LengthMismatch", "InvalidParam", "Cuda", "Nccl", "Timeout"};
        return code_ >= 0 && code_ < 12 ? names[code_] : "Unknown";
    }

private:
    int code_;
};

inline void check(qb200_status s) {
    if (s == QB200_OK) return;
    std::string msg(qb200_last_error(nullptr, 0) + 1, '\0');
    qb200_last_error(msg.data(), msg.size());
    msg.resize(msg.size() - 1);
    throw Error(s, msg);
}
inline void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw Error(QB200_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

enum class QuantDtype { Int8 = 8, Int4 = 4 };
inline uint32_t bits(QuantDtype d) { return static_cast<uint32_t>(d); }

struct Granularity {
    int32_t kind;
    uint64_t axis = 0, size = 0, size2 = 0;
    static Granularity PerTensor() { return {QB200_PER_TENSOR}; }
    static Granularity PerChannel(uint64_t axis) { return {QB200_PER_CHANNEL, axis}; }
    static Granularity Group(uint64_t axis, uint64_t size) { return {QB200_GROUP, axis, size}; }
    static Granularity Block(uint64_t rows, uint64_t cols) { return {QB200_BLOCK, 0, rows, cols}; }
    std::pair<uint64_t, uint64_t> tile(uint64_t rows, uint64_t cols) const {
        uint64_t gr = 0, gc = 0;
        check(qb200_tile(kind, axis, size, size2, rows, cols, &gr, &gc));
        return {gr, gc};
    }
    bool operator==(const Granularity& o) const { return kind == o.kind && axis == o.axis && size == o.size && size2 == o.size2; }
};

// A device buffer with a shape; moves, never copies.
template <typename T>
class DeviceArray {
public:
    DeviceArray() = default;
    explicit DeviceArray(std::vector<uint64_t> shape) : shape_(std::move(shape)) {
        cuda_check(cudaMalloc(&ptr_, bytes() ? bytes() : 1), "cudaMalloc");
    }
    static DeviceArray from_slice(const std::vector<T>& host, std::vector<uint64_t> shape) {
        DeviceArray a(std::move(shape));
        if (a.len() != host.size()) throw Error(QB200_ERR_LENGTH, "length mismatch: expected " + std::to_string(a.len()) + ", got " + std::to_string(host.size()));
        cuda_check(cudaMemcpy(a.ptr_, host.data(), a.bytes(), cudaMemcpyHostToDevice), "cudaMemcpy");
        return a;
    }
    DeviceArray(DeviceArray&& o) noexcept : ptr_(o.ptr_), shape_(std::move(o.shape_)) { o.ptr_ = nullptr; }
    DeviceArray& operator=(DeviceArray&& o) noexcept {
        if (this != &o) {
            reset();
            ptr_ = o.ptr_;
            shape_ = std::move(o.shape_);
            o.ptr_ = nullptr;
        }
        return *this;
    }
    DeviceArray(const DeviceArray&) = delete;
    DeviceArray& operator=(const DeviceArray&) = delete;
    ~DeviceArray() { reset(); }
    std::vector<T> to_vec() const {
        std::vector<T> h(len());
        cuda_check(cudaMemcpy(h.data(), ptr_, bytes(), cudaMemcpyDeviceToHost), "cudaMemcpy");
        return h;
    }
    T* data() const { return static_cast<T*>(ptr_); }
    const std::vector<uint64_t>& shape() const { return shape_; }
    uint64_t len() const {
        uint64_t n = 1;
        for (uint64_t d : shape_) n *= d;
        return n;
    }
    uint64_t bytes() const { return len() * sizeof(T); }

private:
    void reset() {
        if (ptr_) cudaFree(ptr_);
        ptr_ = nullptr;
    }
    void* ptr_ = nullptr;
    std::vector<uint64_t> shape_;
};


// quanta-array/src/quant.rs:452-637.  Codes: int8 bytes `[R, C]` or packed u32 words `[R, ceil(C/8)]`.
class QuantizedMatrix {
public:
    // QuantizedMatrix::quantize (quant.rs:480-513) — one device pass.
    static QuantizedMatrix quantize(const DeviceArray<float>& a, QuantDtype dtype, Granularity g, cudaStream_t st = nullptr) {
        if (a.shape().size() != 2 || a.len() == 0) {
            std::string sh = "[";
            for (size_t i = 0; i < a.shape().size(); i++) sh += (i ? ", " : "") + std::to_string(a.shape()[i]);
            throw Error(QB200_ERR_RANK, "quantized leaves must be rank-2 with nonzero extents, got shape " + sh +
                                            "] (reshape rank-2 views before quantizing)");
        }
        const uint64_t rows = a.shape()[0], cols = a.shape()[1];
        auto [gr, gc] = g.tile(rows, cols);
        QuantizedMatrix m(rows, cols, gr, gc, dtype, g);
        m.scales_ = DeviceArray<float>({(rows + gr - 1) / gr, (cols + gc - 1) / gc});
        m.alloc_codes();
        check(qb200_quantize(a.data(), QB200_F32, rows, cols, bits(dtype), gr, gc, m.codes_ptr(), m.scales_.data(), st));
        return m;
    }
    // QuantizedMatrix::from_parts (quant.rs:521-568): total validation of already-resident parts.
    static QuantizedMatrix from_parts(DeviceArray<int8_t> codes, uint64_t rows, uint64_t cols, DeviceArray<float> scales, Granularity g) {
        const std::vector<uint64_t> cshape = codes.shape();  // read before the move below
        return assemble(QuantDtype::Int8, cshape, rows, cols, std::move(scales), g, std::move(codes), {});
    }
    static QuantizedMatrix from_parts(DeviceArray<uint32_t> words, uint64_t rows, uint64_t cols, DeviceArray<float> scales, Granularity g) {
        const std::vector<uint64_t> cshape = words.shape();
        return assemble(QuantDtype::Int4, cshape, rows, cols, std::move(scales), g, {}, std::move(words));
    }
    // QuantizedMatrix::dequantize (quant.rs:605-637): bit-exact s * f32(q).
    DeviceArray<float> dequantize(cudaStream_t st = nullptr) const {
        DeviceArray<float> out({rows_, cols_});
        check(qb200_dequantize(codes_ptr(), scales_.data(), rows_, cols_, bits(dtype_), gr_, gc_, out.data(), st));
        return out;
    }
    std::pair<uint64_t, uint64_t> shape() const { return {rows_, cols_}; }
    QuantDtype dtype() const { return dtype_; }
    Granularity granularity() const { return gran_; }
    std::pair<uint64_t, uint64_t> tile() const { return {gr_, gc_}; }
    const DeviceArray<int8_t>& codes_i8() const { return c8_; }
    const DeviceArray<uint32_t>& codes_u32() const { return c4_; }
    const DeviceArray<float>& scales() const { return scales_; }
    void* codes_ptr() const { return dtype_ == QuantDtype::Int8 ? static_cast<void*>(c8_.data()) : static_cast<void*>(c4_.data()); }

private:
    QuantizedMatrix(uint64_t r, uint64_t c, uint64_t gr, uint64_t gc, QuantDtype d, Granularity g)
        : rows_(r), cols_(c), gr_(gr), gc_(gc), dtype_(d), gran_(g) {}
    void alloc_codes() {
        if (dtype_ == QuantDtype::Int8) c8_ = DeviceArray<int8_t>({rows_, cols_});
        else c4_ = DeviceArray<uint32_t>({rows_, (cols_ + 7) / 8});
    }
    static QuantizedMatrix assemble(QuantDtype d, const std::vector<uint64_t>& cshape, uint64_t rows, uint64_t cols,
                                    DeviceArray<float> scales, Granularity g, DeviceArray<int8_t> c8, DeviceArray<uint32_t> c4) {
        uint64_t tmp = 0;
        if (rows == 0 || cols == 0) check(qb200_codes_bytes(rows, cols, bits(d), &tmp));
        auto [gr, gc] = g.tile(rows, cols);
        const uint64_t cr = cshape.size() == 2 ? cshape[0] : 0, cc = cshape.size() == 2 ? cshape[1] : 0;
        const auto& ss = scales.shape();
        check(qb200_check_parts(cr, cc, ss.size() == 2 ? ss[0] : 0, ss.size() == 2 ? ss[1] : 0, rows, cols, bits(d), gr, gc));
        QuantizedMatrix m(rows, cols, gr, gc, d, g);
        m.c8_ = std::move(c8);
        m.c4_ = std::move(c4);
        m.scales_ = std::move(scales);
        return m;
    }
    uint64_t rows_, cols_, gr_, gc_;
    QuantDtype dtype_;
    Granularity gran_;
    DeviceArray<int8_t> c8_;
    DeviceArray<uint32_t> c4_;
    DeviceArray<float> scales_;
};

// quanta-nn/src/quant.rs:830-919 — a frozen quantized dense layer; Mode B (resident codes).
class QuantizedLinear {
public:
    // QuantizedLinear::new (quant.rs:853-862).  layout: QB200_IN_OUT (`[in, out]`, the reference's
    // Linear) or QB200_OUT_IN (`[out, in]`).
    static QuantizedLinear new_(QuantizedMatrix w, DeviceArray<float> bias = {}, int32_t layout = QB200_IN_OUT) {
        QuantizedLinear q;
        q.w_ = std::make_unique<QuantizedMatrix>(std::move(w));
        q.b_ = std::move(bias);
        auto [rows, cols] = q.w_->shape();
        auto [gr, gc] = q.w_->tile();
        const bool has_b = q.b_.data() != nullptr;
        check(qb200_qlinear_create(q.w_->codes_ptr(), q.w_->scales().data(), rows, cols, bits(q.w_->dtype()), gr, gc, layout,
                                   has_b ? q.b_.data() : nullptr, has_b ? q.b_.len() : 0, &q.h_));
        return q;
    }
    QuantizedLinear(QuantizedLinear&& o) noexcept : w_(std::move(o.w_)), b_(std::move(o.b_)), h_(o.h_) { o.h_ = nullptr; }
    QuantizedLinear(const QuantizedLinear&) = delete;
    ~QuantizedLinear() {
        if (h_) qb200_qlinear_destroy(h_);
    }
    uint64_t in_dim() const { return qb200_qlinear_in_dim(h_); }
    uint64_t out_dim() const { return qb200_qlinear_out_dim(h_); }
    // Layer::apply without the tape (quant.rs:903-918): y = x @ deq(w) (+ b), f32 in / f32 out.
    DeviceArray<float> forward(const DeviceArray<float>& x, cudaStream_t st = nullptr) const {
        if (x.shape().size() != 2 || x.shape()[1] != in_dim())
            throw Error(QB200_ERR_INVALID_PARAM, "QuantizedLinear: input must be [m, " + std::to_string(in_dim()) + "]");
        DeviceArray<float> y({x.shape()[0], out_dim()});
        check(qb200_qlinear_forward(h_, x.data(), QB200_F32, x.shape()[0], y.data(), QB200_F32, st));
        return y;
    }
    // bf16 activations (bit patterns) in, f32 out — the decode / prefill fast paths.
    DeviceArray<float> forward_bf16(const DeviceArray<uint16_t>& x, cudaStream_t st = nullptr) const {
        DeviceArray<float> y({x.shape()[0], out_dim()});
        check(qb200_qlinear_forward(h_, x.data(), QB200_BF16, x.shape()[0], y.data(), QB200_F32, st));
        return y;
    }
    // [layers[i].forward_bf16(*xs[i])...] in one call: layers that share the input width and take the decode path
    // run as ONE persistent launch (fused Q/K/V or gate + up projections; qb200_qlinear_forward_many).
    static std::vector<DeviceArray<float>> forward_many_bf16(const std::vector<const QuantizedLinear*>& layers,
                                                             const std::vector<const DeviceArray<uint16_t>*>& xs,
                                                             cudaStream_t st = nullptr) {
        if (layers.size() != xs.size() || layers.empty()) throw Error(QB200_ERR_INVALID_PARAM, "forward_many: one input per layer");
        const uint64_t m = xs[0]->shape()[0];
        std::vector<DeviceArray<float>> ys;
        std::vector<qb200_qlinear*> hs;
        std::vector<const void*> xp;
        std::vector<void*> yp;
        for (size_t i = 0; i < layers.size(); i++) {
            ys.emplace_back(std::vector<uint64_t>{m, layers[i]->out_dim()});
            hs.push_back(layers[i]->h_);
            xp.push_back(xs[i]->data());
            yp.push_back(ys.back().data());
        }
        check(qb200_qlinear_forward_many(hs.data(), (uint32_t)hs.size(), xp.data(), QB200_BF16, m, yp.data(), QB200_F32, st));
        return ys;
    }
    const char* last_kernel() const { return qb200_qlinear_last_kernel(h_); }
    const QuantizedMatrix& weight() const { return *w_; }

private:
    QuantizedLinear() = default;
    std::unique_ptr<QuantizedMatrix> w_;
    DeviceArray<float> b_;
    qb200_qlinear* h_ = nullptr;
};

// The decode step's support ops (thin wrappers; semantics and reference anchors are in qb200.h).
// h += delta (when given), returns bf16(rmsnorm(h) * gamma) — quanta-nn/src/norm.rs:192-225.
inline DeviceArray<uint16_t> add_rmsnorm(DeviceArray<float>& h, const DeviceArray<float>* delta, const DeviceArray<float>& gamma,
                                         float eps, cudaStream_t st = nullptr) {
    DeviceArray<uint16_t> out({h.shape()[0], h.shape()[1]});
    check(qb200_add_rmsnorm(h.data(), delta ? delta->data() : nullptr, delta ? 1u : 0u, gamma.data(), h.shape()[0], h.shape()[1], eps,
                            out.data(), st));
    return out;
}
// silu(gate) * up as bf16 — quanta-nn/src/activation.rs:145-162.
inline DeviceArray<uint16_t> swiglu(const DeviceArray<float>& gate, const DeviceArray<float>& up, cudaStream_t st = nullptr) {
    const uint64_t n = gate.shape()[0], h = gate.shape()[1];
    DeviceArray<uint16_t> out({n, h});
    const uint32_t width = (uint32_t)h;
    check(qb200_swiglu_sliced(gate.data(), up.data(), n, h, &width, 1, 0, out.data(), st));
    return out;
}

// quanta-blas's quantized entries (crates/sci/quanta-blas/src/mixed_quant.rs:22-147): integer codes for both operands,
// per-tensor symmetric scales, C f32 read for beta * C and overwritten.  Asynchronous on `st`.
enum class GemmQuantType { Q8Symmetric = QB200_Q8_SYMMETRIC, Q4Symmetric = QB200_Q4_SYMMETRIC };
inline void gemm_quant(GemmQuantType qty, uint32_t m, uint32_t n, uint32_t k, float alpha, float a_scale, float b_scale,
                       const DeviceArray<int32_t>& a, const DeviceArray<int32_t>& b, float beta, DeviceArray<float>& c,
                       cudaStream_t st = nullptr) {
    if (a.len() != (uint64_t)m * k || b.len() != (uint64_t)k * n || c.len() != (uint64_t)m * n)
        throw Error(QB200_ERR_LENGTH, "gemm_quant: A must be m x k, B k x n, C m x n");
    check(qb200_gemm_quant((int)qty, m, n, k, alpha, a_scale, b_scale, a.data(), b.data(), beta, c.data(), st));
}
inline void gemm_quant4(GemmQuantType qty, uint32_t m, uint32_t n, uint32_t k, float alpha, float a_scale, float b_scale,
                        const DeviceArray<uint32_t>& a, const DeviceArray<uint32_t>& b, float beta, DeviceArray<float>& c,
                        cudaStream_t st = nullptr) {
    if (a.len() != ((uint64_t)m * k + 7) / 8 || b.len() != ((uint64_t)k * n + 7) / 8 || c.len() != (uint64_t)m * n)
        throw Error(QB200_ERR_LENGTH, "gemm_quant4: A must be ceil(m k / 8) words, B ceil(k n / 8), C m x n");
    check(qb200_gemm_quant4((int)qty, m, n, k, alpha, a_scale, b_scale, a.data(), b.data(), beta, c.data(), st));
}
inline void gemv_quant(GemmQuantType qty, uint32_t m, uint32_t n, float alpha, float a_scale, float x_scale,
                       const DeviceArray<int32_t>& a, const DeviceArray<int32_t>& x, float beta, DeviceArray<float>& y,
                       cudaStream_t st = nullptr) {
    gemm_quant(qty, m, 1, n, alpha, a_scale, x_scale, a, x, beta, y, st);
}
inline void gemv_quant4(GemmQuantType qty, uint32_t m, uint32_t n, float alpha, float a_scale, float x_scale,
                        const DeviceArray<uint32_t>& a, const DeviceArray<uint32_t>& x, float beta, DeviceArray<float>& y,
                        cudaStream_t st = nullptr) {
    gemm_quant4(qty, m, 1, n, alpha, a_scale, x_scale, a, x, beta, y, st);
}
// Waits for the stream; throws for an int8 code out of range or a device wait that ran out.
inline void gemm_quant_check(cudaStream_t st = nullptr) { check(qb200_gemm_quant_check(st)); }

// quanta-nn/src/quant.rs:152-155: a named checkpoint leaf on the host side of save / load.
struct QuantLeaf {
    bool quantized = false;
    std::vector<uint64_t> shape;   // plain: tensor shape; quantized: [rows, cols]
    std::vector<float> f32;        // plain values
    uint32_t bits = 0;             // quantized: 8 / 4
    uint64_t gr = 0, gc = 0;
    std::vector<uint8_t> codes;    // quantized: code bytes as stored (int8, or little-endian u32 words)
    std::vector<float> scales;
    static QuantLeaf F32(const DeviceArray<float>& a) {
        QuantLeaf l;
        l.shape = a.shape();
        l.f32 = a.to_vec();
        return l;
    }
    static QuantLeaf Quantized(const QuantizedMatrix& m) {
        QuantLeaf l;
        l.quantized = true;
        l.shape = {m.shape().first, m.shape().second};
        l.bits = static_cast<uint32_t>(m.dtype());
        l.gr = m.tile().first;
        l.gc = m.tile().second;
        uint64_t nbytes = 0;
        check(qb200_codes_bytes(l.shape[0], l.shape[1], l.bits, &nbytes));
        l.codes.resize(nbytes);
        cuda_check(cudaMemcpy(l.codes.data(), m.codes_ptr(), nbytes, cudaMemcpyDeviceToHost), "cudaMemcpy");
        l.scales = m.scales().to_vec();
        return l;
    }
};

// save_named (quant.rs:279-390): leaves in the given order, metadata keys sorted -> file bytes.
inline std::vector<uint8_t> save_named(const std::vector<std::pair<std::string, QuantLeaf>>& entries,
                                       const std::map<std::string, std::string>* metadata = nullptr) {
    qb200_st_writer* w = nullptr;
    check(qb200_st_writer_create(&w));
    std::unique_ptr<qb200_st_writer, void (*)(qb200_st_writer*)> guard(w, qb200_st_writer_free);
    if (metadata) {
        check(qb200_st_writer_set_has_metadata(w, 1));
        for (auto& kv : *metadata) check(qb200_st_writer_add_metadata(w, kv.first.c_str(), kv.second.c_str()));
    }
    for (auto& e : entries) {
        const QuantLeaf& l = e.second;
        if (l.quantized)
            check(qb200_st_writer_add_quantized(w, e.first.c_str(), l.bits, l.shape[0], l.shape[1], l.gr, l.gc, l.codes.data(), l.scales.data()));
        else
            check(qb200_st_writer_add_f32(w, e.first.c_str(), l.shape.data(), (uint32_t)l.shape.size(), l.f32.data()));
    }
    const uint8_t* bytes = nullptr;
    uint64_t len = 0;
    check(qb200_st_writer_finish(w, &bytes, &len));
    return std::vector<uint8_t>(bytes, bytes + len);
}

struct LoadedQuant {
    std::vector<std::pair<std::string, QuantLeaf>> leaves;
    std::map<std::string, std::string> metadata;
};

// load_named (quant.rs:676-729) up to the upload: total validation, then leaves in header order
// (host copies; QuantizedMatrix::from_parts uploads them).
inline LoadedQuant load_named(const std::vector<uint8_t>& data, bool allow_block = false) {
    qb200_st_file* f = nullptr;
    check(qb200_st_validate(data.data(), data.size(), allow_block ? 1 : 0, &f));
    std::unique_ptr<qb200_st_file, void (*)(qb200_st_file*)> guard(f, qb200_st_free);
    LoadedQuant out;
    for (uint64_t i = 0; i < qb200_st_num_items(f); i++) {
        qb200_st_item it;
        check(qb200_st_item_at(f, i, &it));
        QuantLeaf l;
        l.shape.assign(it.shape, it.shape + it.ndim);
        if (it.quantized) {
            l.quantized = true;
            l.bits = it.bits;
            l.gr = it.gr;
            l.gc = it.gc;
            l.codes.assign(data.begin() + it.data_offset, data.begin() + it.data_offset + it.data_len);
            l.scales.resize(it.scales_len / 4);
            std::copy(data.begin() + it.scales_offset, data.begin() + it.scales_offset + it.scales_len,
                      reinterpret_cast<uint8_t*>(l.scales.data()));
        } else {
            uint64_t n = 1;
            for (uint64_t d : l.shape) n *= d;
            if (n < 1) n = 1;
            l.f32.resize(n);
            check(qb200_st_plain_to_f32(f, i, l.f32.data(), n));
        }
        out.leaves.emplace_back(it.name, std::move(l));
    }
    for (uint64_t i = 0; i < qb200_st_num_metadata(f); i++) {
        const char *k = nullptr, *v = nullptr;
        check(qb200_st_metadata_at(f, i, &k, &v));
        out.metadata[k] = v;
    }
    return out;
}

}  // namespace qb200
