// Parity tests written against the C++ mirror (include/qb200.hpp), in the shape of the reference's
// own suites: crates/sci/quanta-array/tests/quant.rs and crates/ml/quanta-nn/tests/quant.rs.
// Expected values are the reference's source literals.  Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <cstring>

#include "qb200.hpp"

using namespace qb200;

static int failures = 0;
#define EXPECT(cond)                                                      \
    do {                                                                  \
        if (!(cond)) {                                                    \
            std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            failures++;                                                   \
        }                                                                 \
    } while (0)

static bool bits_eq(const std::vector<float>& a, const std::vector<float>& b) {
    return a.size() == b.size() && std::memcmp(a.data(), b.data(), a.size() * 4) == 0;
}

// quanta-array/tests/quant.rs:34-41
static std::vector<float> weights(size_t n) {
    std::vector<float> w(n);
    for (size_t i = 0; i < n; i++) {
        float x = (float)i * 0.7311f - (float)n * 0.317f;
        w[i] = (i % 3 == 0) ? -x * 0.13f : x * 0.171f;
    }
    return w;
}

int main() {
    // dequant_ties_to_even_pinned_int8 / int4 (tests/quant.rs:177-205)
    {
        auto a = DeviceArray<float>::from_slice({63.5f, -63.5f, 0.25f, 0.26f, 0.75f, -0.75f, 1.0f, 0.0f}, {2, 4});
        auto qm = QuantizedMatrix::quantize(a, QuantDtype::Int8, Granularity::PerTensor());
        EXPECT(qm.scales().to_vec() == std::vector<float>{0.5f});
        EXPECT(bits_eq(qm.dequantize().to_vec(), {63.5f, -63.5f, 0.0f, 0.5f, 1.0f, -1.0f, 1.0f, 0.0f}));
        auto b = DeviceArray<float>::from_slice({3.5f, -3.5f, 0.25f, 0.26f, 0.75f, -0.75f, 1.0f, 0.0f}, {2, 4});
        auto q4 = QuantizedMatrix::quantize(b, QuantDtype::Int4, Granularity::PerTensor());
        EXPECT(q4.scales().to_vec() == std::vector<float>{0.5f});
        EXPECT(bits_eq(q4.dequantize().to_vec(), {3.5f, -3.5f, 0.0f, 0.5f, 1.0f, -1.0f, 1.0f, 0.0f}));
    }
    // int4_nibble_order_low_first_pinned / rows pack independently (tests/quant.rs:216-243)
    {
        auto a = DeviceArray<float>::from_slice({1, 2, -1, -7, 7, 0, 3, -3}, {1, 8});
        auto qm = QuantizedMatrix::quantize(a, QuantDtype::Int4, Granularity::PerTensor());
        EXPECT(qm.codes_u32().to_vec() == std::vector<uint32_t>{0xD3079F21u});
        auto b = DeviceArray<float>::from_slice({1, -1, 2, 3, -2, 7}, {2, 3});
        auto q2 = QuantizedMatrix::quantize(b, QuantDtype::Int4, Granularity::PerTensor());
        EXPECT((q2.codes_u32().to_vec() == std::vector<uint32_t>{0x2F1u, 0x7E3u}));
        EXPECT(bits_eq(q2.dequantize().to_vec(), {1, -1, 2, 3, -2, 7}));
    }
    // from_parts (tests/quant.rs:247-282) and its loud errors (:397-435)
    {
        auto qm = QuantizedMatrix::from_parts(DeviceArray<int8_t>::from_slice({2, -2, 4, -4}, {2, 2}), 2, 2,
                                              DeviceArray<float>::from_slice({0.5f, 0.25f}, {2, 1}), Granularity::PerChannel(0));
        EXPECT((qm.dequantize().to_vec() == std::vector<float>{1, -1, 1, -1}));
        auto q4 = QuantizedMatrix::from_parts(DeviceArray<uint32_t>::from_slice({0xF1u, 0xE2u}, {2, 1}), 2, 2,
                                              DeviceArray<float>::from_slice({0.5f, 0.25f}, {2, 1}), Granularity::PerChannel(0));
        EXPECT((q4.dequantize().to_vec() == std::vector<float>{0.5f, -0.5f, 0.5f, -0.5f}));
        try {
            QuantizedMatrix::from_parts(DeviceArray<int8_t>::from_slice({1, 2, 3, 4}, {2, 2}), 4, 2,
                                        DeviceArray<float>::from_slice({1.0f}, {1, 1}), Granularity::PerTensor());
            EXPECT(false);
        } catch (const Error& e) {
            EXPECT(std::string(e.kind()) == "Grid" && std::string(e.what()).find("[4, 2]") != std::string::npos);
        }
        try {
            Granularity::Group(1, 99).tile(4, 4);
            EXPECT(false);
        } catch (const Error& e) {
            EXPECT(std::string(e.kind()) == "Granularity" && std::string(e.what()).find("99") != std::string::npos);
        }
    }
    // record accessors (tests/quant.rs:322-338)
    {
        auto a = DeviceArray<float>::from_slice(weights(35), {5, 7});
        auto qm = QuantizedMatrix::quantize(a, QuantDtype::Int4, Granularity::Group(0, 3));
        EXPECT((qm.shape() == std::pair<uint64_t, uint64_t>{5, 7}) && qm.dtype() == QuantDtype::Int4);
        EXPECT((qm.tile() == std::pair<uint64_t, uint64_t>{3, 1}) && qm.granularity() == Granularity::Group(0, 3));
        EXPECT((qm.scales().shape() == std::vector<uint64_t>{2, 7}) && (qm.codes_u32().shape() == std::vector<uint64_t>{5, 1}));
    }
    // save matches the reference bytes (quanta-nn/tests/quant.rs:80-140), load round trip (:175-237)
    {
        auto b = DeviceArray<float>::from_slice({0.5f, -1.5f}, {2});
        auto w = DeviceArray<float>::from_slice({1, -2, 3, -4, 5, -6, 7, 127}, {2, 4});
        auto v = DeviceArray<float>::from_slice({7, -2, 3, -4}, {1, 4});
        auto qw = QuantizedMatrix::quantize(w, QuantDtype::Int8, Granularity::PerTensor());
        auto qv = QuantizedMatrix::quantize(v, QuantDtype::Int4, Granularity::PerTensor());
        auto bytes = save_named({{"b", QuantLeaf::F32(b)}, {"w", QuantLeaf::Quantized(qw)}, {"v", QuantLeaf::Quantized(qv)}});
        const std::string header =
            "{\"__metadata__\":{\"quant:v\":\"q4s;gr=1;gc=4;rows=1;cols=4\",\"quant:w\":\"q8s;gr=2;gc=4;rows=2;cols=4\","
            "\"quanta.quant\":\"1\"},\"b\":{\"dtype\":\"F32\",\"shape\":[2],\"data_offsets\":[0,8]},"
            "\"w.q\":{\"dtype\":\"I8\",\"shape\":[2,4],\"data_offsets\":[8,16]},\"w.qs\":{\"dtype\":\"F32\",\"shape\":[1,1],\"data_offsets\":[16,20]},"
            "\"v.q\":{\"dtype\":\"U32\",\"shape\":[1,1],\"data_offsets\":[20,24]},\"v.qs\":{\"dtype\":\"F32\",\"shape\":[1,1],\"data_offsets\":[24,28]}}";
        std::string padded = header;
        while ((padded.size() + 8) % 8) padded += ' ';
        EXPECT(bytes.size() == 8 + padded.size() + 28 && std::memcmp(bytes.data() + 8, padded.data(), padded.size()) == 0);
        const uint8_t want_codes[8] = {0x01, 0xFE, 0x03, 0xFC, 0x05, 0xFA, 0x07, 0x7F};
        EXPECT(std::memcmp(bytes.data() + 8 + padded.size() + 8, want_codes, 8) == 0);
        auto loaded = load_named(bytes);
        EXPECT(loaded.leaves.size() == 3 && loaded.leaves[1].first == "w" && loaded.leaves[2].second.bits == 4);
        EXPECT(save_named(loaded.leaves) == bytes);
        bytes[bytes.size() - 1] = 0x7F;  // scale of v becomes non-finite? (0x7F80.. needs two bytes) -> corrupt the exponent
        bytes[bytes.size() - 2] = 0x80;
        try {
            load_named(bytes);
            EXPECT(false);
        } catch (const Error& e) {
            EXPECT(std::string(e.kind()) == "Scale" && std::string(e.what()).find("non-finite") != std::string::npos);
        }
    }
    // QuantizedLinear == Linear(dequantized w) (quanta-nn/tests/quant.rs:467-524), both orientations
    for (int layout : {QB200_IN_OUT, QB200_OUT_IN}) {
        const uint64_t r = 64, c = 40, m = 3;
        auto wv = weights(r * c);
        for (auto& x : wv) x *= 0.01f;
        auto qm = QuantizedMatrix::quantize(DeviceArray<float>::from_slice(wv, {r, c}), QuantDtype::Int4, Granularity::Group(0, 8));
        auto wd = qm.dequantize().to_vec();
        const uint64_t in = layout == QB200_IN_OUT ? r : c, out = layout == QB200_IN_OUT ? c : r;
        std::vector<float> bias(out), xh(m * in);
        for (size_t i = 0; i < bias.size(); i++) bias[i] = 0.01f * (float)i;
        for (size_t i = 0; i < xh.size(); i++) xh[i] = std::sin((float)i);
        auto ql = QuantizedLinear::new_(std::move(qm), DeviceArray<float>::from_slice(bias, {out}), layout);
        EXPECT(ql.in_dim() == in && ql.out_dim() == out);
        auto y = ql.forward(DeviceArray<float>::from_slice(xh, {m, in})).to_vec();
        for (uint64_t i = 0; i < m; i++)
            for (uint64_t j = 0; j < out; j++) {
                float acc = 0.0f;
                for (uint64_t k = 0; k < in; k++) acc = acc + xh[i * in + k] * (layout == QB200_IN_OUT ? wd[k * c + j] : wd[j * c + k]);
                acc += bias[j];
                EXPECT(std::fabs(y[i * out + j] - acc) <= 1e-4f * (1.0f + std::fabs(acc)));
            }
        try {
            auto q2 = QuantizedMatrix::quantize(DeviceArray<float>::from_slice(wv, {r, c}), QuantDtype::Int8, Granularity::PerTensor());
            QuantizedLinear::new_(std::move(q2), DeviceArray<float>::from_slice({0, 0, 0}, {3}), layout);
            EXPECT(false);
        } catch (const Error& e) {
            EXPECT(std::string(e.what()).find("bias") != std::string::npos);
        }
    }
    // grouped decode launch == one forward per layer, bit for bit (the reference stacks layers and loops over
    // Layer::apply, quanta-nn/tests/quant.rs:507-523); then the decode step's elementwise ops
    {
        const uint64_t n_out = 96, k = 256, m = 2;
        std::vector<QuantizedLinear> layers;
        for (int l = 0; l < 3; l++) {
            auto wv = weights(n_out * k);
            for (auto& x : wv) x *= 0.001f * (float)(l + 1);
            layers.push_back(QuantizedLinear::new_(
                QuantizedMatrix::quantize(DeviceArray<float>::from_slice(wv, {n_out, k}), QuantDtype::Int4, Granularity::Group(1, 128)), {},
                QB200_OUT_IN));
        }
        std::vector<uint16_t> xb(m * k);
        for (size_t i = 0; i < xb.size(); i++) {
            float v = std::sin((float)i);
            uint32_t bits;
            std::memcpy(&bits, &v, 4);
            xb[i] = (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);  // dtype.rs:14-21
        }
        auto x = DeviceArray<uint16_t>::from_slice(xb, {m, k});
        auto ys = QuantizedLinear::forward_many_bf16({&layers[0], &layers[1], &layers[2]}, {&x, &x, &x});
        EXPECT(std::string(layers[0].last_kernel()) == "gemv_mma_grouped");
        for (int l = 0; l < 3; l++) EXPECT(bits_eq(ys[l].to_vec(), layers[l].forward_bf16(x).to_vec()));

        std::vector<float> hv(2 * 64), dv(2 * 64), gv(64, 1.5f);
        for (size_t i = 0; i < hv.size(); i++) hv[i] = std::cos((float)i), dv[i] = 0.25f * (float)(i % 7);
        auto h = DeviceArray<float>::from_slice(hv, {2, 64});
        auto d = DeviceArray<float>::from_slice(dv, {2, 64});
        auto normed = add_rmsnorm(h, &d, DeviceArray<float>::from_slice(gv, {64}), 1e-5f).to_vec();
        auto hs = h.to_vec();
        for (int r = 0; r < 2; r++) {
            float sq = 0.0f;
            for (int c = 0; c < 64; c++) {
                EXPECT(hs[r * 64 + c] == hv[r * 64 + c] + dv[r * 64 + c]);
                sq = sq + hs[r * 64 + c] * hs[r * 64 + c];
            }
            const float rrms = 1.0f / std::sqrt(sq / 64.0f + 1e-5f);  // norm.rs:192-212
            for (int c = 0; c < 64; c++) {
                uint32_t b = (uint32_t)normed[r * 64 + c] << 16;
                float got;
                std::memcpy(&got, &b, 4);
                const float want = hs[r * 64 + c] * rrms * 1.5f;
                EXPECT(std::fabs(got - want) <= 1e-2f * (1.0f + std::fabs(want)));
            }
        }
        {
            // quanta-blas/tests/gemm_quant.rs: the q8 "larger" and q4 "rectangular" cases against a plain f32 loop
            // (reference.rs:104-131: codes cast to f32, left-to-right f32 sums, alpha_eff * acc + beta * c)
            auto code = [](uint32_t i, uint32_t seed, uint32_t span) { return (int32_t)(((i * 2654435761u) ^ seed) % span) - (int32_t)(span / 2); };
            const uint32_t m = 32, n = 24, k = 40;
            std::vector<int32_t> a(m * k), b(k * n);
            std::vector<float> c0(m * n);
            for (uint32_t i = 0; i < m * k; i++) a[i] = code(i, 1, 64);
            for (uint32_t i = 0; i < k * n; i++) b[i] = code(i, 2, 64);
            for (uint32_t i = 0; i < m * n; i++) c0[i] = (float)i * 0.25f - 1.0f;
            auto c = DeviceArray<float>::from_slice(c0, {m, n});
            gemm_quant(GemmQuantType::Q8Symmetric, m, n, k, 1.0f, 0.02f, 0.03f, DeviceArray<int32_t>::from_slice(a, {m, k}),
                       DeviceArray<int32_t>::from_slice(b, {k, n}), 0.5f, c);
            gemm_quant_check();
            auto got = c.to_vec();
            const float ae = 1.0f * 0.02f * 0.03f;
            for (uint32_t r = 0; r < m; r++)
                for (uint32_t j = 0; j < n; j++) {
                    float acc = 0.0f;
                    for (uint32_t p = 0; p < k; p++) acc += (float)a[r * k + p] * (float)b[p * n + j];
                    const float t1 = ae * acc, t2 = 0.5f * c0[r * n + j];
                    EXPECT(got[r * n + j] == t1 + t2);
                }
            const uint32_t m4 = 3, n4 = 5, k4 = 7;  // k not a multiple of 8: rows start inside words
            std::vector<int32_t> a4(m4 * k4), b4(k4 * n4);
            for (uint32_t i = 0; i < m4 * k4; i++) a4[i] = code(i, 1, 16);
            for (uint32_t i = 0; i < k4 * n4; i++) b4[i] = code(i, 2, 16);
            auto pack = [](const std::vector<int32_t>& q) {
                std::vector<uint32_t> w((q.size() + 7) / 8, 0u);
                for (size_t i = 0; i < q.size(); i++) w[i / 8] |= ((uint32_t)q[i] & 0xFu) << (4 * (i % 8));
                return w;
            };
            auto aw = pack(a4), bw = pack(b4);
            DeviceArray<float> c4({m4, n4});
            cuda_check(cudaMemset(c4.data(), 0, c4.bytes()), "cudaMemset");
            gemm_quant4(GemmQuantType::Q4Symmetric, m4, n4, k4, 1.0f, 0.2f, 0.05f, DeviceArray<uint32_t>::from_slice(aw, {aw.size()}),
                        DeviceArray<uint32_t>::from_slice(bw, {bw.size()}), 0.0f, c4);
            gemm_quant_check();
            auto got4 = c4.to_vec();
            for (uint32_t r = 0; r < m4; r++)
                for (uint32_t j = 0; j < n4; j++) {
                    float acc = 0.0f;
                    for (uint32_t p = 0; p < k4; p++) acc += (float)a4[r * k4 + p] * (float)b4[p * n4 + j];
                    EXPECT(got4[r * n4 + j] == (1.0f * 0.2f * 0.05f) * acc);
                }
            {
                // the reference's own literal cases (crates/sci/quanta-blas/src/reference.rs:1119-1148)
                auto c8 = DeviceArray<float>::from_slice({0.0f, 0.0f, 0.0f, 0.0f}, {2, 2});
                gemm_quant(GemmQuantType::Q8Symmetric, 2, 2, 2, 1.0f, 0.5f, 0.25f, DeviceArray<int32_t>::from_slice({2, 4, 6, 8}, {2, 2}),
                           DeviceArray<int32_t>::from_slice({1, 0, 0, 1}, {2, 2}), 0.0f, c8);
                gemm_quant_check();
                EXPECT((c8.to_vec() == std::vector<float>{0.25f, 0.5f, 0.75f, 1.0f}));
                auto c4b = DeviceArray<float>::from_slice({0.0f, 0.0f, 0.0f, 0.0f}, {2, 2});
                auto wa = pack({1, 2, 3, -1}), wb = pack({1, 0, 0, 1});
                gemm_quant4(GemmQuantType::Q4Symmetric, 2, 2, 2, 1.0f, 1.0f, 2.0f, DeviceArray<uint32_t>::from_slice(wa, {wa.size()}),
                            DeviceArray<uint32_t>::from_slice(wb, {wb.size()}), 0.0f, c4b);
                gemm_quant_check();
                EXPECT((c4b.to_vec() == std::vector<float>{2.0f, 4.0f, 6.0f, -2.0f}));
            }
            bool threw = false;  // gemm_quant.rs:215-238: Q4 through the Q8 entry must error
            try {
                gemm_quant(GemmQuantType::Q4Symmetric, m, n, k, 1.0f, 0.1f, 0.1f, DeviceArray<int32_t>::from_slice(a, {m, k}),
                           DeviceArray<int32_t>::from_slice(b, {k, n}), 0.0f, c);
            } catch (const Error&) { threw = true; }
            EXPECT(threw);
        }
        auto act = swiglu(DeviceArray<float>::from_slice({-40.0f, -1.0f, 0.0f, 2.0f}, {1, 4}), DeviceArray<float>::from_slice({1, 1, 1, 1}, {1, 4})).to_vec();
        const float av[4] = {-40.0f, -1.0f, 0.0f, 2.0f};
        for (int i = 0; i < 4; i++) {
            uint32_t b = (uint32_t)act[i] << 16;
            float got;
            std::memcpy(&got, &b, 4);
            const float want = av[i] * (1.0f / (1.0f + std::exp(std::fmin(-av[i], 30.0f))));  // activation.rs:145-162
            EXPECT(std::fabs(got - want) <= 1e-2f * (1.0f + std::fabs(want)));
        }
    }
    std::printf(failures ? "%d FAILED\n" : "all C++ mirror tests passed\n", failures);
    return failures ? 1 : 0;
}
