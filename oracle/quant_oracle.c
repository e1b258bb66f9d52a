/*
 * CPU oracle for the quantized-inference path of zelez-lab/quanta.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's host algorithm.  It is the checker the CUDA kernels are compared
 * against and the timed CPU baseline of the benchmark; the product library
 * never links, loads or calls it.
 *
 * Parity status: PINNED.  tests/test_oracle_golden.py checks every function
 * below against the literals the reference's own test-suites hold for this
 * path (crates/gpu/quanta-ir/src/dtype.rs:407-451,
 * crates/gpu/quanta-ir/src/op_matrix_cases.rs:1680-1742,
 * crates/sci/quanta-array/tests/quant.rs, crates/ml/quanta-nn/tests/quant.rs).
 * The reference itself is Rust and no Rust toolchain exists in the build
 * image, so the reference could not be executed; the pins are its source
 * literals.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (IEEE f32, no FMA
 * contraction: the reference's host loops use a separate multiply and add).
 *
 * Rust semantics restated where C differs:
 *   f32::max(a, b)        NaN operand is ignored           -> qo_max_f32
 *   f32 as i32            saturates, NaN -> 0              -> qo_f32_as_i32
 *   round_ties_even       IEEE roundTiesToEven             -> rintf (default mode)
 *   i32 as i8             truncation (safe after clamp)
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define QO_OK 0
#define QO_ERR_RANK 1        /* QuantError::Rank          */
#define QO_ERR_GRANULARITY 2 /* QuantError::Granularity   */
#define QO_ERR_LENGTH 7      /* ArrayError::LengthMismatch */

/* ---- quanta-ir/src/dtype.rs:8-21 : bf16 conversions ------------------- */

static float qo_from_bits(uint32_t b) {
    float f;
    memcpy(&f, &b, 4);
    return f;
}
static uint32_t qo_to_bits(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
}

/* dtype.rs:9-11 — bf16 is the top 16 bits of an f32. */
float qo_bf16_to_f32(uint16_t bits) { return qo_from_bits(((uint32_t)bits) << 16); }

/* dtype.rs:14-21 — round to nearest even; NaN keeps its top half and is quieted. */
uint16_t qo_f32_to_bf16(float val) {
    uint32_t bits = qo_to_bits(val);
    if (val != val) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t bias = 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}

/* quanta-nn/src/safetensors.rs:354-373 — IEEE half to f32 (all classes). */
float qo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)(h >> 15)) << 31;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0 && man == 0) {
        bits = sign;
    } else if (exp == 0) {
        uint32_t p = 31u - (uint32_t)__builtin_clz(man);
        uint32_t exp32 = 127u + p - 24u;
        uint32_t man32 = (man << (10u - p)) & 0x3FFu;
        bits = sign | (exp32 << 23) | (man32 << 13);
    } else if (exp == 0x1F) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127u - 15u) << 23) | (man << 13);
    }
    return qo_from_bits(bits);
}

/* ---- quanta-ir/src/dtype.rs:232-268 : the quant arithmetic ------------ */

/* dtype.rs:232-235 */
void qo_quant_range(uint32_t bits, int32_t* lo, int32_t* hi) {
    int32_t h = (int32_t)((1u << (bits - 1)) - 1u);
    *lo = -(h + 1);
    *hi = h;
}

/* Rust `f32 as i32`: saturating, NaN -> 0. */
static int32_t qo_f32_as_i32(float r) {
    if (r != r) return 0;
    if (r >= 2147483648.0f) return INT32_MAX;
    if (r <= -2147483648.0f) return INT32_MIN;
    return (int32_t)r;
}

/* dtype.rs:238-242 — clamp(round_ties_even(x / scale), lo, hi). */
int32_t qo_quantize_sym(float x, float scale, uint32_t bits) {
    int32_t lo, hi;
    qo_quant_range(bits, &lo, &hi);
    int32_t r = qo_f32_as_i32(rintf(x / scale));
    return r < lo ? lo : (r > hi ? hi : r);
}

/* dtype.rs:245-247 — scale * q. */
float qo_dequantize_sym(int32_t q, float scale) { return scale * (float)q; }

/* dtype.rs:256-260 — nibble i (0..8) of a word, sign-extended. */
int32_t qo_int4_unpack(uint32_t word, uint32_t i) {
    uint32_t n = (word >> (i * 4u)) & 0xFu;
    return (int32_t)((n ^ 0x8u) - 0x8u);
}

/* dtype.rs:264-268 — read-modify-write of nibble i. */
uint32_t qo_int4_pack(uint32_t word, uint32_t i, int32_t q) {
    uint32_t shift = i * 4u;
    uint32_t n = ((uint32_t)q) & 0xFu;
    return (word & ~(0xFu << shift)) | (n << shift);
}

/* ---- quanta-array/src/quant.rs:109-144 : Granularity::tile ------------ */

/* kind: 0 PerTensor, 1 PerChannel{axis}, 2 Group{axis,size},
 *       3 Block{rows=size, cols=size2} (additive arm: the reference's
 *         arithmetic takes any (gr, gc); only its enum lacks the spelling). */
int qo_tile(int kind, uint64_t axis, uint64_t size, uint64_t size2, uint64_t rows, uint64_t cols,
            uint64_t* gr, uint64_t* gc) {
    switch (kind) {
        case 0:
            *gr = rows;
            *gc = cols;
            return QO_OK;
        case 1:
            if (axis == 0) {
                *gr = 1;
                *gc = cols;
                return QO_OK;
            }
            if (axis == 1) {
                *gr = rows;
                *gc = 1;
                return QO_OK;
            }
            return QO_ERR_GRANULARITY;
        case 2: {
            if (axis > 1) return QO_ERR_GRANULARITY;
            uint64_t extent = axis == 0 ? rows : cols;
            if (size == 0 || size > extent) return QO_ERR_GRANULARITY;
            if (axis == 0) {
                *gr = size;
                *gc = 1;
            } else {
                *gr = 1;
                *gc = size;
            }
            return QO_OK;
        }
        case 3:
            if (size == 0 || size > rows || size2 == 0 || size2 > cols) return QO_ERR_GRANULARITY;
            *gr = size;
            *gc = size2;
            return QO_OK;
        default:
            return QO_ERR_GRANULARITY;
    }
}

static uint64_t qo_div_ceil(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

/* Rust f32::max: if either operand is NaN the other is returned. */
static float qo_max_f32(float a, float b) {
    if (a != a) return b;
    if (b != b) return a;
    return a > b ? a : b;
}

/* ---- quanta-array/src/quant.rs:293-367 : quantize_host ---------------- */

/* codes: int8 -> rows*cols bytes; int4 -> rows*ceil(cols/8) u32 words.
 * scales: ceil(rows/gr)*ceil(cols/gc) f32, row-major.  wlen = element count
 * of w (the slice-length check of quant.rs:324-329). */
int qo_quantize_host(const float* w, uint64_t wlen, uint64_t rows, uint64_t cols, uint32_t bits,
                     uint64_t gr, uint64_t gc, void* codes, float* scales) {
    if (rows == 0 || cols == 0) return QO_ERR_RANK; /* check_dims, quant.rs:192-200 */
    if (wlen != rows * cols) return QO_ERR_LENGTH;
    if (gr == 0 || gc == 0 || gr > rows || gc > cols) return QO_ERR_GRANULARITY;
    int32_t lo, hi;
    qo_quant_range(bits, &lo, &hi);
    uint64_t tr = qo_div_ceil(rows, gr), tc = qo_div_ceil(cols, gc);
    /* max_abs_scales, quant.rs:293-309 */
    for (uint64_t i = 0; i < tr * tc; i++) scales[i] = 0.0f;
    for (uint64_t r = 0; r < rows; r++)
        for (uint64_t c = 0; c < cols; c++) {
            float* m = &scales[(r / gr) * tc + (c / gc)];
            *m = qo_max_f32(*m, fabsf(w[r * cols + c]));
        }
    for (uint64_t i = 0; i < tr * tc; i++) scales[i] = scales[i] / (float)hi;
    /* codes, quant.rs:336-365 */
    if (bits == 8) {
        int8_t* q = (int8_t*)codes;
        for (uint64_t r = 0; r < rows; r++)
            for (uint64_t c = 0; c < cols; c++) {
                float s = scales[(r / gr) * tc + (c / gc)];
                int32_t code = (s == 0.0f) ? 0 : qo_quantize_sym(w[r * cols + c], s, bits);
                q[r * cols + c] = (int8_t)code;
            }
    } else {
        uint32_t* words = (uint32_t*)codes;
        uint64_t wpr = qo_div_ceil(cols, 8);
        for (uint64_t i = 0; i < rows * wpr; i++) words[i] = 0;
        for (uint64_t r = 0; r < rows; r++)
            for (uint64_t c = 0; c < cols; c++) {
                float s = scales[(r / gr) * tc + (c / gc)];
                int32_t code = (s == 0.0f) ? 0 : qo_quantize_sym(w[r * cols + c], s, bits);
                uint32_t* word = &words[r * wpr + c / 8];
                *word = qo_int4_pack(*word, (uint32_t)(c % 8), code);
            }
    }
    return QO_OK;
}

/* ---- quanta-array/src/quant.rs:373-413 : dequantize_host -------------- */

/* codes_len: element count of the codes payload (bytes for int8, words for
 * int4); scales_len: element count of the scale grid. */
int qo_dequantize_host(const void* codes, uint64_t codes_len, const float* scales,
                       uint64_t scales_len, uint64_t rows, uint64_t cols, uint32_t bits,
                       uint64_t gr, uint64_t gc, float* out) {
    if (rows == 0 || cols == 0) return QO_ERR_RANK;
    if (gr == 0 || gc == 0 || gr > rows || gc > cols) return QO_ERR_GRANULARITY;
    uint64_t tr = qo_div_ceil(rows, gr), tc = qo_div_ceil(cols, gc);
    if (scales_len != tr * tc) return QO_ERR_LENGTH;
    uint64_t wpr = qo_div_ceil(cols, 8);
    uint64_t want = bits == 8 ? rows * cols : rows * wpr;
    if (codes_len != want) return QO_ERR_LENGTH;
    for (uint64_t r = 0; r < rows; r++)
        for (uint64_t c = 0; c < cols; c++) {
            float s = scales[(r / gr) * tc + (c / gc)];
            int32_t q = bits == 8 ? (int32_t)((const int8_t*)codes)[r * cols + c]
                                  : qo_int4_unpack(((const uint32_t*)codes)[r * wpr + c / 8],
                                                   (uint32_t)(c % 8));
            out[r * cols + c] = qo_dequantize_sym(q, s);
        }
    return QO_OK;
}

/* ---- QuantizedLinear forward ------------------------------------------
 * quanta-nn/src/quant.rs:903-918: y = x @ deq(w) (+ b) where the f32 GEMM is
 * quanta-blas/src/gemm.rs:47-82 / 91-180: for every output entry
 * acc = 0; for p in 0..k { acc = acc + a*b }; result = alpha*acc + beta*c
 * with alpha = 1, beta = 0 over a zeroed C (quanta-array/src/linalg.rs:143-168),
 * then one broadcast f32 add of the bias.
 *
 * wd is the already-dequantized weight.  layout 0: wd is [in, out] (the
 * reference's Linear orientation, y = x @ wd); layout 1: wd is [out, in]
 * (y = x @ wd^T, the K-contiguous orientation of the decode and prefill workloads).  The
 * summation order over k is the same in both.  threads <= 1 runs serial;
 * otherwise output rows*cols are spread over OpenMP threads (the reference's
 * CPU lane spreads workgroups over available_parallelism() threads,
 * quanta-core/src/driver/cpu/device.rs:711-760). */
int qo_linear_forward_f32(const float* x, const float* wd, const float* bias, uint64_t m,
                          uint64_t in_dim, uint64_t out_dim, int layout, int threads, float* y) {
    const float alpha = 1.0f, beta = 0.0f;
#ifdef _OPENMP
    int nt = threads > 1 ? threads : 1;
#pragma omp parallel for collapse(2) num_threads(nt) schedule(static)
#endif
    for (uint64_t i = 0; i < m; i++)
        for (uint64_t j = 0; j < out_dim; j++) {
            float acc = 0.0f;
            if (layout == 0) {
                for (uint64_t p = 0; p < in_dim; p++) acc = acc + x[i * in_dim + p] * wd[p * out_dim + j];
            } else {
                const float* wr = wd + j * in_dim;
                for (uint64_t p = 0; p < in_dim; p++) acc = acc + x[i * in_dim + p] * wr[p];
            }
            float result = alpha * acc + beta * 0.0f;
            if (bias) result = result + bias[j];
            y[i * out_dim + j] = result;
        }
    (void)threads;
    return QO_OK;
}

/* The same forward accumulated in f64 over optionally bf16-staged operands:
 * the checker for the tensor-core prefill path, whose stated staging is
 * x -> bf16 (already bf16 on input) and w_staged = bf16_rn(s * q).
 * stage_w != 0 rounds every dequantized weight through bf16 first. */
int qo_linear_forward_f64(const float* x, const float* wd, const float* bias, uint64_t m,
                          uint64_t in_dim, uint64_t out_dim, int layout, int stage_w, int threads,
                          double* y) {
#ifdef _OPENMP
    int nt = threads > 1 ? threads : 1;
#pragma omp parallel for collapse(2) num_threads(nt) schedule(static)
#endif
    for (uint64_t i = 0; i < m; i++)
        for (uint64_t j = 0; j < out_dim; j++) {
            double acc = 0.0;
            for (uint64_t p = 0; p < in_dim; p++) {
                float wv = layout == 0 ? wd[p * out_dim + j] : wd[j * in_dim + p];
                if (stage_w) wv = qo_bf16_to_f32(qo_f32_to_bf16(wv));
                acc += (double)x[i * in_dim + p] * (double)wv;
            }
            if (bias) acc += (double)bias[j];
            y[i * out_dim + j] = acc;
        }
    (void)threads;
    return QO_OK;
}

/* Dequantize + forward in one call with all host threads: the timed CPU
 * baseline of the whole QuantizedLinear::apply (dequantize dispatch, then the
 * GEMM).  scratch must hold rows*cols f32 (the reference materialises the
 * whole f32 weight every forward, quanta-array/src/quant.rs:616-637). */
int qo_qlinear_apply(const void* codes, const float* scales, uint64_t rows, uint64_t cols,
                     uint32_t bits, uint64_t gr, uint64_t gc, int layout, const float* x,
                     uint64_t m, const float* bias, int threads, float* scratch, float* y) {
    uint64_t tc = qo_div_ceil(cols, gc), wpr = qo_div_ceil(cols, 8);
#ifdef _OPENMP
    int nt = threads > 1 ? threads : 1;
#pragma omp parallel for num_threads(nt) schedule(static)
#endif
    for (uint64_t r = 0; r < rows; r++)
        for (uint64_t c = 0; c < cols; c++) {
            float s = scales[(r / gr) * tc + (c / gc)];
            int32_t q = bits == 8 ? (int32_t)((const int8_t*)codes)[r * cols + c]
                                  : qo_int4_unpack(((const uint32_t*)codes)[r * wpr + c / 8],
                                                   (uint32_t)(c % 8));
            scratch[r * cols + c] = qo_dequantize_sym(q, s);
        }
    uint64_t in_dim = layout == 0 ? rows : cols, out_dim = layout == 0 ? cols : rows;
    return qo_linear_forward_f32(x, scratch, bias, m, in_dim, out_dim, layout, threads, y);
}

int qo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
