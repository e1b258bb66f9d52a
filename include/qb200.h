/*
 * qb200.h — C ABI of the B200-native quantized-inference path.
 *
 * The drop-in boundary for quanta's weight-only int8/int4 path
 * (`quanta::sci::quant` / `quanta::nn::quant`): QuantizedMatrix quantize /
 * dequantize, QuantizedLinear forward over resident codes with a 2-D scale
 * grid, and the quantized-safetensors byte layout.  Each entry point names the
 * reference interface it replaces (path within the reference project : line).
 *
 * Conventions
 *   - Every function returns a qb200_status (0 = OK).  On failure a
 *     self-contained message naming the offender is kept per host thread and
 *     read back with qb200_last_error(); its wording carries the reference's
 *     message substrings (crates/sci/quanta-array/src/quant.rs:235-265).
 *   - `*_dev` pointers are device pointers on the current CUDA device.  Device
 *     work is asynchronous on the caller's stream (a cudaStream_t passed as
 *     void*; NULL = the legacy default stream) unless the name ends in `_host`
 *     or `_sync`.
 *   - No entry point falls back to the CPU: without a usable CUDA device the
 *     device entry points return QB200_ERR_CUDA.
 *   - Matrices are rank-2 `[rows, cols]`, row-major.  Scale grid: tile
 *     `(gr, gc)`, scales `[ceil(rows/gr), ceil(cols/gc)]` f32 row-major, the
 *     scale of element (r, c) is scales[(r/gr)*ceil(cols/gc) + c/gc]
 *     (crates/sci/quanta-array/src/quant.rs:4-8).
 *   - Codes: bits = 8 -> int8, one byte per element `[rows, cols]`;
 *     bits = 4 -> uint32 words `[rows, ceil(cols/8)]`, 8 nibbles per word, low
 *     nibble first, every row starts a fresh word, pad nibbles zero
 *     (crates/sci/quanta-array/src/quant.rs:27-30).
 *   - Handles are not thread-safe; distinct handles are independent.
 */
#ifndef QB200_H
#define QB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define QB200_API __attribute__((visibility("default")))
#else
#define QB200_API
#endif

typedef int32_t qb200_status;

/* Status codes.  1..6 mirror the arms of QuantError
 * (crates/sci/quanta-array/src/quant.rs:210-233); 7 is
 * ArrayError::LengthMismatch; 8 is QuantaError::invalid_param. */
enum {
    QB200_OK = 0,
    QB200_ERR_RANK = 1,
    QB200_ERR_GRANULARITY = 2,
    QB200_ERR_GRID = 3,
    QB200_ERR_FORMAT = 4,
    QB200_ERR_NOT_SUPPORTED = 5,
    QB200_ERR_SCALE = 6,
    QB200_ERR_LENGTH = 7,
    QB200_ERR_INVALID_PARAM = 8,
    QB200_ERR_CUDA = 9,
    QB200_ERR_NCCL = 10,
    QB200_ERR_TIMEOUT = 11
};

/* Granularity spellings (crates/sci/quanta-array/src/quant.rs:94-104).
 * BLOCK{rows, cols} is an additive arm: the reference's arithmetic takes any
 * (gr, gc) but its enum cannot spell a 2-D block such as 32x32. */
enum { QB200_PER_TENSOR = 0, QB200_PER_CHANNEL = 1, QB200_GROUP = 2, QB200_BLOCK = 3 };

/* Weight orientation of a QuantizedLinear.
 * IN_OUT: the matrix is `[in, out]`, y = x @ deq(w)  (the reference's Linear,
 *         crates/ml/quanta-nn/src/quant.rs:820-835).
 * OUT_IN: the matrix is `[out, in]`, y = x @ deq(w)^T (K-contiguous rows). */
enum { QB200_IN_OUT = 0, QB200_OUT_IN = 1 };

/* Activation / output element types. */
enum { QB200_F32 = 0, QB200_BF16 = 1, QB200_F16 = 2 };

/* ---- library ------------------------------------------------------------ */

/* "major.minor.patch" of this library. */
QB200_API const char* qb200_version(void);

/* Copies the calling thread's last error message (NUL-terminated, truncated to
 * cap) and returns its full length.  Replaces Display for QuantError /
 * ArrayError (crates/sci/quanta-array/src/quant.rs:235-265). */
QB200_API size_t qb200_last_error(char* buf, size_t cap);

/* Number of CUDA devices visible (0 when none / no driver). */
QB200_API int32_t qb200_device_count(void);

/* ---- grid vocabulary (host only) --------------------------------------- */

/* Granularity::tile — spelling -> (gr, gc)
 * (crates/sci/quanta-array/src/quant.rs:109-144).  size is Group's size or
 * Block's rows; size2 is Block's cols. */
QB200_API qb200_status qb200_tile(int32_t kind, uint64_t axis, uint64_t size, uint64_t size2, uint64_t rows,
                        uint64_t cols, uint64_t* gr, uint64_t* gc);

/* granularity_from_grid — canonical spelling of a stored grid, precedence
 * PerTensor > PerChannel > Group (crates/ml/quanta-nn/src/quant.rs:119-145).
 * Returns QB200_ERR_FORMAT for a grid no v1 writer produces unless
 * allow_block is non-zero (then kind = QB200_BLOCK). */
QB200_API qb200_status qb200_granularity_from_grid(uint64_t rows, uint64_t cols, uint64_t gr, uint64_t gc,
                                         int32_t allow_block, int32_t* kind, uint64_t* axis,
                                         uint64_t* size, uint64_t* size2);

/* Byte size of the codes payload and element count of the scale grid. */
QB200_API qb200_status qb200_codes_bytes(uint64_t rows, uint64_t cols, uint32_t bits, uint64_t* bytes);
QB200_API qb200_status qb200_scales_count(uint64_t rows, uint64_t cols, uint64_t gr, uint64_t gc,
                                uint64_t* tile_rows, uint64_t* tile_cols);

/* QuantizedMatrix::from_parts validation: codes / scales element counts
 * against the logical shape and grid
 * (crates/sci/quanta-array/src/quant.rs:521-568). */
QB200_API qb200_status qb200_check_parts(uint64_t codes_rows, uint64_t codes_cols, uint64_t scales_rows,
                               uint64_t scales_cols, uint64_t rows, uint64_t cols, uint32_t bits,
                               uint64_t gr, uint64_t gc);

/* ---- quantize / dequantize on the device ------------------------------- */

/* QuantizedMatrix::quantize + quantize_host: per-tile max-abs -> s = m/hi ->
 * clamp(round_ties_even(w/s)) -> pack
 * (crates/sci/quanta-array/src/quant.rs:293-367, 480-513).  The reference runs
 * this loop on one host thread over a device read-back; here it is one pass
 * over HBM.  src_dtype is the element type of w_dev (F32 exact; BF16 / F16
 * are widened exactly first, crates/ml/quanta-nn/src/safetensors.rs:497-551).
 * Bit-exact codes and scales. */
QB200_API qb200_status qb200_quantize(const void* w_dev, int32_t src_dtype, uint64_t rows, uint64_t cols,
                            uint32_t bits, uint64_t gr, uint64_t gc, void* codes_dev,
                            float* scales_dev, void* stream);

/* QuantizedMatrix::dequantize / dequantize_host: out[r,c] = s * f32(q)
 * (crates/sci/quanta-array/src/quant.rs:373-413, 605-752).  Bit-exact. */
QB200_API qb200_status qb200_dequantize(const void* codes_dev, const float* scales_dev, uint64_t rows,
                              uint64_t cols, uint32_t bits, uint64_t gr, uint64_t gc,
                              float* out_dev, void* stream);

/* ---- QuantizedLinear ---------------------------------------------------- */

typedef struct qb200_qlinear qb200_qlinear;

/* QuantizedLinear::new (Mode B, resident codes)
 * (crates/ml/quanta-nn/src/quant.rs:853-862).  Borrows the caller's device
 * buffers (codes, scales, optional f32 bias of out_dim elements): they must
 * outlive the handle.  bias_len is the bias element count (checked against
 * out_dim like check_bias, quant.rs:838-848); pass bias_dev = NULL for none.
 * Where the stored layout does not feed the fast kernels as it is, the handle builds an execution copy here (and
 * synchronises the device once):
 *   - an `[in, out]` weight whose tile height is a multiple of 16 that divides in_dim, or spans it (int4
 *     Group{axis: 0, size: 128}, the reference's own orientation; int8 32 x 32 blocks; per-column scales ...) is transposed
 *     to `[out, in]` together with its scale grid;
 *   - an int4 grid whose scale is constant over whole 128-column runs (tile widths that are multiples of 128, per-row and
 *     per-tensor scales) gets its scales spelt out per run, `[out][in / 128]` f32, and is a 1x128 layer from then on;
 *   - a weight with more than 4096 inputs (up to 32768) is cut into column slices for the decode kernels (int4 1x128;
 *     int8 with tiles 32, 64 or 128 columns wide).
 * A copy of codes costs them again (0.5 or 1 byte per weight) plus its scales (and 16 rows of f32 partial outputs per
 * slice); the caller's buffers stay the record. */
QB200_API qb200_status qb200_qlinear_create(const void* codes_dev, const float* scales_dev, uint64_t rows,
                                  uint64_t cols, uint32_t bits, uint64_t gr, uint64_t gc,
                                  int32_t layout, const float* bias_dev, uint64_t bias_len,
                                  qb200_qlinear** out);
QB200_API void qb200_qlinear_destroy(qb200_qlinear* ql);

/* Layer::in_dim / Layer::out_dim (crates/ml/quanta-nn/src/quant.rs:882-887). */
QB200_API uint64_t qb200_qlinear_in_dim(const qb200_qlinear* ql);
QB200_API uint64_t qb200_qlinear_out_dim(const qb200_qlinear* ql);

/* Layer::apply without the tape — y = x @ deq(w) (+ b), fused: the f32 weight
 * is never materialised (crates/ml/quanta-nn/src/quant.rs:892-918, the
 * "INTEGRATOR SEAM").  x is `[m, in_dim]` of x_dtype, y is `[m, out_dim]` of
 * y_dtype, both device, row-major.  f32 accumulation.
 * Fast paths (bf16 x): int4 with a 1x128 grid — `[out, in]`, or `[in, out]` with Group{axis: 0, size: 128} through the
 * transposed execution copy made at creation; also every int4 grid whose scale is constant over whole 128-column runs
 * (tile widths that are multiples of 128, per-row and per-tensor scales), spelt out as 1x128 at creation — on the decode GEMV (m <= 16; inputs wider than 4096 as column slices) and
 * the tcgen05 GEMM (m > 16), which also takes the other int4 grids whose tile width along the inputs is a multiple of 16 that
 * divides in_dim or spans it (Group sizes 32, 64, 256 ..., per-row, per-tensor; `[in, out]` with such groups along axis 0
 * through the transposed copy) from m = 9; int8 `[out, in]` with any grid whose tiles are a multiple of 32 columns wide on
 * its own decode GEMV (m <= 16; inputs wider than 4096 as column slices when the tiles are 32, 64 or 128 columns wide), and with in_dim a multiple of 64 and tiles of whole 16-column steps that
 * divide in_dim (or span it) on the same tcgen05 GEMM (from m = 5); int8 `[in, out]` whose tile height is such a number through a transposed copy
 * of codes and scale grid made at creation.  f32 activations (the reference's own dtype) whose layer has such a fast path
 * are split into three bf16 parts whose sum is the f32 exactly (x -> [3 m, in_dim], two small kernels and grow-only staging
 * in the handle), run on the bf16 kernel for 3 m rows, and the three partial outputs are added: exact products, f32
 * accumulation (calls of fewer than 2^24 multiply-adds keep the generic kernel's single launch; QB200_F32_SPLIT=0 in the
 * environment keeps every f32 call there).  Everything else (other grids and layouts) runs on the generic kernels.
 * A call whose scratch is not allocated yet (the GEMM's split-K workspace, the generic column kernel's partial sums)
 * allocates it; on a stream that is recording a CUDA graph that is refused with QB200_ERR_INVALID_PARAM — run the shape
 * once before capturing.  The decode GEMVs need finite activations with |x| < 2^87 (see qb200_qlinear_check). */
QB200_API qb200_status qb200_qlinear_forward(qb200_qlinear* ql, const void* x_dev, int32_t x_dtype,
                                   uint64_t m, void* y_dev, int32_t y_dtype, void* stream);

/* qb200_qlinear_forward for callers that may not allocate device memory (serving
 * loops with a frozen memory budget, hosts that hand every device buffer to another
 * runtime, latency-critical code where cudaMalloc's implicit synchronisation is not
 * acceptable).  No counterpart in the reference.
 * Serves `[in, out]` handles (QB200_IN_OUT), whose column kernel splits K and needs
 * room for partial sums: here that room is a 2 MiB array built into the library
 * image (held by every GPU that loads the library until the process exits) instead
 * of the handle's grow-on-demand buffer.  The call performs no cudaMalloc / cudaFree.
 *   - `K slices * m * out_dim` partial sums must fit 2^19 floats; larger calls are
 *     refused with QB200_ERR_INVALID_PARAM and a message naming the sizes.
 *   - The first call on a device looks the array's address up (cudaGetSymbolAddress);
 *     make that first call outside any stream capture.
 *   - All calls share the one array: two calls that overlap on the GPU (different
 *     streams, or different handles) race on it.  Calls ordered on one stream are safe.
 *     The array keeps the last call's contents; nothing in it needs to start at zero.
 * Results are identical to qb200_qlinear_forward. */
QB200_API qb200_status qb200_qlinear_forward_static(qb200_qlinear* ql, const void* x_dev, int32_t x_dtype,
                                          uint64_t m, void* y_dev, int32_t y_dtype, void* stream);

/* `count` forwards in one call: entry i computes y_dev[i] = layers[i](x_dev[i]), the
 * result of calling qb200_qlinear_forward once per layer in order (the reference
 * stacks layers and loops over Layer::apply,
 * crates/ml/quanta-nn/tests/quant.rs:507-523).  Layers that share the input width
 * and take the decode path run as ONE persistent launch that streams all their
 * codes back to back (fused QKV / gate+up projections); any other mix falls back
 * to the per-layer loop.  The outputs must not alias each other's inputs. */
QB200_API qb200_status qb200_qlinear_forward_many(qb200_qlinear* const* layers, uint32_t count,
                                        const void* const* x_dev, int32_t x_dtype, uint64_t m,
                                        void* const* y_dev, int32_t y_dtype, void* stream);

/* ---- support ops of a decode step (needed to time the whole-model configuration; f32 arithmetic,
 * bf16 storage for what feeds the next linear and for the KV cache) ----
 * qb200_add_rmsnorm: h += delta[0] + ... + delta[delta_parts - 1] (arrays of n * c floats back to back, for example the
 *   partial outputs of a sliced linear; delta_parts = 0: nothing is added), out = bf16(h * rrms * gamma),
 *   rrms = 1 / sqrt(sum(h^2) / c + eps) (crates/ml/quanta-nn/src/norm.rs:192-225).
 * qb200_rope_append: rotate-half RoPE of q and k with one position's cos / sin rows ([hd] each, built in f64 on the
 *   host as crates/sci/quanta-array/src/autograd/rope.rs:43-63 does); q -> bf16 [b, heads, hd], rotated k and v ->
 *   row `pos` of the caches [b, ctx_max, heads, hd] (crates/ml/quanta-nn/src/rope.rs:23-58).
 * qb200_sdpa_decode: one query per (batch row, head) against the first kv_len cache rows, online softmax,
 *   score = scale * (q . k) (crates/ml/quanta-nn/src/kernel.rs:64-175); head dim 128; scratch holds
 *   qb200_sdpa_decode_scratch_floats(b, heads, kv_len) floats.
 * qb200_swiglu_sliced: out = a * s * b with s = 1 / (1 + exp(min(-a, 30))) (crates/ml/quanta-nn/src/activation.rs:
 *   145-162), a = gate[n, h], b = up[n, h]; the result is written as `slices` blocks [n, width_s] laid back to back
 *   (column slices of the [n, h] result; with pad_to > 0 every block is [n, pad_to] and the columns past the slice's
 *   width are left as they are), so a following linear wider than the decode kernel's input limit can run as a
 *   grouped launch over contiguous inputs of one width.
 * qb200_sum_arrays: y = parts[0] + ... + parts[count - 1], n floats each (the partial outputs of such a linear). */
QB200_API qb200_status qb200_add_rmsnorm(float* h, const float* delta, uint32_t delta_parts, const float* gamma, uint64_t n,
                                         uint64_t c, float eps, uint16_t* out_bf16, void* stream);
QB200_API qb200_status qb200_rope_append(const float* q, const float* k, const float* v, const float* cos_row,
                                         const float* sin_row, uint32_t b, uint32_t heads, uint32_t hd, uint16_t* q_out,
                                         uint16_t* kcache, uint16_t* vcache, uint32_t ctx_max, uint32_t pos, void* stream);
QB200_API uint64_t qb200_sdpa_decode_scratch_floats(uint32_t b, uint32_t heads, uint32_t kv_len);
QB200_API qb200_status qb200_sdpa_decode(const uint16_t* q, const uint16_t* kcache, const uint16_t* vcache, uint32_t b,
                                         uint32_t heads, uint32_t hd, uint32_t ctx_max, uint32_t kv_len, float scale,
                                         float* scratch, uint16_t* out, void* stream);
QB200_API qb200_status qb200_swiglu_sliced(const float* gate, const float* up, uint64_t n, uint64_t h,
                                           const uint32_t* slice_widths, uint32_t slices, uint32_t pad_to, uint16_t* out,
                                           void* stream);
QB200_API qb200_status qb200_sum_arrays(const float* parts, uint32_t count, uint64_t n, float* y, void* stream);

/* ---- fused all-gather for column-sharded layers (no counterpart in the reference: it has no
 * multi-GPU code, crates/ml/quanta-nn/PARITY.md:76-79) ----
 * Every rank of a node owns one gather buffer of the same layout (for example [world][layer][m][n]);
 * the buffers are cudaMalloc allocations shared between the ranks' processes by CUDA IPC handles.
 * qb200_qlinear_forward_many_gather is qb200_qlinear_forward_many whose kernel stores each output
 * element into EVERY rank's buffer (plain stores to peer memory over NVLink, no collective):
 * y_own[i] points into this rank's own buffer, gather_bases[p] is rank p's buffer as mapped in this
 * process (gather_bases[rank] the own one), and the element goes to y_own[i] + (gather_bases[p] -
 * gather_bases[rank]) for every p.  Decode shapes only (int4, grid 1x128, [out, in], bf16 x, m <= 16,
 * in <= 4096), else QB200_ERR_NOT_SUPPORTED.  The arrival barrier — "this rank's outputs of this step
 * are written" published to every peer, then a wait for theirs, bounded to about a second — runs inside
 * the same launch when flag_arrays is given (its last CTA does it; a timeout lands in layers[0]'s status
 * word, read with qb200_qlinear_check), or as qb200_peer_signal_wait on the same stream afterwards when
 * flag_arrays is null (QB200_ERR_TIMEOUT then lands in status_dev).  flag_arrays[p] is a
 * zero-initialised array of 16 uint64 inside rank p's shared allocation, as mapped in this process. */
QB200_API qb200_status qb200_peer_alloc(uint64_t bytes, void** dev_ptr, uint8_t* handle64);
QB200_API qb200_status qb200_peer_open(const uint8_t* handle64, void** dev_ptr);
QB200_API qb200_status qb200_peer_close(void* dev_ptr);
QB200_API qb200_status qb200_peer_free(void* dev_ptr);
QB200_API qb200_status qb200_qlinear_forward_many_gather(qb200_qlinear* const* layers, uint32_t count,
                                               const void* const* x_dev, int32_t x_dtype, uint64_t m,
                                               void* const* y_own, int32_t y_dtype, void* const* gather_bases,
                                               uint64_t* const* flag_arrays, uint32_t world, uint32_t rank,
                                               void* stream);
QB200_API qb200_status qb200_peer_signal_wait(uint64_t* const* flag_arrays, uint32_t world, uint32_t rank,
                                    int32_t* status_dev, void* stream);
/* Polls (about a quarter of a microsecond each) that an arrival barrier spends on one peer's flag before it
 * gives up with QB200_ERR_TIMEOUT; process-wide, read at launch time.  Default: the environment variable
 * QB200_SPIN_LIMIT (polls) when set at first use, else 4 Mi (about a second). */
QB200_API qb200_status qb200_peer_set_spin_limit(uint32_t polls);

/* ---- pushed exchanges for tensor-parallel decode (no counterpart in the reference) ----
 * The barrier of qb200_qlinear_forward_many_gather costs several microseconds per exchange (a system-scope fence
 * waits for the peers to acknowledge every store in flight, then the flags travel).  A decode step of a sharded
 * model makes dozens of exchanges of a few hundred KB, so here the data validates itself instead: every output is
 * stored as ONE 8-byte element {f32 bits, exchange number} into the same offset of every rank's arena
 * (arena_bases[p] as mapped in this process, arena_bases[rank] the own one; slot_own[i] is where layer i's
 * `[m, out]` elements start inside the own arena, 8 bytes each), and the launch ends without any fence or wait.
 * The consumers poll each element until it carries the exchange number they expect:
 *   qb200_add_rmsnorm_pushed — qb200_add_rmsnorm over `parts` pushed arrays of n * c elements laid back to back
 *     (for example one partial output per rank of a row-parallel layer), summed in part order;
 *   qb200_gather_pushed — part r holds `rows` x w_r elements of a column-sharded output (w_r = cols / parts, one
 *     more for the first cols % parts ranks), parts `part_stride` elements apart; they are written as f32 into
 *     columns [lo_r, lo_r + w_r) of dst (rows dst_stride floats apart).
 * state_own is this rank's zero-initialised array of 16 uint64 (device memory): word 8 counts the exchanges this
 * rank has launched, which is the number the next consumer expects — every rank must go through the same
 * sequence of pushes and consumers.  A buffer may be pushed into again only after another exchange (into another
 * buffer) has been consumed in between: a rank cannot finish that one before every rank has read the first.
 * Waits are bounded by qb200_peer_set_spin_limit; a consumer that gives up writes QB200_ERR_TIMEOUT to status_dev
 * (an int32 in device memory, zero-initialised) and uses zeros.  Decode shapes only, all layers in ONE launch
 * (else QB200_ERR_NOT_SUPPORTED).  Exchange numbers are 32 bits wide.
 * slot_stride = 0: the launch only pushes (the consumers above wait for the data).  slot_stride > 0 makes the launch a
 * complete all-gather: every rank runs the SAME layers shapes into slot `rank` of a buffer whose slots lie slot_stride
 * bytes apart (slot_own[i] inside slot `rank`), and each CTA, after its own rows, polls the same rows of every other
 * rank's slot in the own arena — its twin on that rank pushes them at about the same time — so when the launch ends all
 * ranks' elements are in place (a timeout lands in layers[0]'s status word, qb200_qlinear_check). */
QB200_API qb200_status qb200_qlinear_forward_many_push(qb200_qlinear* const* layers, uint32_t count, const void* const* x_dev,
                                                       int32_t x_dtype, uint64_t m, void* const* slot_own, void* const* arena_bases,
                                                       uint32_t world, uint32_t rank, uint64_t* state_own, uint64_t slot_stride,
                                                       void* stream);
QB200_API qb200_status qb200_add_rmsnorm_pushed(float* h, const void* pushed, uint32_t parts, const uint64_t* state_own,
                                                const float* gamma, uint64_t n, uint64_t c, float eps, uint16_t* out_bf16,
                                                int32_t* status_dev, void* stream);
QB200_API qb200_status qb200_gather_pushed(const void* pushed, uint32_t parts, uint64_t part_stride, uint32_t rows, uint64_t cols,
                                           const uint64_t* state_own, float* dst, uint64_t dst_stride, int32_t* status_dev,
                                           void* stream);

/* ---- tensor parallelism over a library collective (no counterpart in the reference) ----
 * For every shape the fused exchanges above do not take (prefill batches, int8 layers, inputs wider than 4096, GPUs
 * without peer access): each rank runs its shard's ordinary forward and NCCL moves the outputs.  NCCL is opened at
 * run time (libnccl.so.2); a failure to load it or an NCCL error is QB200_ERR_NCCL.
 *   qb200_shard_rows — rows [lo, hi) of rank's block of an `[out, in]` weight: equal blocks of whole scale tiles
 *     (`gr` rows), trailing ranks short or empty; the codes and scales of the block are contiguous: a pointer offset.
 *   qb200_shard_cols — columns [lo, hi) for the row-parallel pairing: whole scale tiles (`gc`) and whole packed words.
 *   qb200_tp_unique_id / qb200_tp_create — rank 0 makes the 128-byte id, the caller hands it to every rank, every
 *     rank creates its communicator with its own device current.
 *   qb200_qlinear_forward_tp — QB200_TP_COLUMN: `shard` holds rank's row block (qb200_shard_rows(full_dim, granule)),
 *     x is the full `[m, in]`, y receives the gathered `[m, full_dim]` on every rank (f32 or bf16).
 *     QB200_TP_ROW: `shard` holds rank's column block, x is rank's `[m, hi - lo]` slice, y receives the f32 sum of the
 *     partial outputs on every rank (the order of the sum differs from the unsharded layer's: equal to 1e-4, not bit for
 *     bit; give the bias to one rank's shard only).  A rank that owns nothing passes shard = NULL.  The gather's staging
 *     buffer grows on demand: run the largest shape once before capturing calls into a CUDA graph.
 *   qb200_tp_status — synchronises `stream` and reports the shard's device status word (qb200_qlinear_check). */
typedef struct qb200_tp qb200_tp;
enum { QB200_TP_COLUMN = 0, QB200_TP_ROW = 1 };
QB200_API qb200_status qb200_shard_rows(uint64_t rows, uint64_t gr, uint32_t world, uint32_t rank, uint64_t* lo, uint64_t* hi);
QB200_API qb200_status qb200_shard_cols(uint64_t cols, uint64_t gc, uint32_t bits, uint32_t world, uint32_t rank, uint64_t* lo,
                                        uint64_t* hi);
QB200_API qb200_status qb200_tp_unique_id(uint8_t* id128);
QB200_API qb200_status qb200_tp_create(uint32_t rank, uint32_t world, const uint8_t* id128, qb200_tp** out);
QB200_API void qb200_tp_destroy(qb200_tp* tp);
QB200_API uint32_t qb200_tp_rank(const qb200_tp* tp);
QB200_API uint32_t qb200_tp_world(const qb200_tp* tp);
QB200_API qb200_status qb200_qlinear_forward_tp(qb200_tp* tp, qb200_qlinear* shard, int32_t mode, uint64_t full_dim, uint64_t granule,
                                                const void* x_dev, int32_t x_dtype, uint64_t m, void* y_dev, int32_t y_dtype,
                                                void* stream);
QB200_API qb200_status qb200_tp_status(qb200_tp* tp, qb200_qlinear* shard, void* stream);

/* qb200_qlinear_forward_many over HOST buffers: every distinct input pointer is
 * copied to the device once, the forwards run, all outputs are copied back and
 * the call synchronises.  Staging buffers belong to layers[0] and grow on demand.
 * Decode-shaped calls whose outputs lie in pinned, device-mapped host memory
 * (cudaHostAlloc / cudaHostRegister) skip the copy back: the kernel stores there
 * itself while it is still streaming weights. */
QB200_API qb200_status qb200_qlinear_forward_many_host(qb200_qlinear* const* layers, uint32_t count,
                                             const void* const* x_host, int32_t x_dtype, uint64_t m,
                                             void* const* y_host, int32_t y_dtype);

/* Synchronises `stream` and reads the handle's device status word: kernels whose
 * bounded waits (on an async copy) ran out of polls record QB200_ERR_TIMEOUT there
 * and return early instead of spinning.  A recorded error is reported once and the word is cleared.
 * No counterpart in the reference (its
 * error taxonomy names Timeout, crates/gpu/quanta-core/src/api/error.rs:29-60). */
QB200_API qb200_status qb200_qlinear_check(qb200_qlinear* ql, void* stream);

/* The same call over HOST buffers: copies x to the device, runs the forward,
 * copies y back and synchronises.  Staging buffers are owned by the handle
 * and grow on demand. */
QB200_API qb200_status qb200_qlinear_forward_host(qb200_qlinear* ql, const void* x_host, int32_t x_dtype,
                                        uint64_t m, void* y_host, int32_t y_dtype);

/* Name of the kernel family the last forward on this handle dispatched to: "gemv_mma" (int4 decode), "gemv_mma_grouped",
 * "gemv_mma_sliced" (inputs wider than 4096), "gemv_mma_grouped_gather" / "gemv_mma_grouped_push" (fused exchanges),
 * "gemv_mma_i8", "gemv_mma_i8_grouped", "gemv_mma_i8_x2", "gemv_mma_i8_sliced" (int8 decode), "gemm_tcgen05" (int4 prefill), "gemm_tcgen05_i8" (int8 prefill), "generic_rows",
 * "generic_cols". */
QB200_API const char* qb200_qlinear_last_kernel(const qb200_qlinear* ql);

/* ---- quantized-safetensors (host bytes in, host bytes out) -------------- */

typedef struct qb200_st_file qb200_st_file;
typedef struct qb200_st_writer qb200_st_writer;

/* One validated leaf in header order. */
typedef struct {
    const char* name;      /* leaf name (quantized: without the .q / .qs suffix) */
    int32_t quantized;     /* 0 = plain tensor, 1 = quantized leaf                */
    const char* dtype;     /* plain: "F32" / "F16" / "BF16"; quantized: "I8"/"U32" */
    uint32_t ndim;         /* plain: rank; quantized: 2                            */
    const uint64_t* shape; /* plain: tensor shape; quantized: logical [rows, cols] */
    uint64_t data_offset;  /* byte offset of the tensor / codes in the input bytes */
    uint64_t data_len;
    uint32_t bits;         /* quantized only: 8 / 4                                */
    uint64_t gr, gc;       /* quantized only                                       */
    uint64_t scales_offset; /* quantized only: F32 scale grid in the input bytes   */
    uint64_t scales_len;
    int32_t gran_kind;     /* canonical granularity spelling of the grid           */
    uint64_t gran_axis, gran_size, gran_size2;
} qb200_st_item;

/* validate(): container parse, version gate and total per-leaf validation
 * before anything is interpreted (crates/ml/quanta-nn/src/quant.rs:420-635,
 * crates/ml/quanta-nn/src/safetensors.rs:398-492).  bytes must stay alive
 * while the handle is used.  allow_block admits 2-D block grids. */
QB200_API qb200_status qb200_st_validate(const uint8_t* bytes, uint64_t len, int32_t allow_block,
                               qb200_st_file** out);
QB200_API void qb200_st_free(qb200_st_file* f);
QB200_API uint64_t qb200_st_num_items(const qb200_st_file* f);
QB200_API qb200_status qb200_st_item_at(const qb200_st_file* f, uint64_t i, qb200_st_item* out);
/* User metadata (the quant:* entries and the version key are stripped). */
QB200_API uint64_t qb200_st_num_metadata(const qb200_st_file* f);
QB200_API qb200_status qb200_st_metadata_at(const qb200_st_file* f, uint64_t i, const char** key,
                                  const char** value);

/* entry_to_f32 on the host: widen a plain F32 / F16 / BF16 tensor to f32
 * (crates/ml/quanta-nn/src/safetensors.rs:497-551).  out holds count f32. */
QB200_API qb200_status qb200_st_plain_to_f32(const qb200_st_file* f, uint64_t i, float* out, uint64_t count);

/* save_named(): leaves in the given order, metadata keys sorted, the version
 * key and quant:<leaf> entries synthesised
 * (crates/ml/quanta-nn/src/quant.rs:279-390,
 * crates/ml/quanta-nn/src/safetensors.rs:72-125). */
QB200_API qb200_status qb200_st_writer_create(qb200_st_writer** out);
QB200_API void qb200_st_writer_free(qb200_st_writer* w);
/* has_metadata: the caller passed Some(map) even when it is empty. */
QB200_API qb200_status qb200_st_writer_set_has_metadata(qb200_st_writer* w, int32_t has_metadata);
QB200_API qb200_status qb200_st_writer_add_metadata(qb200_st_writer* w, const char* key, const char* value);
QB200_API qb200_status qb200_st_writer_add_f32(qb200_st_writer* w, const char* name, const uint64_t* shape,
                                     uint32_t ndim, const float* data);
QB200_API qb200_status qb200_st_writer_add_quantized(qb200_st_writer* w, const char* name, uint32_t bits,
                                           uint64_t rows, uint64_t cols, uint64_t gr, uint64_t gc,
                                           const void* codes, const float* scales);
/* Serialises; the returned bytes belong to the writer until it is freed. */
QB200_API qb200_status qb200_st_writer_finish(qb200_st_writer* w, const uint8_t** bytes, uint64_t* len);

/* parse_quant_meta(): the `quant:<leaf>` value grammar
 * (crates/ml/quanta-nn/src/quant.rs:211-271). */
QB200_API qb200_status qb200_st_parse_quant_meta(const char* leaf, const char* value, uint32_t* bits,
                                       uint64_t* gr, uint64_t* gc, uint64_t* rows, uint64_t* cols);

/* ---- quantized BLAS entries: integer codes for BOTH operands, per-tensor symmetric scales ----
 * GemmQuantType (crates/sci/quanta-blas/src/mixed_quant.rs:22-31). */
enum { QB200_Q8_SYMMETRIC = 0, QB200_Q4_SYMMETRIC = 1 };

/* gemm_quant(): C <- alpha * (a_scale * A) * (b_scale * B) + beta * C; A [m, k] and B [k, n] row-major int8
 * codes, one per i32 word; C [m, n] f32, read for beta * C and overwritten
 * (crates/sci/quanta-blas/src/mixed_quant.rs:47-81; CPU twin crates/sci/quanta-blas/src/reference.rs:212-226).
 * qty other than QB200_Q8_SYMMETRIC: QB200_ERR_INVALID_PARAM, as the reference errors.  All pointers are device
 * memory; the call is asynchronous on `stream`.  The sum of code products is formed exactly in integers
 * (tcgen05 kind::i8), where the reference accumulates the products in f32: equal bit for bit while the
 * running sum stays below 2^24, and within the reference's own test tolerance (1e-3 * (1 + |want|)) beyond.
 * Codes outside [-128, 127] and k > 131071 are not served: the first is reported by qb200_gemm_quant_check,
 * the second returns QB200_ERR_NOT_SUPPORTED. */
QB200_API qb200_status qb200_gemm_quant(int qty, uint32_t m, uint32_t n, uint32_t k, float alpha, float a_scale,
                                        float b_scale, const int32_t* a_dev, const int32_t* b_dev, float beta,
                                        float* c_dev, void* stream);
/* gemm_quant4(): the same over int4 codes packed eight per u32 word by FLAT element index (word i / 8,
 * nibble i % 8; A holds ceil(m * k / 8) words, B ceil(k * n / 8))
 * (crates/sci/quanta-blas/src/mixed_quant.rs:104-127; reference.rs:235-262). */
QB200_API qb200_status qb200_gemm_quant4(int qty, uint32_t m, uint32_t n, uint32_t k, float alpha, float a_scale,
                                         float b_scale, const uint32_t* a_dev, const uint32_t* b_dev, float beta,
                                         float* c_dev, void* stream);
/* gemv_quant() / gemv_quant4(): A [m, n] codes, x [n] codes, y [m] f32 — gemm_quant(m, 1, n, ...)
 * (crates/sci/quanta-blas/src/mixed_quant.rs:83-100, 129-147).  One pass over A's codes. */
QB200_API qb200_status qb200_gemv_quant(int qty, uint32_t m, uint32_t n, float alpha, float a_scale, float x_scale,
                                        const int32_t* a_dev, const int32_t* x_dev, float beta, float* y_dev,
                                        void* stream);
QB200_API qb200_status qb200_gemv_quant4(int qty, uint32_t m, uint32_t n, float alpha, float a_scale, float x_scale,
                                         const uint32_t* a_dev, const uint32_t* x_dev, float beta, float* y_dev,
                                         void* stream);
/* Waits for `stream` and reports what the quantized BLAS kernels launched on it recorded since the last
 * check: QB200_ERR_INVALID_PARAM for an int8 code out of range, QB200_ERR_TIMEOUT for a bounded wait that
 * ran out.  The packed operands live in a buffer per (device, stream) that grows on demand and is reused; growing it
 * allocates and synchronises, so a caller that captures these entries into a CUDA graph runs the largest shape once
 * on that stream before the capture. */
QB200_API qb200_status qb200_gemm_quant_check(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QB200_H */
