/* halo_b200: B200 (sm_100a) replacements for halo-flash's fused per-layer
 * elementwise kernels, behind a C ABI.
 *
 * halo-flash's engine never links kernels: it looks a kernel up by name
 * (rt::Device::Kernel, src/rt/device.hpp:120) and launches it with a grid, a block
 * and an ordered argument list (rt::Device::Launch, src/rt/device.hpp:127; pointer
 * parameters are buffers, everything else a by-value scalar, device.hpp:8-11).
 * Each function below replaces one such kernel entry point of src/kernels/core.hip
 * or src/kernels/batch_decode.hip. It keeps the kernel's name and its parameter
 * list in the kernel's own order, and adds
 *   - the stream first (the engine's single stream, src/rt/hip_device.cpp:49-50),
 *   - the row / batch counts the reference passes through its grid dimensions,
 *   - the error out-parameters of the repository's C ABIs
 *     (include/halo_variant.h:12-13).
 * Launch geometry is this library's own; a caller's block size is irrelevant.
 * halo_b200_launch() takes the reference's (name, grid, block, args) call as is.
 *
 * Contract
 *   - Returns 0 on success, -1 on failure with a NUL-terminated message in err
 *     (truncated to errlen; err may be NULL).
 *   - All pointers are device pointers owned by the caller. No call allocates or
 *     synchronizes (halo_b200_stage_timeouts, a diagnostic read, is the exception):
 *     every other call only enqueues kernels on `stream` and may be recorded by CUDA
 *     stream capture.
 *   - State the library keeps, all of it listed here: (1) the fixed 4 MiB device array of
 *     halo_b200_norm_rope_qk_noalloc (per GPU, shared by its calls); (2) a device counter
 *     of staging waits that ran out (halo_b200_stage_timeouts; zero in normal
 *     operation); (3) the process-wide tuning switches of halo_b200_tune (host atomics,
 *     for experiments; production code never needs to touch them). Everything else is
 *     stateless and re-entrant.
 *   - Ordering: kernels are launched with programmatic stream serialization. A kernel reads
 *     and writes memory only after the kernel ahead of it in the stream has completed; while
 *     it waits for that it may already ask L2 to prefetch the input rows it was given (a hint
 *     by address, no data is consumed). Every input pointer must therefore be a mapped device
 *     address when the call is made, as any kernel argument must; its contents may still be
 *     produced by earlier work in the stream.
 *   - In-place use is allowed wherever the reference kernel works in place.
 *   - Buffers that are 16-byte aligned with row lengths that are multiples of 8
 *     elements take the vector kernels; anything else takes a slower scalar
 *     kernel with results inside the same tolerances. Q8 outputs need cols % 32 == 0.
 *   - No CPU fallback exists: without a CUDA device every call fails.
 *   - Thread-compatible: concurrent calls on different streams are fine (the noalloc
 *     entry point excepted, see there).
 *
 * Numerics: fp32 arithmetic in the evaluation order of the CPU operators
 * (src/model/cpu_ops.cpp), multiplies and adds rounded separately (-fmad=false), with
 * these deliberate departures, each far inside the 1e-5 relative the path allows:
 *   - sums of squares are accumulated in fp32 with fused multiply-adds (the CPU sums in
 *     double), and the norm scale is the hardware rsqrt (2 ulp) of fma(ss, 1/d, eps) or
 *     of ss + eps (L2 norm) instead of 1 / sqrtf;
 *   - SiLU and sigmoid gates use the hardware exp2 and reciprocal (ex2.approx.ftz,
 *     rcp.approx.ftz; relative error about 1e-6; a gate whose exact value is subnormal
 *     comes out as zero); the scatter weights of the hyper-connection ops, which scale
 *     whole rows, use expf and a true division;
 *   - RoPE angles are float(pos) * inv_freq with inv_freq computed on the host by the CPU
 *     operator's own pow(), and cos / sin by the device's full-range sincosf.
 * Bit-exact by construction: residual sums (one add, one rounding), Q8_0 dequantisation
 * (fp16 scale x int8, exact in fp32), position selection, copies and conversions, and the
 * Q8 encoders: their scales amax / 127 and codes rint(x / d) are the IEEE results,
 * obtained without dividing (two fused multiply-adds correct x * (1/127) to the exactly
 * rounded quotient for every finite x; codes come from x * rcp(d) and are redone with a
 * true division for the values, about 1 in 5000, that land within 1e-4 of a rounding
 * boundary). 16-bit outputs are rounded once from the fp32 result, to nearest even.
 */
#ifndef HALO_B200_H_
#define HALO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* halo_b200_stream; /* a cudaStream_t; NULL is the default stream */

enum halo_b200_dtype { HALO_B200_F32 = 0, HALO_B200_F16 = 1, HALO_B200_BF16 = 2 };

/* Version string of the library, e.g. "halo_b200 0.1 sm_100a". */
const char* halo_b200_version(void);

/* ---- group 1: residual add, RMSNorm, Q8 re-quantise ------------------------------ */

/* halo_add, src/kernels/core.hip:313-315: y[i] += x[i]. */
int halo_b200_add(halo_b200_stream stream, float* y, const float* x, uint32_t n, char* err, size_t errlen);
/* halo_axpy, src/kernels/core.hip:317-319: y[i] += a * x[i]. */
int halo_b200_axpy(halo_b200_stream stream, float* y, const float* x, float a, uint32_t n, char* err, size_t errlen);

/* halo_rmsnorm, src/kernels/core.hip:247-262: nvec vectors of length d (grid.x in the
 * reference); vector b uses gamma w_all + b * w_stride (0 = shared). x == y allowed. */
int halo_b200_rmsnorm(halo_b200_stream stream, const float* x, const float* w_all, float* y, uint32_t d, float eps,
                      uint32_t w_stride, uint32_t nvec, char* err, size_t errlen);
/* halo_rmsnorm_rows, src/kernels/core.hip:4045-4056: row r uses gamma (r % w_period) * w_stride.
 * _r16 / _rb (core.hip:4070-4077) read fp16 / bf16 rows and write fp32. rows = grid.x. */
int halo_b200_rmsnorm_rows(halo_b200_stream stream, const float* x, const float* w_all, float* y, uint32_t d,
                           float eps, uint32_t w_stride, uint32_t w_period, uint32_t rows, char* err, size_t errlen);
int halo_b200_rmsnorm_rows_r16(halo_b200_stream stream, const uint16_t* x, const float* w_all, float* y, uint32_t d,
                               float eps, uint32_t w_stride, uint32_t w_period, uint32_t rows, char* err,
                               size_t errlen);
int halo_b200_rmsnorm_rows_rb(halo_b200_stream stream, const uint16_t* x, const float* w_all, float* y, uint32_t d,
                              float eps, uint32_t w_stride, uint32_t w_period, uint32_t rows, char* err,
                              size_t errlen);
/* halo_rmsnorm_rows_h (+ _r16, _rb), src/kernels/core.hip:4502-4552: also writes an fp16
 * copy y16, row-major or (y16_tokens > 0) K-blocked [cols / 64][y16_tokens][64]. With iw
 * (irows <= 8 fp32 rows of w_period * d) it also writes the partial products
 * ipart[row * irows + r] = <y_row, iw[r][(row % w_period) d ..]>; that form needs w_stride == d and
 * rows % w_period == 0. x_dtype selects the variant. */
int halo_b200_rmsnorm_rows_h(halo_b200_stream stream, const void* x, int x_dtype, const float* w_all, float* y,
                             uint16_t* y16, uint32_t d, float eps, uint32_t w_stride, uint32_t w_period,
                             const float* iw, float* ipart, uint32_t irows, uint32_t y16_tokens, uint32_t rows,
                             char* err, size_t errlen);
/* halo_rmsnorm_y, src/kernels/batch_decode.hip:1685-1691: in place, entry e (grid.y) at
 * x + e * stride, nvec vectors (grid.x) per entry. */
int halo_b200_rmsnorm_y(halo_b200_stream stream, float* x, const float* w_all, uint32_t d, float eps,
                        uint32_t w_stride, uint32_t stride, uint32_t nvec, uint32_t batch, char* err, size_t errlen);

/* Typed RMSNorm: x_dtype rows in, y_dtype rows out, gamma = w or (one_plus) 1 + w, the
 * zero-centred form the GGUF converter folds into the stored weight
 * (src/model/qwen35.cpp:55-58). w may be NULL (raw scale). */
int halo_b200_rmsnorm_ex(halo_b200_stream stream, const void* x, int x_dtype, const float* w, void* y, int y_dtype,
                         uint32_t d, float eps, uint32_t w_stride, uint32_t w_period, int one_plus, uint32_t rows,
                         char* err, size_t errlen);

/* Fused residual add + RMSNorm with optional Q8 epilogues: one pass over
 *   res[r] += delta[r]            (stored back in res_dtype; the norm reads the stored value,
 *                                  as src/kernels/core.hip:4132-4135 does for 16-bit residuals)
 *   xn[r]   = res[r] * scale * g  (g = w or 1 + w; src/model/qwen35.cpp:319-329)
 * Outputs, each optional (NULL to skip) but at least one present: xn in xn_dtype; xn_q8_0 =
 * Q8_0 rows of the fp32 xn (d / 32 blocks of 34 bytes, src/core/lowbit.cpp:285-298); xq / xd =
 * int8 codes + fp32 scales per 32 values (src/kernels/core.hip:4160-4170), row-major.
 * This is the add + norm fusion of halo_hc_combine_norm_rows(_q8) (core.hip:4105-4238)
 * for a plain residual stream. delta NULL skips the add (res is then read only). */
int halo_b200_add_rmsnorm(halo_b200_stream stream, void* res, const void* delta, int res_dtype, const float* w,
                          int one_plus, void* xn, int xn_dtype, uint8_t* xn_q8_0, int8_t* xq, float* xd, uint32_t d,
                          float eps, uint32_t rows, char* err, size_t errlen);

/* halo_quantize_q8_rows, src/kernels/core.hip:3086-3101 (rows = grid.x). */
int halo_b200_quantize_q8_rows(halo_b200_stream stream, const float* x, int8_t* xq, float* xd, uint32_t cols,
                               uint32_t rows, char* err, size_t errlen);
/* halo_quantize_q8_kblocked, src/kernels/core.hip:3313-3331 (grid.x = tokens). */
int halo_b200_quantize_q8_kblocked(halo_b200_stream stream, const float* x, int8_t* xq, float* xd, uint32_t cols,
                                   uint32_t tokens, char* err, size_t errlen);
/* halo_q8x_cols, src/kernels/batch_decode.hip:197-222 (batch = grid.y); xq2 / xs2 may be NULL. */
int halo_b200_q8x_cols(halo_b200_stream stream, const float* x, uint32_t xstride, uint32_t cols, int8_t* xq,
                       float* xs, int8_t* xq2, float* xs2, uint32_t batch, char* err, size_t errlen);
/* halo_hc_norm_q8x, src/kernels/batch_decode.hip:977-999 (batch = grid.y): xn[b][i] = (res[b][i] * scale[b * hc + i / h])
 * norm_w[i] over the hc * h values of each column, stored, and quantized to two int8 levels per 32 values as by
 * halo_q8x_cols (xq2 / xs2 may be NULL: one level). */
int halo_b200_hc_norm_q8x(halo_b200_stream stream, const float* res, const float* scale, const float* norm_w,
                          float* xn, uint32_t hc, uint32_t h, int8_t* xq, float* xs, int8_t* xq2, float* xs2,
                          uint32_t batch, char* err, size_t errlen);
/* EncodeQ8_0, src/core/lowbit.cpp:285-298, as a device op over rows of x_dtype values. */
int halo_b200_encode_q8_0_rows(halo_b200_stream stream, const void* x, int x_dtype, uint8_t* out, uint32_t cols,
                               uint32_t rows, char* err, size_t errlen);

/* ---- group 2: L2 norm and gated RMSNorm -------------------------------------------- */

/* halo_l2norm, src/kernels/core.hip:264-273: in place, nvec vectors (grid.x). */
int halo_b200_l2norm(halo_b200_stream stream, float* x, uint32_t d, float eps, uint32_t nvec, char* err,
                     size_t errlen);
int halo_b200_l2norm_ex(halo_b200_stream stream, const void* x, int x_dtype, void* y, int y_dtype, uint32_t d,
                        float eps, uint32_t rows, char* err, size_t errlen);

/* halo_gated_norm, src/kernels/core.hip:495-510: in place on o, rows = grid.x heads. mode 0 =
 * SiLU(z) (src/model/qwen35.cpp:232-234), 1 = sigmoid(z) (src/model/reference.cpp:359-363). */
int halo_b200_gated_norm(halo_b200_stream stream, float* o, const float* w, const float* z, uint32_t d, float eps,
                         uint32_t mode, uint32_t rows, char* err, size_t errlen);
/* halo_gated_norm_h / _hz, src/kernels/core.hip:4554-4585: fp16 output only; _hz reads fp16 z. */
int halo_b200_gated_norm_h(halo_b200_stream stream, const float* o, const float* w, const float* z, uint16_t* y16,
                           uint32_t d, float eps, uint32_t mode, uint32_t rows, char* err, size_t errlen);
int halo_b200_gated_norm_hz(halo_b200_stream stream, const float* o, const float* w, const uint16_t* z,
                            uint16_t* y16, uint32_t d, float eps, uint32_t mode, uint32_t rows, char* err,
                            size_t errlen);
/* halo_gated_norm_h128w / _h128w_hh, src/kernels/core.hip:4587-4632: d = 128, rows is a parameter. */
int halo_b200_gated_norm_h128w(halo_b200_stream stream, const float* o, const float* w, const float* z,
                               uint16_t* y16, uint32_t rows, float eps, uint32_t mode, char* err, size_t errlen);
int halo_b200_gated_norm_h128w_hh(halo_b200_stream stream, const uint16_t* o, const float* w, const uint16_t* z,
                                  uint16_t* y16, uint32_t rows, float eps, uint32_t mode, char* err, size_t errlen);
/* Typed form. Supported (o, z, y) dtypes: (f32,f32,f32|f16|bf16), (f32,f16,f16), (f16,f16,f16),
 * (bf16,bf16,bf16|f32). y may alias o when the dtypes match. */
int halo_b200_gated_norm_ex(halo_b200_stream stream, const void* o, int o_dtype, const float* w, const void* z,
                            int z_dtype, void* y, int y_dtype, uint32_t d, float eps, uint32_t mode, uint32_t rows,
                            char* err, size_t errlen);

/* ---- group 3: partial rotary embedding (NEOX pairs i, i + rot/2) ------------------- */

/* halo_rope_neox, src/kernels/core.hip:289-292: heads = grid.x, all at position pos. */
int halo_b200_rope_neox(halo_b200_stream stream, float* x, uint32_t head_dim, uint32_t rotary_dim, uint32_t pos,
                        float theta, uint32_t heads, char* err, size_t errlen);
/* halo_rope_neox_rows, src/kernels/core.hip:293-298: rows = grid.x = T * heads, token t at pos0 + t. */
int halo_b200_rope_neox_rows(halo_b200_stream stream, float* x, uint32_t head_dim, uint32_t rotary_dim,
                             uint32_t pos0, uint32_t heads, float theta, uint32_t rows, char* err, size_t errlen);
/* halo_rope_neox_p, src/kernels/core.hip:299-304: position params[slot] * scale read on the device. */
int halo_b200_rope_neox_p(halo_b200_stream stream, float* x, const uint32_t* params, uint32_t head_dim,
                          uint32_t rotary_dim, uint32_t slot, uint32_t scale, float theta, uint32_t heads, char* err,
                          size_t errlen);
/* halo_rope_neox_blocks, src/kernels/core.hip:306-311: block b (grid.x) at (b0 + b) * ratio. */
int halo_b200_rope_neox_blocks(halo_b200_stream stream, float* x, uint32_t head_dim, uint32_t rotary_dim,
                               uint32_t b0, uint32_t ratio, float theta, uint32_t nblocks, char* err, size_t errlen);
/* halo_rope_neox_p_y, src/kernels/batch_decode.hip:1693-1697: entry e (grid.y) at x + e * stride
 * with params + e * pstride. */
int halo_b200_rope_neox_p_y(halo_b200_stream stream, float* x, const uint32_t* params, uint32_t head_dim,
                            uint32_t rotary_dim, uint32_t slot, uint32_t scale, float theta, uint32_t stride,
                            uint32_t pstride, uint32_t heads, uint32_t batch, char* err, size_t errlen);
/* Typed form rotating Q [tokens][q_heads][hd] and (optionally, k may be NULL) K
 * [tokens][k_heads][hd] in one launch. Token t rotates at
 * (params ? params[t * pstride + slot] : pos0 + t) * scale. pos_out (optional, [tokens])
 * receives the position each token used. rotary_dim <= 256. */
int halo_b200_rope_ex(halo_b200_stream stream, void* q, uint32_t q_heads, void* k, uint32_t k_heads, int dtype,
                      uint32_t head_dim, uint32_t rotary_dim, float theta, uint32_t tokens, const uint32_t* params,
                      uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale, uint32_t* pos_out, char* err,
                      size_t errlen);

/* halo_split_qgate, src/kernels/core.hip:356-366 (rows = grid.x), and halo_split_qgate_y,
 * src/kernels/batch_decode.hip:1680-1684 (heads = grid.x, batch = grid.y). */
int halo_b200_split_qgate(halo_b200_stream stream, const float* qg, float* q, float* gate, uint32_t hd,
                          uint32_t rows, char* err, size_t errlen);
int halo_b200_split_qgate_y(halo_b200_stream stream, const float* qg, float* q, float* gate, uint32_t hd,
                            uint32_t qg_stride, uint32_t q_stride, uint32_t heads, uint32_t batch, char* err,
                            size_t errlen);
/* halo_split_qgate_norm_rope, src/kernels/core.hip:368-405: hd is the reference's block size,
 * rows = grid.x = T * heads; gate may be NULL. */
int halo_b200_split_qgate_norm_rope(halo_b200_stream stream, const float* qg, float* q, float* gate, const float* w,
                                    float eps, uint32_t rotary_dim, uint32_t pos0, uint32_t heads, float theta,
                                    uint32_t hd, uint32_t rows, char* err, size_t errlen);
/* halo_norm_rope_rows, src/kernels/core.hip:407-443: in place, d <= 256, cache may be NULL. */
int halo_b200_norm_rope_rows(halo_b200_stream stream, float* x, const float* w, float eps, uint32_t d,
                             uint32_t rotary_dim, uint32_t pos0, uint32_t heads, float theta, float* cache,
                             uint32_t rows, char* err, size_t errlen);
/* Typed fused per-head RMSNorm + RoPE. in rows are in_row_stride elements apart (d, or 2 * d
 * for interleaved q|gate rows, whose second half is copied to `gate` when given); out may alias
 * in when in_row_stride == d. w NULL skips the norm. d <= 256 and a multiple of 8. */
int halo_b200_norm_rope_ex(halo_b200_stream stream, const void* in, int in_dtype, uint64_t in_row_stride, void* out,
                           int out_dtype, void* gate, void* cache, const float* w, int one_plus, float eps,
                           uint32_t d, uint32_t rotary_dim, uint32_t heads, uint32_t rows, float theta,
                           const uint32_t* params, uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale,
                           uint32_t* pos_out, char* err, size_t errlen);

/* Q and K of one attention layer in ONE launch: per-head RMSNorm (gammas w_q / w_k, or 1 + w) and
 * RoPE at the same positions, the sequence of src/model/qwen35.cpp:251-255. Q rows
 * [tokens * q_heads] are q_row_stride elements apart in q_in (d, or 2 * d with the gate halves
 * copied to q_gate); K rows [tokens * k_heads][d] may also be appended to k_cache. Outputs may
 * alias inputs (q_row_stride == d). The small K tensor stops paying a launch of its own and
 * the (cos, sin) tables are computed once for both. */
int halo_b200_norm_rope_qk_ex(halo_b200_stream stream, const void* q_in, uint64_t q_row_stride, void* q_out,
                              void* q_gate, const float* w_q, uint32_t q_heads, const void* k_in, void* k_out,
                              void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype, int out_dtype,
                              int one_plus, float eps, uint32_t d, uint32_t rotary_dim, uint32_t tokens, float theta,
                              const uint32_t* params, uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale,
                              uint32_t* pos_out, char* err, size_t errlen);

/* The rotation table of one step: table[t][0][i] = cos, table[t][1][i] = sin of
 * float(pos_t) * pow(theta, -2 i / rotary_dim), i < rotary_dim / 2 - the angle, cosf and sinf that
 * RopeNeox (src/kernels/core.hip:275-288) evaluates per head and element - as tokens * rotary_dim
 * floats, 16-byte aligned, caller-owned. Positions as in halo_b200_rope_ex. Every attention layer of a step rotates at
 * the same positions, so the table is computed once and shared by all of them. */
int halo_b200_rope_table_ex(halo_b200_stream stream, float* table, uint32_t tokens, uint32_t rotary_dim, float theta,
                            const uint32_t* params, uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale,
                            uint32_t* pos_out, char* err, size_t errlen);
/* halo_b200_norm_rope_qk_ex (src/kernels/core.hip:368-443 for Q and K of one layer) reading
 * (cos, sin) from a table made by halo_b200_rope_table_ex instead of computing them: same results bit for bit, no sincosf, shared memory or barrier in the kernel.
 * k_heads may be 0 (Q only). */
int halo_b200_norm_rope_qk_table_ex(halo_b200_stream stream, const void* q_in, uint64_t q_row_stride, void* q_out,
                                    void* q_gate, const float* w_q, uint32_t q_heads, const void* k_in, void* k_out,
                                    void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype, int out_dtype,
                                    int one_plus, float eps, uint32_t d, uint32_t rotary_dim, uint32_t tokens,
                                    const float* table, char* err, size_t errlen);

/* No counterpart in the reference. halo_b200_norm_rope_qk_ex for callers that cannot allocate
 * device memory and have no buffer to lend for the rotation table: an engine that committed and
 * accounts for all of its device memory at load time, a serving loop that cannot afford cudaMalloc's
 * device-wide synchronisation, a host that forbids allocation after start-up. Same arguments and
 * results (bit for bit) as halo_b200_norm_rope_qk_ex; the rotation table lives in a fixed 4 MiB
 * array inside the library (on every GPU that loads it, until exit) and nothing is allocated.
 * Limits: tokens * rotary_dim <= 1048576, otherwise -1 with a message. Every call shares that
 * array: calls on one stream are ordered, calls whose kernels overlap on the GPU race. The first
 * call on each device resolves the array's address and must be made outside stream capture. */
int halo_b200_norm_rope_qk_noalloc(halo_b200_stream stream, const void* q_in, uint64_t q_row_stride, void* q_out,
                                   void* q_gate, const float* w_q, uint32_t q_heads, const void* k_in, void* k_out,
                                   void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype, int out_dtype,
                                   int one_plus, float eps, uint32_t d, uint32_t rotary_dim, uint32_t tokens,
                                   float theta, const uint32_t* params, uint32_t pstride, uint32_t slot,
                                   uint32_t pos0, uint32_t scale, uint32_t* pos_out, char* err, size_t errlen);

/* ---- group 4: SwiGLU ----------------------------------------------------------------- */

/* halo_silu_mul, src/kernels/core.hip:321-325: g = SiLU(g) * up. */
int halo_b200_silu_mul(halo_b200_stream stream, float* g, const float* up, uint32_t n, char* err, size_t errlen);
/* halo_silu_mul_h, src/kernels/core.hip:326-333: fp16 output only. */
int halo_b200_silu_mul_h(halo_b200_stream stream, const float* g, const float* up, uint16_t* y, uint32_t n, char* err,
                         size_t errlen);
/* Typed form over n elements (rows x ff flattened; routed-expert rows are (token, slot) pairs,
 * pair = t * k + slot, src/kernels/core.hip:4718-4722). (in, y) dtypes: (f32, f32|f16|bf16),
 * (f16,f16), (bf16, bf16|f32). y may alias g when the dtypes match. */
int halo_b200_silu_mul_ex(halo_b200_stream stream, const void* g, const void* up, int in_dtype, void* y, int y_dtype,
                          uint64_t n, char* err, size_t errlen);
/* The same op over up to 4 independent tensors in ONE launch (e.g. the shared-expert rows [T x ff]
 * and the routed-expert rows [T*k x ff] of a MoE layer, which the reference computes in two GEMM
 * epilogues, src/kernels/core.hip:2937, 5257). g, up, y, n are HOST arrays of nseg entries, read
 * at call time; small tensors stop paying a launch of their own. */
int halo_b200_silu_mul_multi_ex(halo_b200_stream stream, uint32_t nseg, const void* const* g, const void* const* up,
                                void* const* y, const uint64_t* n, int in_dtype, int y_dtype, char* err,
                                size_t errlen);
/* halo_sigmoid_gate, src/kernels/core.hip:335-339: x *= sigmoid(gate). */
int halo_b200_sigmoid_gate(halo_b200_stream stream, float* x, const float* gate, uint32_t n, char* err,
                           size_t errlen);

/* ---- group 5: token-embedding gather with Q8_0 dequant -------------------------------- */

/* halo_matvec_q8_0_embed, _embed_p, _embed_rows, src/kernels/core.hip:200-232. _embed_p reads the
 * token from params[kHaloToken] (slot 0, src/kernels/step_params.h:7-8); _embed_rows reads token t
 * from params[t * 16 + kHaloToken] and writes row t (tokens = grid.y). fp32 output. */
int halo_b200_matvec_q8_0_embed(halo_b200_stream stream, const uint8_t* w, float* out, uint32_t token, uint32_t cols,
                                uint64_t row_bytes, char* err, size_t errlen);
int halo_b200_matvec_q8_0_embed_p(halo_b200_stream stream, const uint8_t* w, float* out, const uint32_t* params,
                                  uint32_t cols, uint64_t row_bytes, char* err, size_t errlen);
int halo_b200_matvec_q8_0_embed_rows(halo_b200_stream stream, const uint8_t* w, float* out, const uint32_t* params,
                                     uint32_t cols, uint64_t row_bytes, uint32_t tokens, char* err, size_t errlen);
/* Typed form: token t from ids[t * id_stride + id_slot], out in out_dtype. vocab > 0 guards the
 * gather: an id >= vocab yields a zero row instead of an out-of-range read. */
int halo_b200_embed_q8_0_ex(halo_b200_stream stream, const uint8_t* w, uint64_t row_bytes, uint32_t vocab,
                            const uint32_t* ids, uint32_t id_stride, uint32_t id_slot, uint32_t tokens, void* out,
                            int out_dtype, uint32_t cols, char* err, size_t errlen);

/* ---- hyper-connection residual (Flash-Next: hc streams of h values per token) ----------------- */

/* halo_hc_combine_norm_rows (+ _r16, _rb: res_dtype), src/kernels/core.hip:4105-4230; CPU operators
 * HcCombine + GroupedNorm, src/model/reference.cpp:151-202. Per (token t, stream s) row:
 * res += out[t] * 2 sigmoid(inject[t][s] / hc), stored in res' type; y = RMSNorm of the stored row with
 * gamma w_all[s]; optional fp16 copy y16 (row-major, or K-blocked [hc h / 64][y16_tokens][64] when
 * y16_tokens > 0), optional row scales rscale[t hc + s], optional partial products
 * ipart[(t hc + s) irows + r] = <y, iw[r][s h ..]> (irows <= 8). y may be NULL. rows = grid.x = tokens * hc. */
int halo_b200_hc_combine_norm_rows(halo_b200_stream stream, void* res, int res_dtype, const float* out,
                                   const float* inject, const float* w_all, float* y, uint16_t* y16, uint32_t hc,
                                   uint32_t h, float eps, const float* iw, float* ipart, uint32_t irows,
                                   float* rscale, uint32_t y16_tokens, uint32_t rows, char* err, size_t errlen);
/* halo_hc_combine_norm_rows_q8, src/kernels/core.hip:4231-4238: also the K-blocked int8 copy
 * yq [hc h / 64][y16_tokens][64] with fp32 scales yd [hc h / 32][y16_tokens] (amax / 127, round to even). */
int halo_b200_hc_combine_norm_rows_q8(halo_b200_stream stream, float* res, const float* out, const float* inject,
                                      const float* w_all, float* y, uint16_t* y16, uint32_t hc, uint32_t h, float eps,
                                      const float* iw, float* ipart, uint32_t irows, float* rscale,
                                      uint32_t y16_tokens, int8_t* yq, float* yd, uint32_t rows, char* err,
                                      size_t errlen);
/* halo_hc_combine_norm_tok (+ _r16, _rb), src/kernels/core.hip:4240-4435: hc = 4, one launch unit per
 * token, no fp32 y. tokens = grid.x. */
int halo_b200_hc_combine_norm_tok(halo_b200_stream stream, void* res, int res_dtype, const float* out,
                                  const float* inject, const float* w_all, uint16_t* y16, uint32_t h, float eps,
                                  const float* iw, float* ipart, uint32_t irows, float* rscale, uint32_t y16_tokens,
                                  uint32_t tokens, char* err, size_t errlen);
/* halo_hc_combine_norm_tok_moe and _moev (+ _r16, _rb), src/kernels/core.hip:4437-4485: the block output
 * is built in the kernel as halo_moe_combine_shared builds it (core.hip:5466-5480; CPU operator
 * src/model/reference.cpp:558-578): out[t] = sum over slots, in order, of mw[t k + s] * yp[pos[t k + s]]
 * (fp16 rows), then + sigmoid(sg[t]) * sx[t]. */
int halo_b200_hc_combine_norm_tok_moe(halo_b200_stream stream, void* res, int res_dtype, const uint16_t* yp,
                                      const uint32_t* pos, const float* mw, const float* sx, const float* sg,
                                      uint32_t k, const float* inject, const float* w_all, uint16_t* y16, uint32_t h,
                                      float eps, const float* iw, float* ipart, uint32_t irows, float* rscale,
                                      uint32_t y16_tokens, uint32_t tokens, char* err, size_t errlen);
/* Typed forms of the two above (the arithmetic of src/kernels/core.hip:4105-4230): block output and y in
 * fp32, fp16 or bf16 (supported (res, out, y) triples: (any, f32 | f16, f32), (bf16, bf16, bf16),
 * (f16, f16, f16)), gamma w or 1 + w, any hc. inject == NULL and out == NULL: grouped norm only, res is
 * read and not written. */
int halo_b200_hc_combine_norm_ex(halo_b200_stream stream, void* res, int res_dtype, const void* out, int out_dtype,
                                 const float* inject, const float* w_all, int one_plus, void* y, int y_dtype,
                                 uint16_t* y16, uint32_t y16_tokens, float* rscale, const float* iw, float* ipart,
                                 uint32_t irows, int8_t* yq, float* yd, uint32_t hc, uint32_t h, float eps,
                                 uint32_t tokens, char* err, size_t errlen);
int halo_b200_hc_combine_norm_moe_ex(halo_b200_stream stream, void* res, int res_dtype, const void* yp, int yp_dtype,
                                     const uint32_t* pos, const float* mw, const void* sx, int sx_dtype,
                                     const float* sg, uint32_t k, const float* inject, const float* w_all,
                                     int one_plus, void* y, int y_dtype, uint16_t* y16, uint32_t y16_tokens,
                                     float* rscale, const float* iw, float* ipart, uint32_t irows, uint32_t hc,
                                     uint32_t h, float eps, uint32_t tokens, char* err, size_t errlen);
/* halo_hc_combine and halo_hc_combine_rows (+ _r16, _rb), src/kernels/core.hip:610-617, 4649-4673:
 * res [tokens][hc][h] += out [tokens][h] * 2 sigmoid(inject [tokens][hc] / hc). */
int halo_b200_hc_combine_rows(halo_b200_stream stream, void* res, int res_dtype, const float* out, const float* inject,
                              uint32_t hc, uint32_t h, uint32_t tokens, char* err, size_t errlen);
int halo_b200_hc_combine_rows_ex(halo_b200_stream stream, void* res, int res_dtype, const void* out, int out_dtype,
                                 const float* inject, uint32_t hc, uint32_t h, uint32_t tokens, char* err,
                                 size_t errlen);
/* halo_broadcast and halo_broadcast_rows (+ _r16, _rb), src/kernels/core.hip:619-623, 4675-4697:
 * res [tokens][hc][h] = x [tokens][h]. */
int halo_b200_broadcast_rows(halo_b200_stream stream, void* res, int res_dtype, const float* x, uint32_t hc,
                             uint32_t h, uint32_t tokens, char* err, size_t errlen);
int halo_b200_broadcast_rows_ex(halo_b200_stream stream, void* res, int res_dtype, const void* x, int x_dtype,
                                uint32_t hc, uint32_t h, uint32_t tokens, char* err, size_t errlen);
/* halo_hc_mix and halo_hc_mix_rows, src/kernels/core.hip:600-608, 4634-4647; CPU operator
 * src/model/reference.cpp:179-188: mixed[t][i] = (sum over s of xn[t][s][i] * sigmoid(gate[t][s][i])) / hc. */
int halo_b200_hc_mix_rows(halo_b200_stream stream, const float* xn, const float* gate, float* mixed, uint32_t hc,
                          uint32_t h, uint32_t tokens, char* err, size_t errlen);
int halo_b200_hc_mix_rows_ex(halo_b200_stream stream, const void* xn, const void* gate, void* mixed, int dtype,
                             uint32_t hc, uint32_t h, uint32_t tokens, char* err, size_t errlen);
/* halo_axpy_sigmoid and halo_axpy_sigmoid_rows, src/kernels/core.hip:1129-1133, 4707-4714:
 * y [tokens][n] += sigmoid(g [tokens]) * x [tokens][n] (the shared expert's gated add). */
int halo_b200_axpy_sigmoid_rows(halo_b200_stream stream, float* y, const float* x, const float* g, uint32_t n,
                                uint32_t tokens, char* err, size_t errlen);
/* halo_inject_reduce, src/kernels/core.hip:4486-4496: inject[t][r] = sum over streams, in order, of
 * ipart[(t hc + s) irows + r]. */
int halo_b200_inject_reduce(halo_b200_stream stream, const float* ipart, float* inject, uint32_t hc, uint32_t irows,
                            uint32_t tokens, char* err, size_t errlen);
/* halo_res_to_f32_r16 and _rb, src/kernels/core.hip:4698-4705: y[i] = float(x[i]). */
int halo_b200_res_to_f32(halo_b200_stream stream, float* y, const void* x, int x_dtype, uint32_t n, char* err,
                         size_t errlen);
/* halo_hc_norm_scales and _u, src/kernels/core.hip:2768-2776, 9383-9400: scale[row] = 1 / sqrt(mean(res_row^2) + eps). */
int halo_b200_hc_norm_scales(halo_b200_stream stream, const float* res, float* scale, uint32_t h, float eps,
                             uint32_t rows, char* err, size_t errlen);

/* ---- Gated DeltaNet causal conv + SiLU + per-head L2 norm ---------------------------------------- */

/* halo_conv_l2norm_prefill, src/kernels/core.hip:3486-3509; CPU operator Qwen35Reference::Linear,
 * src/model/qwen35.cpp:180-198. in, out [tokens][channels]; out[t][ch] = SiLU(w[ch][kern-1] in[t][ch] +
 * sum over k < kern-1 of w[ch][k] x(t - (kern-1) + k)), inputs before the chunk taken from the conv state
 * [kern-1][channels] (oldest first; NULL = zeros); the first l2_channels channels are then L2-normalized per
 * head of d channels (x / sqrt(sum x^2 + eps)). The state is not written. d = block.x, tokens = grid.y.
 * in and out must be different buffers. */
int halo_b200_conv_l2norm_prefill(halo_b200_stream stream, const float* in, const float* state, const float* w,
                                  float* out, uint32_t channels, uint32_t kern, uint32_t l2_channels, float eps,
                                  uint32_t d, uint32_t tokens, char* err, size_t errlen);
/* halo_conv_l2norm_prefill8 (+ _h: fp16 in, _hh: fp16 in and out), src/kernels/core.hip:3511-3576: kern = 4. */
int halo_b200_conv_l2norm_prefill8(halo_b200_stream stream, const void* in, int in_dtype, const float* state,
                                   const float* w, void* out, int out_dtype, uint32_t channels, uint32_t tokens,
                                   uint32_t l2_channels, float eps, uint32_t d, char* err, size_t errlen);
/* Typed form of the two above: (in, out) in (f32, f32), (f16, f32), (f16, f16), (bf16, bf16), (bf16, f32). */
int halo_b200_conv_l2norm_ex(halo_b200_stream stream, const void* in, int in_dtype, const float* state, const float* w,
                             void* out, int out_dtype, uint32_t channels, uint32_t kern, uint32_t l2_channels,
                             uint32_t d, float eps, uint32_t tokens, char* err, size_t errlen);
/* halo_conv_state_advance (+ _h), src/kernels/core.hip:3578-3611: the state after a chunk of `tokens`
 * inputs = its last kern - 1 inputs (older rows from the previous state when the chunk is shorter). */
int halo_b200_conv_state_advance(halo_b200_stream stream, const void* in, int in_dtype, float* state,
                                 uint32_t channels, uint32_t kern, uint32_t tokens, char* err, size_t errlen);
/* halo_conv_l2norm, src/kernels/core.hip:3002-3028: one decode step (conv of one token, then the state
 * shifts by it), in one launch. d = block.x; in and out may be the same buffer. */
int halo_b200_conv_l2norm(halo_b200_stream stream, const float* in, float* state, const float* w, float* out,
                          uint32_t channels, uint32_t kern, uint32_t l2_channels, float eps, uint32_t d, char* err,
                          size_t errlen);
/* halo_conv_l2norm_y, src/kernels/batch_decode.hip:1741-1748: the same step for `entries` (= grid.y) sessions in
 * one launch. Entry e reads in + e * stride, writes out + e * stride (floats), and owns the conv state whose
 * device address is tab[e * tstride + tslot] (a table of 64-bit device addresses in device memory). */
int halo_b200_conv_l2norm_y(halo_b200_stream stream, const float* in, const uint64_t* tab, uint32_t tstride,
                            uint32_t tslot, const float* w, float* out, uint32_t channels, uint32_t kern,
                            uint32_t l2_channels, float eps, uint32_t stride, uint32_t d, uint32_t entries, char* err,
                            size_t errlen);
/* halo_conv_step, src/kernels/core.hip:445-456: the same without the L2 norm. */
int halo_b200_conv_step(halo_b200_stream stream, const float* in, float* state, const float* w, float* out,
                        uint32_t channels, uint32_t kern, char* err, size_t errlen);

/* No counterpart in the reference. The persistent kernels of the library (the conv + SiLU + L2 norm and the fused
 * norm + RoPE at streaming sizes) stage their input rows in shared memory with bulk asynchronous copies and wait
 * for them on a barrier object for a bounded time (about a second); a CTA whose wait ran out (never
 * observed) returns without writing its remaining output tiles and is counted. halo_b200_stage_timeouts reads the
 * count (this call synchronizes the device). A non-zero count means the outputs of the calls made before it are
 * invalid. halo_b200_conv_stage_timeouts is the same call under its earlier name. */
int halo_b200_stage_timeouts(unsigned int* count, char* err, size_t errlen);
int halo_b200_conv_stage_timeouts(unsigned int* count, char* err, size_t errlen);

/* ---- MoE combine (the step after the routed experts' down projections) --------------------------- */

/* halo_moe_combine_grouped, src/kernels/core.hip:5456-5464: out[t][i] = sum over slots s, in order, of
 * w[t k + s] * yp[pos[t k + s]][i] (yp: fp16 rows of the per-pair down projections). tokens = grid.y. */
int halo_b200_moe_combine_grouped(halo_b200_stream stream, const uint16_t* yp, const uint32_t* pos, const float* w,
                                  float* out, uint32_t k, uint32_t n, uint32_t tokens, char* err, size_t errlen);
/* halo_moe_combine_shared, src/kernels/core.hip:5466-5480 (CPU operator ReferenceModel::Moe,
 * src/model/reference.cpp:558-578): the same, then + sigmoid(g[t]) * x[t][i] (the gated shared expert). */
int halo_b200_moe_combine_shared(halo_b200_stream stream, const uint16_t* yp, const uint32_t* pos, const float* w,
                                 const float* x, const float* g, float* out, uint32_t k, uint32_t n, uint32_t tokens,
                                 char* err, size_t errlen);
/* halo_moe_combine and halo_moe_combine_u, src/kernels/core.hip:2372-2380, 9401-9420: one token,
 * out[i] = sum over slots of weights[s] * part[s][i] (fp32 rows). */
int halo_b200_moe_combine(halo_b200_stream stream, const float* part, const float* weights, float* out, uint32_t slots,
                          uint32_t n, char* err, size_t errlen);
/* halo_axpy_slot, src/kernels/core.hip:1123-1127: y += weights[slot] * x. */
int halo_b200_axpy_slot(halo_b200_stream stream, float* y, const float* x, const float* weights, uint32_t slot,
                        uint32_t n, char* err, size_t errlen);
/* Typed form: (yp, out) in (f16, f32), (f32, f32), (bf16, bf16), (bf16, f32), (f16, f16); sx (may be NULL, with
 * sg) fp32 or of yp's type; pos == NULL: slot s of token t is row t k + s of yp. */
int halo_b200_moe_combine_ex(halo_b200_stream stream, const void* yp, int yp_dtype, const uint32_t* pos, const float* mw,
                             const void* sx, int sx_dtype, const float* sg, void* out, int out_dtype, uint32_t k,
                             uint32_t n, uint32_t tokens, char* err, size_t errlen);

/* ---- row copies and conversions around the attention block --------------------------------------- */

/* halo_copy_at and halo_copy_at_h, src/kernels/core.hip:341-350, 921-927: dst[params[slot] * stride + i] =
 * src[i] (appends one row to a K/V cache at a position read from device memory); dst fp32, or fp16 / bf16
 * rounded to nearest even. */
int halo_b200_copy_at(halo_b200_stream stream, void* dst, int dst_dtype, const float* src, const uint32_t* params,
                      uint32_t slot, uint32_t stride, uint32_t n, char* err, size_t errlen);
/* halo_copy_at_y, src/kernels/batch_decode.hip:1700-1707: the row append for `entries` (= grid.y) sessions in one
 * launch. Entry e copies src[e * src_stride ..+ n] to row params[e * pstride + slot] (rows `stride` elements apart)
 * of the buffer whose device address is tab[e * tstride + tslot]; the buffers hold dst_dtype elements. */
int halo_b200_copy_at_y(halo_b200_stream stream, const uint64_t* tab, uint32_t tstride, uint32_t tslot, int dst_dtype,
                        const float* src, const uint32_t* params, uint32_t slot, uint32_t stride, uint32_t n,
                        uint32_t src_stride, uint32_t pstride, uint32_t entries, char* err, size_t errlen);
/* halo_copy, src/kernels/core.hip:352-354. */
int halo_b200_copy(halo_b200_stream stream, float* dst, const float* src, uint32_t n, char* err, size_t errlen);
/* halo_f16_rows, src/kernels/core.hip:8157-8161: y[i] = fp16(x[i]). */
int halo_b200_f16_rows(halo_b200_stream stream, const float* x, uint16_t* y, uint32_t n, char* err, size_t errlen);
/* halo_scale_silu and halo_scale_silu_h, src/kernels/core.hip:586-598: y = SiLU(x * scale), y fp32 (may be x)
 * or fp16 (the hyper-connection mixer's silu(down(xn) / hc), src/model/reference.cpp:172-174). */
int halo_b200_scale_silu(halo_b200_stream stream, const float* x, void* y, int y_dtype, float scale, uint32_t n,
                         char* err, size_t errlen);

/* ---- launch by kernel name -------------------------------------------------------------- */

/* One launch argument, as rt::Arg (src/rt/device.hpp:35-59): a device pointer (buffer base +
 * byte offset already added) or a by-value scalar of <= 8 bytes. A NULL optional pointer may be
 * passed either way (the engine passes Arg::Val<uint64_t>(0), src/engine/prefill_chunk.cpp:384). */
typedef struct halo_b200_arg {
  uint32_t is_buffer; /* 1: `ptr` is a device pointer; 0: scalar in `bytes` */
  uint32_t size;      /* scalar size in bytes (1..8); ignored for buffers */
  union {
    void* ptr;
    uint8_t bytes[8];
  } v;
} halo_b200_arg;

/* Runs the replacement of reference kernel `name` ("halo_rmsnorm_rows", ...) given the
 * reference's own launch: its argument list, grid and block. Row and batch counts are decoded
 * from `grid` exactly as the reference kernel reads blockIdx; `block` is only used where the
 * reference derives a size from it (halo_split_qgate_norm_rope: hd = block[0]). */
int halo_b200_launch(halo_b200_stream stream, const char* name, const halo_b200_arg* args, size_t nargs,
                     const uint32_t grid[3], const uint32_t block[3], char* err, size_t errlen);
/* Names halo_b200_launch accepts. */
size_t halo_b200_kernel_count(void);
const char* halo_b200_kernel_name(size_t index);

/* Tuning hook for experiments (process-wide host atomics read at call time; not for production dispatch). Keys:
 * "norm_threads_per_row" (power of two <= 256; 0 = built-in choice),
 * "norm_short_rows_k1" (1 = rows of <= 256 elements use one 8-element chunk per thread; 0 = built-in choice),
 * "norm_force_general" (1 = the row norms always run their general kernel, never the lean one),
 * "l2_keep" (1, the default = the add + norm stores a residual of at most 40 MB with an L2 evict_last hint; 0 = plain stores),
 * "embed_direct" (1, the default = embedding launches with more rows than resident warps read rows straight into
 * registers; 0 = every launch stages rows in shared memory),
 * "gated_rows_per_group" (1 or 2 rows in flight per thread group of the gated norm on short rows; 0 = built-in),
 * "rope_rows_per_group" (2 or 4 rows in flight per thread group of the general fused norm + RoPE kernel; 0 = built-in),
 * "rope_lean_k" (chunks per lane of the fused norm + RoPE kernels on rows of 256: 1 or 2; 0 = built-in, four),
 * "rope_staged" (1, the default = the lean fused norm + RoPE kernel at streaming sizes runs persistent CTAs that stage
 * rows in shared memory by bulk asynchronous copies; 0 = every CTA loads its rows directly),
 * "hc_row_level" (1 = the hyper-connection combine + norm always runs one (token, stream) row per thread group),
 * "conv_staged" (1, the default = the conv kernel stages rows in shared memory by bulk asynchronous copies; 0 = rows in registers),
 * "conv_tile" (tokens per thread of the register form of the conv kernel: 4 or 8; 0 = built-in), "hc_token_k" (2 = two
 * chunks per stream per thread in the token-level hyper-connection kernel where they fit),
 * "hc_fused_inject" (1 = the inject partial products are computed inside the combine kernel even where a second
 * pass over the normalized rows would do; 0 = built-in choice),
 * "pdl" (1, the default = kernels are launched with programmatic stream serialization, so a kernel is scheduled
 * while its predecessor in the stream drains and waits on the device for it to complete; 0 = plain launches).
 * Returns 0, or -1 for an unknown key or value. */
int halo_b200_tune(const char* key, int value);

#ifdef __cplusplus
}
#endif

#endif /* HALO_B200_H_ */
