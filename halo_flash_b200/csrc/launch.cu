// halo_b200_launch: the reference's launch-by-name call (rt::Device::Kernel + Launch,
// src/rt/device.hpp:120-127) mapped onto this library's typed entry points. Each
// handler unpacks the reference kernel's argument list in its declared order and
// recovers the row / batch counts from the grid exactly as the kernel reads
// blockIdx (src/kernels/core.hip, src/kernels/batch_decode.hip).
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/halo_b200.h"

namespace {

struct Reader {
  const halo_b200_arg* args;
  size_t n;
  size_t i = 0;
  bool bad = false;

  const halo_b200_arg* next() {
    if (i >= n) {
      bad = true;
      return nullptr;
    }
    return &args[i++];
  }
  template <typename T>
  T* ptr() {
    const halo_b200_arg* a = next();
    if (!a) return nullptr;
    if (a->is_buffer) return static_cast<T*>(a->v.ptr);
    // a null optional pointer passed as a 64-bit zero scalar
    uint64_t v = 0;
    if (a->size != 8) bad = true;
    std::memcpy(&v, a->v.bytes, 8);
    if (v != 0) bad = true;
    return nullptr;
  }
  template <typename T>
  T val() {
    const halo_b200_arg* a = next();
    T v{};
    if (!a) return v;
    if (a->is_buffer || a->size != sizeof(T)) {
      bad = true;
      return v;
    }
    std::memcpy(&v, a->v.bytes, sizeof(T));
    return v;
  }
  uint32_t u32() { return val<uint32_t>(); }
  uint64_t u64() { return val<uint64_t>(); }
  float f32() { return val<float>(); }
};

struct Ctx {
  halo_b200_stream s;
  const uint32_t* grid;
  const uint32_t* block;
  char* err;
  size_t errlen;
};

using Handler = int (*)(Reader&, const Ctx&);

int BadArgs(const Ctx& c, const char* name) {
  if (c.err && c.errlen) std::snprintf(c.err, c.errlen, "%s: argument list does not match the kernel's parameters", name);
  return -1;
}

#define HANDLER(fn) static int fn(Reader& r, const Ctx& c)
#define CHECK_ARGS(name) \
  if (r.bad || r.i != r.n) return BadArgs(c, name)

HANDLER(H_add) {
  auto* y = r.ptr<float>(); auto* x = r.ptr<const float>(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_add");
  return halo_b200_add(c.s, y, x, n, c.err, c.errlen);
}
HANDLER(H_axpy) {
  auto* y = r.ptr<float>(); auto* x = r.ptr<const float>(); const float a = r.f32(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_axpy");
  return halo_b200_axpy(c.s, y, x, a, n, c.err, c.errlen);
}
HANDLER(H_rmsnorm) {
  auto* x = r.ptr<const float>(); auto* w = r.ptr<const float>(); auto* y = r.ptr<float>();
  const uint32_t d = r.u32(); const float eps = r.f32(); const uint32_t ws = r.u32();
  CHECK_ARGS("halo_rmsnorm");
  return halo_b200_rmsnorm(c.s, x, w, y, d, eps, ws, c.grid[0], c.err, c.errlen);
}
template <int DT>
HANDLER(H_rmsnorm_rows) {
  auto* x = r.ptr<const void>(); auto* w = r.ptr<const float>(); auto* y = r.ptr<float>();
  const uint32_t d = r.u32(); const float eps = r.f32(); const uint32_t ws = r.u32(), wp = r.u32();
  CHECK_ARGS("halo_rmsnorm_rows");
  if (DT == HALO_B200_F32)
    return halo_b200_rmsnorm_rows(c.s, static_cast<const float*>(x), w, y, d, eps, ws, wp, c.grid[0], c.err, c.errlen);
  if (DT == HALO_B200_F16)
    return halo_b200_rmsnorm_rows_r16(c.s, static_cast<const uint16_t*>(x), w, y, d, eps, ws, wp, c.grid[0], c.err,
                                      c.errlen);
  return halo_b200_rmsnorm_rows_rb(c.s, static_cast<const uint16_t*>(x), w, y, d, eps, ws, wp, c.grid[0], c.err,
                                   c.errlen);
}
template <int DT>
HANDLER(H_rmsnorm_rows_h) {
  auto* x = r.ptr<const void>(); auto* w = r.ptr<const float>(); auto* y = r.ptr<float>();
  auto* y16 = r.ptr<uint16_t>();
  const uint32_t d = r.u32(); const float eps = r.f32(); const uint32_t ws = r.u32(), wp = r.u32();
  auto* iw = r.ptr<const float>(); auto* ipart = r.ptr<float>();
  const uint32_t irows = r.u32(), y16_tokens = r.u32();
  CHECK_ARGS("halo_rmsnorm_rows_h");
  return halo_b200_rmsnorm_rows_h(c.s, x, DT, w, y, y16, d, eps, ws, wp, iw, ipart, irows, y16_tokens, c.grid[0], c.err,
                                  c.errlen);
}
HANDLER(H_rmsnorm_y) {
  auto* x = r.ptr<float>(); auto* w = r.ptr<const float>();
  const uint32_t d = r.u32(); const float eps = r.f32(); const uint32_t ws = r.u32(), stride = r.u32();
  CHECK_ARGS("halo_rmsnorm_y");
  return halo_b200_rmsnorm_y(c.s, x, w, d, eps, ws, stride, c.grid[0], c.grid[1], c.err, c.errlen);
}
HANDLER(H_l2norm) {
  auto* x = r.ptr<float>(); const uint32_t d = r.u32(); const float eps = r.f32();
  CHECK_ARGS("halo_l2norm");
  return halo_b200_l2norm(c.s, x, d, eps, c.grid[0], c.err, c.errlen);
}
HANDLER(H_gated_norm) {
  auto* o = r.ptr<float>(); auto* w = r.ptr<const float>(); auto* z = r.ptr<const float>();
  const uint32_t d = r.u32(); const float eps = r.f32(); const uint32_t mode = r.u32();
  CHECK_ARGS("halo_gated_norm");
  return halo_b200_gated_norm(c.s, o, w, z, d, eps, mode, c.grid[0], c.err, c.errlen);
}
template <bool ZH>
HANDLER(H_gated_norm_h) {
  auto* o = r.ptr<const float>(); auto* w = r.ptr<const float>(); auto* z = r.ptr<const void>();
  auto* y16 = r.ptr<uint16_t>();
  const uint32_t d = r.u32(); const float eps = r.f32(); const uint32_t mode = r.u32();
  CHECK_ARGS("halo_gated_norm_h");
  if (ZH)
    return halo_b200_gated_norm_hz(c.s, o, w, static_cast<const uint16_t*>(z), y16, d, eps, mode, c.grid[0], c.err,
                                   c.errlen);
  return halo_b200_gated_norm_h(c.s, o, w, static_cast<const float*>(z), y16, d, eps, mode, c.grid[0], c.err, c.errlen);
}
template <bool HH>
HANDLER(H_gated_norm_h128w) {
  auto* o = r.ptr<const void>(); auto* w = r.ptr<const float>(); auto* z = r.ptr<const void>();
  auto* y16 = r.ptr<uint16_t>();
  const uint32_t rows = r.u32(); const float eps = r.f32(); const uint32_t mode = r.u32();
  CHECK_ARGS("halo_gated_norm_h128w");
  if (HH)
    return halo_b200_gated_norm_h128w_hh(c.s, static_cast<const uint16_t*>(o), w, static_cast<const uint16_t*>(z), y16,
                                         rows, eps, mode, c.err, c.errlen);
  return halo_b200_gated_norm_h128w(c.s, static_cast<const float*>(o), w, static_cast<const float*>(z), y16, rows, eps,
                                    mode, c.err, c.errlen);
}
HANDLER(H_rope_neox) {
  auto* x = r.ptr<float>(); const uint32_t hd = r.u32(), rot = r.u32(), pos = r.u32(); const float theta = r.f32();
  CHECK_ARGS("halo_rope_neox");
  return halo_b200_rope_neox(c.s, x, hd, rot, pos, theta, c.grid[0], c.err, c.errlen);
}
HANDLER(H_rope_neox_rows) {
  auto* x = r.ptr<float>(); const uint32_t hd = r.u32(), rot = r.u32(), pos0 = r.u32(), heads = r.u32();
  const float theta = r.f32();
  CHECK_ARGS("halo_rope_neox_rows");
  return halo_b200_rope_neox_rows(c.s, x, hd, rot, pos0, heads, theta, c.grid[0], c.err, c.errlen);
}
HANDLER(H_rope_neox_p) {
  auto* x = r.ptr<float>(); auto* params = r.ptr<const uint32_t>();
  const uint32_t hd = r.u32(), rot = r.u32(), slot = r.u32(), scale = r.u32(); const float theta = r.f32();
  CHECK_ARGS("halo_rope_neox_p");
  return halo_b200_rope_neox_p(c.s, x, params, hd, rot, slot, scale, theta, c.grid[0], c.err, c.errlen);
}
HANDLER(H_rope_neox_blocks) {
  auto* x = r.ptr<float>(); const uint32_t hd = r.u32(), rot = r.u32(), b0 = r.u32(), ratio = r.u32();
  const float theta = r.f32();
  CHECK_ARGS("halo_rope_neox_blocks");
  return halo_b200_rope_neox_blocks(c.s, x, hd, rot, b0, ratio, theta, c.grid[0], c.err, c.errlen);
}
HANDLER(H_rope_neox_p_y) {
  auto* x = r.ptr<float>(); auto* params = r.ptr<const uint32_t>();
  const uint32_t hd = r.u32(), rot = r.u32(), slot = r.u32(), scale = r.u32(); const float theta = r.f32();
  const uint32_t stride = r.u32(), pstride = r.u32();
  CHECK_ARGS("halo_rope_neox_p_y");
  return halo_b200_rope_neox_p_y(c.s, x, params, hd, rot, slot, scale, theta, stride, pstride, c.grid[0], c.grid[1],
                                 c.err, c.errlen);
}
HANDLER(H_split_qgate) {
  auto* qg = r.ptr<const float>(); auto* q = r.ptr<float>(); auto* gate = r.ptr<float>(); const uint32_t hd = r.u32();
  CHECK_ARGS("halo_split_qgate");
  return halo_b200_split_qgate(c.s, qg, q, gate, hd, c.grid[0], c.err, c.errlen);
}
HANDLER(H_split_qgate_y) {
  auto* qg = r.ptr<const float>(); auto* q = r.ptr<float>(); auto* gate = r.ptr<float>();
  const uint32_t hd = r.u32(), qs = r.u32(), os = r.u32();
  CHECK_ARGS("halo_split_qgate_y");
  return halo_b200_split_qgate_y(c.s, qg, q, gate, hd, qs, os, c.grid[0], c.grid[1], c.err, c.errlen);
}
HANDLER(H_split_qgate_norm_rope) {
  auto* qg = r.ptr<const float>(); auto* q = r.ptr<float>(); auto* gate = r.ptr<float>(); auto* w = r.ptr<const float>();
  const float eps = r.f32(); const uint32_t rot = r.u32(), pos0 = r.u32(), heads = r.u32(); const float theta = r.f32();
  CHECK_ARGS("halo_split_qgate_norm_rope");
  return halo_b200_split_qgate_norm_rope(c.s, qg, q, gate, w, eps, rot, pos0, heads, theta, c.block[0], c.grid[0], c.err,
                                         c.errlen);
}
HANDLER(H_norm_rope_rows) {
  auto* x = r.ptr<float>(); auto* w = r.ptr<const float>(); const float eps = r.f32();
  const uint32_t d = r.u32(), rot = r.u32(), pos0 = r.u32(), heads = r.u32(); const float theta = r.f32();
  auto* cache = r.ptr<float>();
  CHECK_ARGS("halo_norm_rope_rows");
  return halo_b200_norm_rope_rows(c.s, x, w, eps, d, rot, pos0, heads, theta, cache, c.grid[0], c.err, c.errlen);
}
HANDLER(H_silu_mul) {
  auto* g = r.ptr<float>(); auto* up = r.ptr<const float>(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_silu_mul");
  return halo_b200_silu_mul(c.s, g, up, n, c.err, c.errlen);
}
HANDLER(H_silu_mul_h) {
  auto* g = r.ptr<const float>(); auto* up = r.ptr<const float>(); auto* y = r.ptr<uint16_t>(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_silu_mul_h");
  return halo_b200_silu_mul_h(c.s, g, up, y, n, c.err, c.errlen);
}
HANDLER(H_sigmoid_gate) {
  auto* x = r.ptr<float>(); auto* gate = r.ptr<const float>(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_sigmoid_gate");
  return halo_b200_sigmoid_gate(c.s, x, gate, n, c.err, c.errlen);
}
HANDLER(H_quantize_q8_rows) {
  auto* x = r.ptr<const float>(); auto* xq = r.ptr<int8_t>(); auto* xd = r.ptr<float>(); const uint32_t cols = r.u32();
  CHECK_ARGS("halo_quantize_q8_rows");
  return halo_b200_quantize_q8_rows(c.s, x, xq, xd, cols, c.grid[0], c.err, c.errlen);
}
HANDLER(H_quantize_q8_kblocked) {
  auto* x = r.ptr<const float>(); auto* xq = r.ptr<int8_t>(); auto* xd = r.ptr<float>();
  const uint32_t cols = r.u32(), tokens = r.u32();
  CHECK_ARGS("halo_quantize_q8_kblocked");
  if (tokens != c.grid[0]) return BadArgs(c, "halo_quantize_q8_kblocked (tokens != grid.x)");
  return halo_b200_quantize_q8_kblocked(c.s, x, xq, xd, cols, tokens, c.err, c.errlen);
}
HANDLER(H_q8x_cols) {
  auto* x = r.ptr<const float>(); const uint32_t xstride = r.u32(), cols = r.u32();
  auto* xq = r.ptr<int8_t>(); auto* xs = r.ptr<float>(); auto* xq2 = r.ptr<int8_t>(); auto* xs2 = r.ptr<float>();
  CHECK_ARGS("halo_q8x_cols");
  return halo_b200_q8x_cols(c.s, x, xstride, cols, xq, xs, xq2, xs2, c.grid[1], c.err, c.errlen);
}
HANDLER(H_hc_norm_q8x) {
  auto* res = r.ptr<const float>(); auto* scale = r.ptr<const float>(); auto* nw = r.ptr<const float>();
  auto* xn = r.ptr<float>(); const uint32_t hc = r.u32(), h = r.u32();
  auto* xq = r.ptr<int8_t>(); auto* xs = r.ptr<float>(); auto* xq2 = r.ptr<int8_t>(); auto* xs2 = r.ptr<float>();
  CHECK_ARGS("halo_hc_norm_q8x");
  return halo_b200_hc_norm_q8x(c.s, res, scale, nw, xn, hc, h, xq, xs, xq2, xs2, c.grid[1], c.err, c.errlen);
}
HANDLER(H_embed) {
  auto* w = r.ptr<const uint8_t>(); auto* out = r.ptr<float>(); const uint32_t token = r.u32(), cols = r.u32();
  const uint64_t rb = r.u64();
  CHECK_ARGS("halo_matvec_q8_0_embed");
  return halo_b200_matvec_q8_0_embed(c.s, w, out, token, cols, rb, c.err, c.errlen);
}
HANDLER(H_embed_p) {
  auto* w = r.ptr<const uint8_t>(); auto* out = r.ptr<float>(); auto* params = r.ptr<const uint32_t>();
  const uint32_t cols = r.u32(); const uint64_t rb = r.u64();
  CHECK_ARGS("halo_matvec_q8_0_embed_p");
  return halo_b200_matvec_q8_0_embed_p(c.s, w, out, params, cols, rb, c.err, c.errlen);
}
HANDLER(H_embed_rows) {
  auto* w = r.ptr<const uint8_t>(); auto* out = r.ptr<float>(); auto* params = r.ptr<const uint32_t>();
  const uint32_t cols = r.u32(); const uint64_t rb = r.u64();
  CHECK_ARGS("halo_matvec_q8_0_embed_rows");
  return halo_b200_matvec_q8_0_embed_rows(c.s, w, out, params, cols, rb, c.grid[1], c.err, c.errlen);
}

template <int DT>
HANDLER(H_hc_combine_norm_rows) {
  auto* res = r.ptr<void>(); auto* out = r.ptr<const float>(); auto* inject = r.ptr<const float>();
  auto* w = r.ptr<const float>(); auto* y = r.ptr<float>(); auto* y16 = r.ptr<uint16_t>();
  const uint32_t hc = r.u32(), h = r.u32(); const float eps = r.f32();
  auto* iw = r.ptr<const float>(); auto* ipart = r.ptr<float>(); const uint32_t irows = r.u32();
  auto* rscale = r.ptr<float>(); const uint32_t y16_tokens = r.u32();
  CHECK_ARGS("halo_hc_combine_norm_rows");
  return halo_b200_hc_combine_norm_rows(c.s, res, DT, out, inject, w, y, y16, hc, h, eps, iw, ipart, irows, rscale,
                                        y16_tokens, c.grid[0], c.err, c.errlen);
}
HANDLER(H_hc_combine_norm_rows_q8) {
  auto* res = r.ptr<float>(); auto* out = r.ptr<const float>(); auto* inject = r.ptr<const float>();
  auto* w = r.ptr<const float>(); auto* y = r.ptr<float>(); auto* y16 = r.ptr<uint16_t>();
  const uint32_t hc = r.u32(), h = r.u32(); const float eps = r.f32();
  auto* iw = r.ptr<const float>(); auto* ipart = r.ptr<float>(); const uint32_t irows = r.u32();
  auto* rscale = r.ptr<float>(); const uint32_t y16_tokens = r.u32();
  auto* yq = r.ptr<int8_t>(); auto* yd = r.ptr<float>();
  CHECK_ARGS("halo_hc_combine_norm_rows_q8");
  return halo_b200_hc_combine_norm_rows_q8(c.s, res, out, inject, w, y, y16, hc, h, eps, iw, ipart, irows, rscale,
                                           y16_tokens, yq, yd, c.grid[0], c.err, c.errlen);
}
template <int DT>
HANDLER(H_hc_combine_norm_tok) {
  auto* res = r.ptr<void>(); auto* out = r.ptr<const float>(); auto* inject = r.ptr<const float>();
  auto* w = r.ptr<const float>(); auto* y16 = r.ptr<uint16_t>();
  const uint32_t h = r.u32(); const float eps = r.f32();
  auto* iw = r.ptr<const float>(); auto* ipart = r.ptr<float>(); const uint32_t irows = r.u32();
  auto* rscale = r.ptr<float>(); const uint32_t y16_tokens = r.u32();
  CHECK_ARGS("halo_hc_combine_norm_tok");
  return halo_b200_hc_combine_norm_tok(c.s, res, DT, out, inject, w, y16, h, eps, iw, ipart, irows, rscale, y16_tokens,
                                       c.grid[0], c.err, c.errlen);
}
template <int DT>
HANDLER(H_hc_combine_norm_tok_moe) {
  auto* res = r.ptr<void>(); auto* yp = r.ptr<const uint16_t>(); auto* pos = r.ptr<const uint32_t>();
  auto* mw = r.ptr<const float>(); auto* sx = r.ptr<const float>(); auto* sg = r.ptr<const float>();
  const uint32_t k = r.u32();
  auto* inject = r.ptr<const float>(); auto* w = r.ptr<const float>(); auto* y16 = r.ptr<uint16_t>();
  const uint32_t h = r.u32(); const float eps = r.f32();
  auto* iw = r.ptr<const float>(); auto* ipart = r.ptr<float>(); const uint32_t irows = r.u32();
  auto* rscale = r.ptr<float>(); const uint32_t y16_tokens = r.u32();
  CHECK_ARGS("halo_hc_combine_norm_tok_moe");
  return halo_b200_hc_combine_norm_tok_moe(c.s, res, DT, yp, pos, mw, sx, sg, k, inject, w, y16, h, eps, iw, ipart,
                                           irows, rscale, y16_tokens, c.grid[0], c.err, c.errlen);
}
template <int DT, bool ROWS>
HANDLER(H_hc_combine) {
  auto* res = r.ptr<void>(); auto* out = r.ptr<const float>(); auto* inject = r.ptr<const float>();
  const uint32_t hc = r.u32(), h = r.u32(); const uint32_t tokens = ROWS ? r.u32() : 1u;
  CHECK_ARGS("halo_hc_combine");
  return halo_b200_hc_combine_rows(c.s, res, DT, out, inject, hc, h, tokens, c.err, c.errlen);
}
template <int DT, bool ROWS>
HANDLER(H_broadcast) {
  auto* res = r.ptr<void>(); auto* x = r.ptr<const float>();
  const uint32_t hc = r.u32(), h = r.u32(); const uint32_t tokens = ROWS ? r.u32() : 1u;
  CHECK_ARGS("halo_broadcast");
  return halo_b200_broadcast_rows(c.s, res, DT, x, hc, h, tokens, c.err, c.errlen);
}
template <bool ROWS>
HANDLER(H_hc_mix) {
  auto* xn = r.ptr<const float>(); auto* gate = r.ptr<const float>(); auto* mixed = r.ptr<float>();
  const uint32_t hc = r.u32(), h = r.u32(); const uint32_t tokens = ROWS ? r.u32() : 1u;
  CHECK_ARGS("halo_hc_mix");
  return halo_b200_hc_mix_rows(c.s, xn, gate, mixed, hc, h, tokens, c.err, c.errlen);
}
template <bool ROWS>
HANDLER(H_axpy_sigmoid) {
  auto* y = r.ptr<float>(); auto* x = r.ptr<const float>(); auto* g = r.ptr<const float>();
  const uint32_t n = r.u32(); const uint32_t tokens = ROWS ? r.u32() : 1u;
  CHECK_ARGS("halo_axpy_sigmoid");
  return halo_b200_axpy_sigmoid_rows(c.s, y, x, g, n, tokens, c.err, c.errlen);
}
HANDLER(H_inject_reduce) {
  auto* ipart = r.ptr<const float>(); auto* inject = r.ptr<float>();
  const uint32_t hc = r.u32(), irows = r.u32(), tokens = r.u32();
  CHECK_ARGS("halo_inject_reduce");
  return halo_b200_inject_reduce(c.s, ipart, inject, hc, irows, tokens, c.err, c.errlen);
}
template <int DT>
HANDLER(H_res_to_f32) {
  auto* y = r.ptr<float>(); auto* x = r.ptr<const void>(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_res_to_f32");
  return halo_b200_res_to_f32(c.s, y, x, DT, n, c.err, c.errlen);
}
HANDLER(H_hc_norm_scales) {
  auto* res = r.ptr<const float>(); auto* scale = r.ptr<float>(); const uint32_t h = r.u32(); const float eps = r.f32();
  CHECK_ARGS("halo_hc_norm_scales");
  return halo_b200_hc_norm_scales(c.s, res, scale, h, eps, c.grid[0], c.err, c.errlen);
}

HANDLER(H_conv_step) {
  auto* in = r.ptr<const float>(); auto* state = r.ptr<float>(); auto* w = r.ptr<const float>(); auto* out = r.ptr<float>();
  const uint32_t channels = r.u32(), kern = r.u32();
  CHECK_ARGS("halo_conv_step");
  return halo_b200_conv_step(c.s, in, state, w, out, channels, kern, c.err, c.errlen);
}
HANDLER(H_conv_l2norm) {
  auto* in = r.ptr<const float>(); auto* state = r.ptr<float>(); auto* w = r.ptr<const float>(); auto* out = r.ptr<float>();
  const uint32_t channels = r.u32(), kern = r.u32(), l2 = r.u32(); const float eps = r.f32();
  CHECK_ARGS("halo_conv_l2norm");
  return halo_b200_conv_l2norm(c.s, in, state, w, out, channels, kern, l2, eps, c.block[0], c.err, c.errlen);
}
HANDLER(H_conv_l2norm_y) {
  auto* in = r.ptr<const float>(); auto* tab = r.ptr<const uint64_t>(); const uint32_t tstride = r.u32(), tslot = r.u32();
  auto* w = r.ptr<const float>(); auto* out = r.ptr<float>();
  const uint32_t channels = r.u32(), kern = r.u32(), l2 = r.u32(); const float eps = r.f32(); const uint32_t stride = r.u32();
  CHECK_ARGS("halo_conv_l2norm_y");
  return halo_b200_conv_l2norm_y(c.s, in, tab, tstride, tslot, w, out, channels, kern, l2, eps, stride, c.block[0],
                                 c.grid[1], c.err, c.errlen);
}
HANDLER(H_conv_l2norm_prefill) {
  auto* in = r.ptr<const float>(); auto* state = r.ptr<const float>(); auto* w = r.ptr<const float>();
  auto* out = r.ptr<float>();
  const uint32_t channels = r.u32(), kern = r.u32(), l2 = r.u32(); const float eps = r.f32();
  CHECK_ARGS("halo_conv_l2norm_prefill");
  return halo_b200_conv_l2norm_prefill(c.s, in, state, w, out, channels, kern, l2, eps, c.block[0], c.grid[1], c.err,
                                       c.errlen);
}
template <int IN, int OUT>
HANDLER(H_conv_l2norm_prefill8) {
  auto* in = r.ptr<const void>(); auto* state = r.ptr<const float>(); auto* w = r.ptr<const float>();
  auto* out = r.ptr<void>();
  const uint32_t channels = r.u32(), tokens = r.u32(), l2 = r.u32(); const float eps = r.f32();
  CHECK_ARGS("halo_conv_l2norm_prefill8");
  if ((tokens + 7) / 8 != c.grid[1]) return BadArgs(c, "halo_conv_l2norm_prefill8 (grid.y != ceil(tokens / 8))");
  return halo_b200_conv_l2norm_prefill8(c.s, in, IN, state, w, out, OUT, channels, tokens, l2, eps, c.block[0], c.err,
                                        c.errlen);
}
template <int IN>
HANDLER(H_conv_state_advance) {
  auto* in = r.ptr<const void>(); auto* state = r.ptr<float>();
  const uint32_t channels = r.u32(), kern = r.u32(), tokens = r.u32();
  CHECK_ARGS("halo_conv_state_advance");
  return halo_b200_conv_state_advance(c.s, in, IN, state, channels, kern, tokens, c.err, c.errlen);
}

template <int DT>
HANDLER(H_copy_at) {
  auto* dst = r.ptr<void>(); auto* src = r.ptr<const float>(); auto* params = r.ptr<const uint32_t>();
  const uint32_t slot = r.u32(), stride = r.u32(), n = r.u32();
  CHECK_ARGS("halo_copy_at");
  return halo_b200_copy_at(c.s, dst, DT, src, params, slot, stride, n, c.err, c.errlen);
}
HANDLER(H_copy_at_y) {
  auto* tab = r.ptr<const uint64_t>(); const uint32_t tstride = r.u32(), tslot = r.u32();
  auto* src = r.ptr<const float>(); auto* params = r.ptr<const uint32_t>();
  const uint32_t slot = r.u32(), stride = r.u32(), n = r.u32(), src_stride = r.u32(), pstride = r.u32();
  CHECK_ARGS("halo_copy_at_y");
  return halo_b200_copy_at_y(c.s, tab, tstride, tslot, HALO_B200_F32, src, params, slot, stride, n, src_stride, pstride,
                             c.grid[1], c.err, c.errlen);
}
HANDLER(H_copy) {
  auto* dst = r.ptr<float>(); auto* src = r.ptr<const float>(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_copy");
  return halo_b200_copy(c.s, dst, src, n, c.err, c.errlen);
}
HANDLER(H_f16_rows) {
  auto* x = r.ptr<const float>(); auto* y = r.ptr<uint16_t>(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_f16_rows");
  return halo_b200_f16_rows(c.s, x, y, n, c.err, c.errlen);
}
HANDLER(H_scale_silu) {
  auto* x = r.ptr<float>(); const float scale = r.f32(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_scale_silu");
  return halo_b200_scale_silu(c.s, x, x, HALO_B200_F32, scale, n, c.err, c.errlen);
}
HANDLER(H_scale_silu_h) {
  auto* x = r.ptr<const float>(); auto* y = r.ptr<uint16_t>(); const float scale = r.f32(); const uint32_t n = r.u32();
  CHECK_ARGS("halo_scale_silu_h");
  return halo_b200_scale_silu(c.s, x, y, HALO_B200_F16, scale, n, c.err, c.errlen);
}

HANDLER(H_moe_combine_grouped) {
  auto* yp = r.ptr<const uint16_t>(); auto* pos = r.ptr<const uint32_t>(); auto* w = r.ptr<const float>();
  auto* out = r.ptr<float>(); const uint32_t k = r.u32(), n = r.u32();
  CHECK_ARGS("halo_moe_combine_grouped");
  return halo_b200_moe_combine_grouped(c.s, yp, pos, w, out, k, n, c.grid[1], c.err, c.errlen);
}
HANDLER(H_moe_combine_shared) {
  auto* yp = r.ptr<const uint16_t>(); auto* pos = r.ptr<const uint32_t>(); auto* w = r.ptr<const float>();
  auto* x = r.ptr<const float>(); auto* g = r.ptr<const float>(); auto* out = r.ptr<float>();
  const uint32_t k = r.u32(), n = r.u32();
  CHECK_ARGS("halo_moe_combine_shared");
  return halo_b200_moe_combine_shared(c.s, yp, pos, w, x, g, out, k, n, c.grid[1], c.err, c.errlen);
}
HANDLER(H_moe_combine) {
  auto* part = r.ptr<const float>(); auto* w = r.ptr<const float>(); auto* out = r.ptr<float>();
  const uint32_t slots = r.u32(), n = r.u32();
  CHECK_ARGS("halo_moe_combine");
  return halo_b200_moe_combine(c.s, part, w, out, slots, n, c.err, c.errlen);
}
HANDLER(H_axpy_slot) {
  auto* y = r.ptr<float>(); auto* x = r.ptr<const float>(); auto* w = r.ptr<const float>();
  const uint32_t slot = r.u32(), n = r.u32();
  CHECK_ARGS("halo_axpy_slot");
  return halo_b200_axpy_slot(c.s, y, x, w, slot, n, c.err, c.errlen);
}

struct Entry {
  const char* name;
  Handler fn;
};

const Entry kTable[] = {
    {"halo_add", H_add},
    {"halo_axpy", H_axpy},
    {"halo_rmsnorm", H_rmsnorm},
    {"halo_rmsnorm_rows", H_rmsnorm_rows<HALO_B200_F32>},
    {"halo_rmsnorm_rows_r16", H_rmsnorm_rows<HALO_B200_F16>},
    {"halo_rmsnorm_rows_rb", H_rmsnorm_rows<HALO_B200_BF16>},
    {"halo_rmsnorm_rows_h", H_rmsnorm_rows_h<HALO_B200_F32>},
    {"halo_rmsnorm_rows_h_r16", H_rmsnorm_rows_h<HALO_B200_F16>},
    {"halo_rmsnorm_rows_h_rb", H_rmsnorm_rows_h<HALO_B200_BF16>},
    {"halo_rmsnorm_y", H_rmsnorm_y},
    {"halo_l2norm", H_l2norm},
    {"halo_gated_norm", H_gated_norm},
    {"halo_gated_norm_h", H_gated_norm_h<false>},
    {"halo_gated_norm_hz", H_gated_norm_h<true>},
    {"halo_gated_norm_h128w", H_gated_norm_h128w<false>},
    {"halo_gated_norm_h128w_hh", H_gated_norm_h128w<true>},
    {"halo_rope_neox", H_rope_neox},
    {"halo_rope_neox_rows", H_rope_neox_rows},
    {"halo_rope_neox_p", H_rope_neox_p},
    {"halo_rope_neox_blocks", H_rope_neox_blocks},
    {"halo_rope_neox_p_y", H_rope_neox_p_y},
    {"halo_split_qgate", H_split_qgate},
    {"halo_split_qgate_y", H_split_qgate_y},
    {"halo_split_qgate_norm_rope", H_split_qgate_norm_rope},
    {"halo_norm_rope_rows", H_norm_rope_rows},
    {"halo_silu_mul", H_silu_mul},
    {"halo_silu_mul_h", H_silu_mul_h},
    {"halo_sigmoid_gate", H_sigmoid_gate},
    {"halo_quantize_q8_rows", H_quantize_q8_rows},
    {"halo_quantize_q8_kblocked", H_quantize_q8_kblocked},
    {"halo_q8x_cols", H_q8x_cols},
    {"halo_hc_norm_q8x", H_hc_norm_q8x},
    {"halo_matvec_q8_0_embed", H_embed},
    {"halo_matvec_q8_0_embed_p", H_embed_p},
    {"halo_matvec_q8_0_embed_rows", H_embed_rows},
    {"halo_hc_combine_norm_rows", H_hc_combine_norm_rows<HALO_B200_F32>},
    {"halo_hc_combine_norm_rows_r16", H_hc_combine_norm_rows<HALO_B200_F16>},
    {"halo_hc_combine_norm_rows_rb", H_hc_combine_norm_rows<HALO_B200_BF16>},
    {"halo_hc_combine_norm_rows_q8", H_hc_combine_norm_rows_q8},
    {"halo_hc_combine_norm_tok", H_hc_combine_norm_tok<HALO_B200_F32>},
    {"halo_hc_combine_norm_tok_r16", H_hc_combine_norm_tok<HALO_B200_F16>},
    {"halo_hc_combine_norm_tok_rb", H_hc_combine_norm_tok<HALO_B200_BF16>},
    {"halo_hc_combine_norm_tok_moe", H_hc_combine_norm_tok_moe<HALO_B200_F32>},
    {"halo_hc_combine_norm_tok_moe_r16", H_hc_combine_norm_tok_moe<HALO_B200_F16>},
    {"halo_hc_combine_norm_tok_moe_rb", H_hc_combine_norm_tok_moe<HALO_B200_BF16>},
    {"halo_hc_combine_norm_tok_moev", H_hc_combine_norm_tok_moe<HALO_B200_F32>},
    {"halo_hc_combine_norm_tok_moev_r16", H_hc_combine_norm_tok_moe<HALO_B200_F16>},
    {"halo_hc_combine_norm_tok_moev_rb", H_hc_combine_norm_tok_moe<HALO_B200_BF16>},
    {"halo_hc_combine", H_hc_combine<HALO_B200_F32, false>},
    {"halo_hc_combine_rows", H_hc_combine<HALO_B200_F32, true>},
    {"halo_hc_combine_rows_r16", H_hc_combine<HALO_B200_F16, true>},
    {"halo_hc_combine_rows_rb", H_hc_combine<HALO_B200_BF16, true>},
    {"halo_broadcast", H_broadcast<HALO_B200_F32, false>},
    {"halo_broadcast_rows", H_broadcast<HALO_B200_F32, true>},
    {"halo_broadcast_rows_r16", H_broadcast<HALO_B200_F16, true>},
    {"halo_broadcast_rows_rb", H_broadcast<HALO_B200_BF16, true>},
    {"halo_hc_mix", H_hc_mix<false>},
    {"halo_hc_mix_rows", H_hc_mix<true>},
    {"halo_axpy_sigmoid", H_axpy_sigmoid<false>},
    {"halo_axpy_sigmoid_rows", H_axpy_sigmoid<true>},
    {"halo_inject_reduce", H_inject_reduce},
    {"halo_res_to_f32_r16", H_res_to_f32<HALO_B200_F16>},
    {"halo_res_to_f32_rb", H_res_to_f32<HALO_B200_BF16>},
    {"halo_hc_norm_scales", H_hc_norm_scales},
    {"halo_hc_norm_scales_u", H_hc_norm_scales},
    {"halo_conv_step", H_conv_step},
    {"halo_conv_l2norm", H_conv_l2norm},
    {"halo_conv_l2norm_y", H_conv_l2norm_y},
    {"halo_conv_l2norm_prefill", H_conv_l2norm_prefill},
    {"halo_conv_l2norm_prefill8", H_conv_l2norm_prefill8<HALO_B200_F32, HALO_B200_F32>},
    {"halo_conv_l2norm_prefill8_h", H_conv_l2norm_prefill8<HALO_B200_F16, HALO_B200_F32>},
    {"halo_conv_l2norm_prefill8_hh", H_conv_l2norm_prefill8<HALO_B200_F16, HALO_B200_F16>},
    {"halo_conv_state_advance", H_conv_state_advance<HALO_B200_F32>},
    {"halo_conv_state_advance_h", H_conv_state_advance<HALO_B200_F16>},
    {"halo_copy_at_y", H_copy_at_y},
    {"halo_copy_at", H_copy_at<HALO_B200_F32>},
    {"halo_copy_at_h", H_copy_at<HALO_B200_F16>},
    {"halo_copy", H_copy},
    {"halo_f16_rows", H_f16_rows},
    {"halo_scale_silu", H_scale_silu},
    {"halo_scale_silu_h", H_scale_silu_h},
    {"halo_moe_combine_grouped", H_moe_combine_grouped},
    {"halo_moe_combine_shared", H_moe_combine_shared},
    {"halo_moe_combine", H_moe_combine},
    {"halo_moe_combine_u", H_moe_combine},
    {"halo_axpy_slot", H_axpy_slot},
};
constexpr size_t kCount = sizeof(kTable) / sizeof(kTable[0]);

}  // namespace

extern "C" {

size_t halo_b200_kernel_count(void) { return kCount; }
const char* halo_b200_kernel_name(size_t index) { return index < kCount ? kTable[index].name : nullptr; }

int halo_b200_launch(halo_b200_stream stream, const char* name, const halo_b200_arg* args, size_t nargs,
                     const uint32_t grid[3], const uint32_t block[3], char* err, size_t errlen) {
  if (!name || !grid || !block || (nargs && !args)) {
    if (err && errlen) std::snprintf(err, errlen, "halo_b200_launch: null argument");
    return -1;
  }
  for (size_t i = 0; i < kCount; ++i) {
    if (std::strcmp(kTable[i].name, name) == 0) {
      Reader r{args, nargs};
      const Ctx c{stream, grid, block, err, errlen};
      return kTable[i].fn(r, c);
    }
  }
  if (err && errlen) std::snprintf(err, errlen, "halo_b200_launch: unknown kernel %s", name);
  return -1;
}

}  // extern "C"
