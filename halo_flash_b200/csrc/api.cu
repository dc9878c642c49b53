// C ABI of libhalo_b200.so (include/halo_b200.h): argument validation, choice
// between the vector and scalar kernels, and launch by reference kernel name.
// No function here allocates, synchronizes or keeps state (one tuning knob aside).
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/halo_b200.h"
#include "kernels.h"

using namespace halo_b200;

namespace {

std::atomic<int> g_norm_threads_per_row{0};
std::atomic<int> g_norm_short_rows_k1{0};
std::atomic<int> g_norm_force_general{0};
std::atomic<int> g_l2_keep{1};
std::atomic<int> g_embed_direct{1};
std::atomic<int> g_rope_rows_per_group{0};
std::atomic<int> g_rope_lean_k{0};
std::atomic<int> g_rope_staged{1};
std::atomic<int> g_gated_rows_per_group{0};
std::atomic<int> g_pdl{1};

int Fail(char* err, size_t errlen, const char* fmt, ...) {
  if (err && errlen) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(err, errlen, fmt, ap);
    va_end(ap);
  }
  return -1;
}

int Done(cudaError_t e, const char* what, char* err, size_t errlen) {
  if (e == cudaSuccess) {
    if (err && errlen) err[0] = '\0';
    return 0;
  }
  return Fail(err, errlen, "%s: %s", what, cudaGetErrorString(e));
}

bool Aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
bool ValidDType(int t) { return t == kF32 || t == kF16 || t == kBF16; }
cudaStream_t S(halo_b200_stream s) { return static_cast<cudaStream_t>(s); }

#define REQUIRE(cond, ...) \
  do {                     \
    if (!(cond)) return Fail(err, errlen, __VA_ARGS__); \
  } while (0)

// pow(theta, -2 i / rot) in fp32 with the host libm: the expression of
// src/model/cpu_ops.cpp:174-175, so device angles equal the CPU operator's bit for bit.
bool FillInvFreq(InvFreq* f, uint32_t rot, float theta) {
  if (rot / 2 > static_cast<uint32_t>(kMaxRotHalf)) return false;
  for (uint32_t i = 0; i < rot / 2; ++i)
    f->f[i] = std::pow(theta, -2.0F * static_cast<float>(i) / static_cast<float>(rot));
  return true;
}

int RunNorm(NormArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.rows == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.x != nullptr, "%s: x is null", what);
  REQUIRE(a.d > 0, "%s: d is 0", what);
  REQUIRE(ValidDType(a.x_dtype) && ValidDType(a.y_dtype), "%s: unknown dtype", what);
  REQUIRE(a.y || a.y16 || a.q8_0 || a.xq || a.res || a.rscale, "%s: no output", what);
  REQUIRE((a.delta == nullptr) == (a.res == nullptr), "%s: delta and res go together", what);
  REQUIRE((a.xq == nullptr) == (a.xd == nullptr), "%s: xq and xd go together", what);
  if (a.q8_0 || a.xq) REQUIRE(a.d % 32 == 0, "%s: Q8 output needs d %% 32 == 0 (d = %u)", what, a.d);
  if (a.q8_0) REQUIRE(Aligned(a.q8_0, 2), "%s: Q8_0 output must be 2-byte aligned", what);
  if (a.kb_tokens || a.y16_tokens) REQUIRE(a.d % 64 == 0, "%s: K-blocked layouts need d %% 64 == 0", what);
  if (a.w_period == 0) a.w_period = 1;
  if (a.kb_period == 0) a.kb_period = 1;
  const size_t xs = DTypeSize(a.x_dtype), ys = DTypeSize(a.y_dtype);
  REQUIRE(Aligned(a.x, xs) && Aligned(a.y, ys) && Aligned(a.delta, xs) && Aligned(a.res, xs) && Aligned(a.w, 4) &&
              Aligned(a.y16, 2) && Aligned(a.xd, 4) && Aligned(a.rscale, 4),
          "%s: pointer not aligned to its element type", what);
  a.threads_per_row = g_norm_threads_per_row.load(std::memory_order_relaxed);
  if (g_norm_short_rows_k1.load(std::memory_order_relaxed)) a.short_rows_k1 = 1;
  a.force_general = g_norm_force_general.load(std::memory_order_relaxed);
  a.keep_hint = g_l2_keep.load(std::memory_order_relaxed);
  bool vec = a.d % 8 == 0 && a.d <= 256u * 8u * 8u && Aligned(a.x, 16) && Aligned(a.y, 16) && Aligned(a.delta, 16) &&
             Aligned(a.res, 16) && Aligned(a.y16, 16) && Aligned(a.w, 16) && a.w_stride % 4 == 0 &&
             Aligned(a.xq, 8) && a.entry_stride % 8 == 0;
  if (vec && a.threads_per_row) {
    const unsigned g = static_cast<unsigned>(a.threads_per_row);
    const unsigned octs = a.d / 8, k = (octs + g - 1) / g;
    if (k > 8 || ((a.q8_0 || a.xq) && g < 4)) a.threads_per_row = 0;
  }
  a.vec = vec;
  return Done(LaunchNorm(a, S(stream)), what, err, errlen);
}

int RunGated(GatedArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.rows == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.o && a.z && a.w && a.y, "%s: null pointer", what);
  REQUIRE(a.d > 0, "%s: d is 0", what);
  REQUIRE(ValidDType(a.o_dtype) && ValidDType(a.z_dtype) && ValidDType(a.y_dtype), "%s: unknown dtype", what);
  REQUIRE(a.mode <= 1, "%s: mode must be 0 (SiLU) or 1 (sigmoid)", what);
  REQUIRE(Aligned(a.o, DTypeSize(a.o_dtype)) && Aligned(a.z, DTypeSize(a.z_dtype)) &&
              Aligned(a.y, DTypeSize(a.y_dtype)) && Aligned(a.w, 4),
          "%s: pointer not aligned to its element type", what);
  a.vec = a.d % 8 == 0 && a.d <= 256u * 8u * 4u && Aligned(a.o, 16) && Aligned(a.z, 16) && Aligned(a.y, 16) &&
          Aligned(a.w, 16);
  a.threads_per_row = g_norm_threads_per_row.load(std::memory_order_relaxed);
  a.short_rows_k1 = g_norm_short_rows_k1.load(std::memory_order_relaxed);
  a.rows_per_group = g_gated_rows_per_group.load(std::memory_order_relaxed);
  a.force_general = g_norm_force_general.load(std::memory_order_relaxed);
  if (a.threads_per_row && (a.d / 8 + a.threads_per_row - 1) / a.threads_per_row > 4) a.threads_per_row = 0;
  const cudaError_t e = LaunchGatedNorm(a, S(stream));
  if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported (o, z, y) dtype combination", what);
  return Done(e, what, err, errlen);
}

int RunRope(RopeArgs a, float theta, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.tokens == 0 || a.heads + a.heads2 == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.x != nullptr, "%s: x is null", what);
  REQUIRE(ValidDType(a.dtype), "%s: unknown dtype", what);
  REQUIRE(a.rot % 2 == 0 && a.rot <= a.hd, "%s: rotary_dim %u must be even and <= head_dim %u", what, a.rot, a.hd);
  REQUIRE(a.heads2 == 0 || a.x2 != nullptr, "%s: k is null", what);
  InvFreq f;
  REQUIRE(FillInvFreq(&f, a.rot, theta), "%s: rotary_dim %u exceeds %d", what, a.rot, 2 * kMaxRotHalf);
  const size_t es = DTypeSize(a.dtype);
  REQUIRE(Aligned(a.x, es) && Aligned(a.x2, es) && Aligned(a.pos.params, 4) && Aligned(a.pos_out, 4),
          "%s: pointer not aligned to its element type", what);
  a.vec = (a.rot / 2) % 8 == 0 && a.hd % 8 == 0 && a.token_stride % 8 == 0 && a.token_stride2 % 8 == 0 &&
          Aligned(a.x, 16) && Aligned(a.x2, 16);
  return Done(LaunchRope(a, f, S(stream)), what, err, errlen);
}

int RunElt(EltArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  REQUIRE(a.nseg >= 1 && a.nseg <= kMaxSegments, "%s: 1..%d segments", what, kMaxSegments);
  REQUIRE(ValidDType(a.in_dtype) && ValidDType(a.y_dtype), "%s: unknown dtype", what);
  // drop empty segments (an empty chunk is a no-op)
  int n = 0;
  for (int i = 0; i < a.nseg; ++i)
    if (a.seg[i].n) a.seg[n++] = a.seg[i];
  a.nseg = n;
  if (n == 0) return Done(cudaSuccess, what, err, errlen);
  a.vec = true;
  for (int i = 0; i < n; ++i) {
    const EltSegment& g = a.seg[i];
    REQUIRE(g.a && g.b && g.y, "%s: null pointer", what);
    REQUIRE(Aligned(g.a, DTypeSize(a.in_dtype)) && Aligned(g.b, DTypeSize(a.in_dtype)) &&
                Aligned(g.y, DTypeSize(a.y_dtype)),
            "%s: pointer not aligned to its element type", what);
    a.vec = a.vec && Aligned(g.a, 16) && Aligned(g.b, 16) && Aligned(g.y, 16);
  }
  const cudaError_t e = LaunchElementwise(a, S(stream));
  if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported (in, out) dtype combination", what);
  return Done(e, what, err, errlen);
}

int RunEmbed(EmbedArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.tokens == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.table && a.out, "%s: null pointer", what);
  REQUIRE(ValidDType(a.out_dtype), "%s: unknown dtype", what);
  REQUIRE(a.cols % 32 == 0, "%s: Q8_0 rows need cols %% 32 == 0 (cols = %u)", what, a.cols);
  REQUIRE(a.row_bytes >= static_cast<uint64_t>(a.cols / 32) * 34, "%s: row_bytes %llu smaller than %u Q8_0 blocks",
          what, static_cast<unsigned long long>(a.row_bytes), a.cols / 32);
  REQUIRE(Aligned(a.out, DTypeSize(a.out_dtype)) && Aligned(a.ids, 4), "%s: pointer not aligned to its element type",
          what);
  a.vec = a.row_bytes % 16 == 0 && Aligned(a.table, 16) && Aligned(a.out, 16);
  a.direct = g_embed_direct.load(std::memory_order_relaxed) != 0;
  return Done(LaunchEmbedQ8_0(a, S(stream)), what, err, errlen);
}

int RunQuant(QuantArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.rows == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.x != nullptr, "%s: x is null", what);
  REQUIRE(ValidDType(a.x_dtype), "%s: unknown dtype", what);
  REQUIRE(a.q8_0 || a.xq, "%s: no output", what);
  REQUIRE((a.xq == nullptr) == (a.xd == nullptr) && (a.xq2 == nullptr) == (a.xd2 == nullptr),
          "%s: codes and scales go together", what);
  REQUIRE(a.xq2 == nullptr || (a.xq != nullptr && a.kb_tokens == 0), "%s: second level needs row-major xq", what);
  REQUIRE(a.cols % 32 == 0, "%s: cols %% 32 != 0 (cols = %u)", what, a.cols);
  if (a.kb_tokens) REQUIRE(a.cols % 64 == 0, "%s: K-blocked layout needs cols %% 64 == 0", what);
  REQUIRE(Aligned(a.x, DTypeSize(a.x_dtype)) && Aligned(a.xd, 4) && Aligned(a.xd2, 4) && Aligned(a.q8_0, 2),
          "%s: pointer not aligned to its element type", what);
  if (a.pre_w) {
    REQUIRE(a.pre_scale && a.xn, "%s: null pointer", what);
    REQUIRE(a.pre_h > 0 && a.cols % a.pre_h == 0, "%s: h = %u does not divide the row of %u", what, a.pre_h, a.cols);
    REQUIRE(Aligned(a.pre_scale, 4) && Aligned(a.pre_w, 4) && Aligned(a.xn, 4), "%s: pointer not aligned to its element type", what);
  }
  a.vec = Aligned(a.x, 16) && a.x_stride % 8 == 0 && Aligned(a.xq, 8) && Aligned(a.xq2, 8) &&
          (a.pre_w == nullptr || (a.pre_h % 8 == 0 && Aligned(a.pre_w, 16) && Aligned(a.xn, 16)));
  return Done(LaunchQuantize(a, S(stream)), what, err, errlen);
}

// check_only: validate and return 0 when the vector kernels (and with them the rotation-table form) can run these
// arguments, 1 when only the unfused fallback can, -1 with a message when the call is invalid; nothing is launched.
int RunNormRope(NormRopeArgs a, float theta, const char* what, halo_b200_stream stream, char* err, size_t errlen,
                bool check_only = false) {
  if (a.rows == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.in && a.out, "%s: null pointer", what);
  REQUIRE(ValidDType(a.in_dtype) && ValidDType(a.out_dtype), "%s: unknown dtype", what);
  REQUIRE(a.d > 0 && a.d <= 256, "%s: d = %u outside 1..256", what, a.d);
  REQUIRE(a.heads > 0, "%s: heads is 0", what);
  REQUIRE(a.rot % 2 == 0 && a.rot <= a.d, "%s: rotary_dim %u must be even and <= d %u", what, a.rot, a.d);
  REQUIRE(a.in_row_stride >= a.d, "%s: in_row_stride < d", what);
  REQUIRE(a.gate == nullptr || a.in_row_stride >= 2ull * a.d, "%s: gate needs q|gate rows (in_row_stride >= 2 d)", what);
  InvFreq f = {};
  if (a.table) {
    REQUIRE(Aligned(a.table, 16), "%s: rotation table must be 16-byte aligned", what);
  } else {
    REQUIRE(FillInvFreq(&f, a.rot, theta), "%s: rotary_dim too large", what);
  }
  a.rows_per_group = g_rope_rows_per_group.load(std::memory_order_relaxed);
  a.lean_k = g_rope_lean_k.load(std::memory_order_relaxed);
  a.staged = g_rope_staged.load(std::memory_order_relaxed);
  a.force_general = g_norm_force_general.load(std::memory_order_relaxed);
  const bool vec = a.d % 8 == 0 && (a.rot / 2) % 8 == 0 && a.in_row_stride % 8 == 0 && Aligned(a.in, 16) &&
                   Aligned(a.out, 16) && Aligned(a.gate, 16) && Aligned(a.cache, 16) && Aligned(a.w, 16) &&
                   a.in_row_stride2 % 8 == 0 && Aligned(a.in2, 16) && Aligned(a.out2, 16) && Aligned(a.cache2, 16) &&
                   Aligned(a.w2, 16);
  if (a.heads2) {
    REQUIRE(a.in2 && a.out2, "%s: second tensor is null", what);
    REQUIRE((a.w == nullptr) == (a.w2 == nullptr), "%s: both tensors need a gamma, or neither", what);
    REQUIRE(a.rows % a.heads == 0, "%s: rows %u not a multiple of heads %u", what, a.rows, a.heads);
    REQUIRE(a.in_row_stride2 >= a.d, "%s: in_row_stride2 < d", what);
    REQUIRE(vec, "%s: two tensors in one launch need 16-byte aligned rows, d %% 8 == 0 and rot %% 16 == 0", what);
  }
  if (vec) {
    const bool combo = a.in_dtype == kF32 || (a.in_dtype == kBF16 && a.out_dtype != kF16) ||
                       (a.in_dtype == kF16 && a.out_dtype == kF16);
    REQUIRE(combo, "%s: unsupported (in, out) dtype combination", what);
  }
  if (check_only) {
    if (err && errlen) err[0] = '\0';
    return vec ? 0 : 1;
  }
  if (vec) {
    const cudaError_t e = LaunchNormRope(a, f, S(stream));
    if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported (in, out) dtype combination", what);
    return Done(e, what, err, errlen);
  }
  REQUIRE(a.table == nullptr, "%s: a rotation table needs 16-byte aligned rows, d %% 8 == 0 and rot %% 16 == 0", what);
  // Odd shapes: the separate kernels in sequence (the reference's own unfused path,
  // src/engine/qwen35_gpu.cpp:204-222): split, per-head norm, rope, cache copy.
  REQUIRE(a.in_dtype == a.out_dtype, "%s: unaligned shapes need in_dtype == out_dtype", what);
  REQUIRE(a.cache == nullptr, "%s: cache append needs 16-byte aligned rows with d %% 8 == 0 and rot %% 16 == 0", what);
  const void* norm_in = a.in;
  if (a.in_row_stride != a.d) {
    REQUIRE(a.in_row_stride == 2ull * a.d && a.gate != nullptr, "%s: strided rows need the q|gate form with gate set",
            what);
    SplitArgs sp;
    sp.qg = a.in;
    sp.q = a.out;
    sp.gate = a.gate;
    sp.dtype = a.in_dtype;
    sp.hd = a.d;
    sp.rows = a.rows;
    const cudaError_t e = LaunchSplitQgate(sp, S(stream));
    if (e != cudaSuccess) return Done(e, what, err, errlen);
    norm_in = a.out;
  }
  if (a.w) {
    NormArgs n;
    n.x = norm_in;
    n.x_dtype = a.in_dtype;
    n.y = a.out;
    n.y_dtype = a.out_dtype;
    n.w = a.w;
    n.one_plus = a.one_plus;
    n.d = a.d;
    n.rows = a.rows;
    n.eps = a.eps;
    n.vec = false;
    const cudaError_t e = LaunchNorm(n, S(stream));
    if (e != cudaSuccess) return Done(e, what, err, errlen);
  } else if (norm_in != a.out) {
    return Fail(err, errlen, "%s: out must alias in when there is neither a norm nor a split", what);
  }
  RopeArgs r;
  r.x = a.out;
  r.dtype = a.out_dtype;
  r.tokens = a.rows / a.heads;
  r.heads = a.heads;
  r.hd = a.d;
  r.rot = a.rot;
  r.token_stride = static_cast<uint64_t>(a.heads) * a.d;
  r.pos = a.pos;
  r.pos_out = a.pos_out;
  r.vec = false;
  REQUIRE(a.rows % a.heads == 0, "%s: rows %u not a multiple of heads %u", what, a.rows, a.heads);
  return Done(LaunchRope(r, f, S(stream)), what, err, errlen);
}


std::atomic<int> g_hc_row_level{0};
std::atomic<int> g_hc_token_k{0};
std::atomic<int> g_hc_fused_inject{0};
std::atomic<int> g_conv_tile{0};
std::atomic<int> g_conv_staged{1};

int RunHc(HcArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.tokens == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.res != nullptr && a.w != nullptr, "%s: null pointer", what);
  REQUIRE(a.hc >= 1 && a.h > 0, "%s: hc and h must be positive", what);
  REQUIRE(!(a.out && a.yp), "%s: a stored block output and an expert sum exclude each other", what);
  const bool combine = a.out || a.yp;
  REQUIRE(combine == (a.inject != nullptr), "%s: inject goes with a block output", what);
  if (a.yp) REQUIRE(a.pos && a.mw && a.sx && a.sg && a.k >= 1, "%s: expert sum needs pos, mw, sx, sg and k >= 1", what);
  REQUIRE(ValidDType(a.res_dtype) && ValidDType(a.out_dtype) && ValidDType(a.y_dtype), "%s: unknown dtype", what);
  REQUIRE(a.y || a.y16 || a.rscale || a.yq || a.iw || combine, "%s: no output", what);
  REQUIRE(a.irows <= 8, "%s: at most 8 inject rows (irows = %u)", what, a.irows);
  if (a.iw) REQUIRE(a.ipart != nullptr && a.irows >= 1, "%s: iw needs ipart and irows >= 1", what);
  else a.irows = 0;
  REQUIRE((a.yq == nullptr) == (a.yd == nullptr), "%s: yq and yd go together", what);
  if (a.yq) REQUIRE(a.h % 32 == 0 && a.y16_tokens >= a.tokens, "%s: the int8 copy needs h %% 32 == 0 and y16_tokens >= tokens", what);
  if (a.y16_tokens) REQUIRE((static_cast<uint64_t>(a.hc) * a.h) % 64 == 0 && a.y16_tokens >= a.tokens,
                            "%s: K-blocked layouts need hc * h %% 64 == 0 and y16_tokens >= tokens", what);
  const size_t rs = DTypeSize(a.res_dtype), os = DTypeSize(a.out_dtype), ys = DTypeSize(a.y_dtype);
  REQUIRE(Aligned(a.res, rs) && Aligned(a.out, os) && Aligned(a.yp, os) && Aligned(a.y, ys) && Aligned(a.y16, 2) &&
              Aligned(a.w, 4) && Aligned(a.inject, 4) && Aligned(a.iw, 4) && Aligned(a.ipart, 4) &&
              Aligned(a.rscale, 4) && Aligned(a.yd, 4) && Aligned(a.sx, a.sx_is_f32 ? 4 : os),
          "%s: pointer not aligned to its element type", what);
  a.vec = a.h % 8 == 0 && a.h >= 32 && a.h <= 256u * 8u * 8u && Aligned(a.res, 16) && Aligned(a.out, 16) &&
          Aligned(a.yp, 16) && Aligned(a.sx, 16) && Aligned(a.y, 16) && Aligned(a.y16, 16) && Aligned(a.w, 16) &&
          Aligned(a.iw, 16) && Aligned(a.yq, 8);
  if (!a.vec) REQUIRE(!a.yp && !a.yq && (a.out || !combine),
                      "%s: the expert sum and the int8 copy need h %% 8 == 0, 32 <= h <= 16384 and 16-byte aligned buffers", what);
  if (!a.vec && !combine) return Fail(err, errlen, "%s: the norm-only form needs h %% 8 == 0 and 16-byte aligned buffers", what);
  if (!a.y)  // no y: any y type of a supported (res, out, y) triple will do
    a.y_dtype = (a.out_dtype == a.res_dtype && a.res_dtype != kF32) ? a.res_dtype : kF32;
  a.row_level = g_hc_row_level.load(std::memory_order_relaxed);
  a.token_k = g_hc_token_k.load(std::memory_order_relaxed);
  a.fused_inject = g_hc_fused_inject.load(std::memory_order_relaxed);
  const cudaError_t e = LaunchHcCombineNorm(a, S(stream));
  if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported (res, out, y) dtype combination or shape", what);
  return Done(e, what, err, errlen);
}

int RunHcElt(HcEltArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.tokens == 0 || a.h == 0) return Done(cudaSuccess, what, err, errlen);
  REQUIRE(a.a != nullptr && a.b != nullptr, "%s: null pointer", what);
  REQUIRE(a.op == kHcBroadcast || a.op == kInjectReduce || a.op == kScaleSilu || a.c != nullptr, "%s: null pointer", what);
  REQUIRE(a.hc >= 1, "%s: hc is 0", what);
  REQUIRE(ValidDType(a.a_dtype) && ValidDType(a.b_dtype), "%s: unknown dtype", what);
  REQUIRE(Aligned(a.a, DTypeSize(a.a_dtype)) && Aligned(a.b, DTypeSize(a.b_dtype)) && Aligned(a.c, a.op == kHcMix ? DTypeSize(a.b_dtype) : 4),
          "%s: pointer not aligned to its element type", what);
  a.vec = a.h % 8 == 0 && Aligned(a.a, 16) && Aligned(a.b, 16) && (a.op != kHcMix || Aligned(a.c, 16)) &&
          (a.at_params == nullptr || (a.at_stride * DTypeSize(a.a_dtype)) % 16 == 0);
  const cudaError_t e = LaunchHcElt(a, S(stream));
  if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported dtype combination", what);
  return Done(e, what, err, errlen);
}


int RunConv(ConvArgs a, bool advance_only, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.tokens == 0 || a.channels == 0) return Done(cudaSuccess, what, err, errlen);  // an empty chunk is a no-op
  REQUIRE(a.in != nullptr, "%s: in is null", what);
  REQUIRE(a.kern >= 1 && a.kern <= 9, "%s: conv kernel length %u outside 1..9", what, a.kern);
  REQUIRE(ValidDType(a.in_dtype) && ValidDType(a.out_dtype), "%s: unknown dtype", what);
  REQUIRE(Aligned(a.in, DTypeSize(a.in_dtype)) && Aligned(a.state, 4), "%s: pointer not aligned to its element type", what);
  if (advance_only) {
    REQUIRE(a.state != nullptr || a.kern < 2, "%s: state is null", what);
    return Done(LaunchConvStateAdvance(a, S(stream)), what, err, errlen);
  }
  REQUIRE(a.w != nullptr && a.out != nullptr, "%s: null pointer", what);
  REQUIRE(a.in != a.out, "%s: in and out must not be the same buffer (a token reads its predecessors' inputs)", what);
  REQUIRE(Aligned(a.out, DTypeSize(a.out_dtype)) && Aligned(a.w, 4), "%s: pointer not aligned to its element type", what);
  REQUIRE(a.l2_channels <= a.channels, "%s: l2_channels exceeds channels", what);
  if (a.l2_channels) REQUIRE(a.d >= 1 && a.d <= 1024 && a.l2_channels % a.d == 0,
                             "%s: the normalized channels must be whole heads of d <= 1024 channels", what);
  if (a.d == 0) a.d = 128;
  a.vec = a.channels % 8 == 0 && Aligned(a.in, 16) && Aligned(a.out, 16) && Aligned(a.w, 16) && Aligned(a.state, 16);
  a.tile = g_conv_tile.load(std::memory_order_relaxed);
  a.staged = g_conv_staged.load(std::memory_order_relaxed);
  const cudaError_t e = LaunchConvL2norm(a, S(stream));
  if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported (in, out) dtype pair or chunk too long", what);
  return Done(e, what, err, errlen);
}


// One decode step: conv, state shift, SiLU and L2 norm in one launch, for one session (`state`) or for
// `entries` sessions whose states come from a table of device addresses.
int RunConvStep(ConvArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.entries == 0 || a.channels == 0) return Done(cudaSuccess, what, err, errlen);
  REQUIRE(a.in && a.out && a.w, "%s: null pointer", what);
  REQUIRE(a.kern >= 1 && a.kern <= 9, "%s: conv kernel length %u outside 1..9", what, a.kern);
  REQUIRE(a.state_tab != nullptr || a.entries == 1, "%s: more than one entry needs the state table", what);
  REQUIRE(a.kern < 2 || a.state_tab != nullptr || a.state != nullptr, "%s: state is null", what);
  REQUIRE(Aligned(a.in, DTypeSize(a.in_dtype)) && Aligned(a.out, DTypeSize(a.out_dtype)) && Aligned(a.w, 4) &&
              Aligned(a.state, 4) && Aligned(a.state_tab, 8),
          "%s: pointer not aligned to its element type", what);
  REQUIRE(a.l2_channels <= a.channels, "%s: l2_channels exceeds channels", what);
  if (a.d == 0) a.d = 128;
  REQUIRE(a.d <= 1024 && (a.l2_channels == 0 || a.l2_channels % a.d == 0),
          "%s: the normalized channels must be whole heads of d <= 1024 channels", what);
  REQUIRE(a.entries <= 65535u, "%s: more than 65535 entries", what);
  const cudaError_t e = LaunchConvStep(a, S(stream));
  if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported (in, out) dtype pair", what);
  return Done(e, what, err, errlen);
}


int RunMoeCombine(MoeCombineArgs a, const char* what, halo_b200_stream stream, char* err, size_t errlen) {
  if (a.tokens == 0 || a.n == 0) return Done(cudaSuccess, what, err, errlen);
  REQUIRE(a.yp && a.mw && a.out, "%s: null pointer", what);
  REQUIRE((a.sx == nullptr) == (a.sg == nullptr), "%s: sx and sg go together", what);
  REQUIRE(ValidDType(a.yp_dtype) && ValidDType(a.out_dtype), "%s: unknown dtype", what);
  const size_t ys = DTypeSize(a.yp_dtype), os = DTypeSize(a.out_dtype);
  REQUIRE(Aligned(a.yp, ys) && Aligned(a.out, os) && Aligned(a.mw, 4) && Aligned(a.pos, 4) && Aligned(a.sg, 4) &&
              Aligned(a.sx, a.sx_is_f32 ? 4 : ys),
          "%s: pointer not aligned to its element type", what);
  a.vec = a.n % 8 == 0 && Aligned(a.yp, 16) && Aligned(a.out, 16) && Aligned(a.sx, 16);
  const cudaError_t e = LaunchMoeCombine(a, S(stream));
  if (e == cudaErrorInvalidValue) return Fail(err, errlen, "%s: unsupported (yp, out) dtype pair", what);
  return Done(e, what, err, errlen);
}

// Q and K of one layer as one NormRopeArgs (positions and table left to the caller).
NormRopeArgs QkArgs(const void* q_in, uint64_t q_row_stride, void* q_out, void* q_gate, const float* w_q, uint32_t q_heads,
                    const void* k_in, void* k_out, void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype,
                    int out_dtype, int one_plus, float eps, uint32_t d, uint32_t rotary_dim, uint32_t tokens) {
  NormRopeArgs a;
  a.in = q_in;
  a.in_dtype = in_dtype;
  a.in_row_stride = q_row_stride;
  a.out = q_out;
  a.out_dtype = out_dtype;
  a.gate = q_gate;
  a.w = w_q;
  a.heads = q_heads;
  a.rows = tokens * q_heads;
  a.in2 = k_heads ? k_in : nullptr;
  a.in_row_stride2 = d;
  a.out2 = k_heads ? k_out : nullptr;
  a.cache2 = k_heads ? k_cache : nullptr;
  a.w2 = k_heads ? w_k : nullptr;
  a.heads2 = k_heads;
  a.one_plus = one_plus;
  a.eps = eps;
  a.d = d;
  a.rot = rotary_dim;
  return a;
}

}  // namespace

namespace halo_b200 {
bool PdlEnabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }

int CheckNormRopeQk(const void* q_in, uint64_t q_row_stride, void* q_out, void* q_gate, const float* w_q, uint32_t q_heads,
                    const void* k_in, void* k_out, void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype,
                    int out_dtype, uint32_t d, uint32_t rotary_dim, uint32_t tokens, float theta, char* err,
                    size_t errlen) {
  const NormRopeArgs a = QkArgs(q_in, q_row_stride, q_out, q_gate, w_q, q_heads, k_in, k_out, k_cache, w_k, k_heads,
                                in_dtype, out_dtype, 0, 0.0f, d, rotary_dim, tokens);
  return RunNormRope(a, theta, "halo_norm_rope_qk_noalloc", nullptr, err, errlen, true);
}
}  // namespace halo_b200

extern "C" {

const char* halo_b200_version(void) { return "halo_b200 0.1 sm_100a"; }

int halo_b200_tune(const char* key, int value) {
  // key, the switch it sets, and the values it accepts (a zero-terminated list; 0 is always one of them)
  struct Key {
    const char* name;
    std::atomic<int>* slot;
    int allowed[10];
  };
  static const Key kKeys[] = {
      {"norm_threads_per_row", &g_norm_threads_per_row, {1, 2, 4, 8, 16, 32, 64, 128, 256, 0}},
      {"norm_short_rows_k1", &g_norm_short_rows_k1, {1, 0}},
      {"norm_force_general", &g_norm_force_general, {1, 0}},
      {"l2_keep", &g_l2_keep, {1, 0}},
      {"embed_direct", &g_embed_direct, {1, 0}},
      {"gated_rows_per_group", &g_gated_rows_per_group, {1, 2, 0}},
      {"rope_rows_per_group", &g_rope_rows_per_group, {2, 4, 0}},
      {"rope_lean_k", &g_rope_lean_k, {1, 2, 0}},
      {"rope_staged", &g_rope_staged, {1, 0}},
      {"conv_staged", &g_conv_staged, {1, 0}},
      {"conv_tile", &g_conv_tile, {4, 8, 0}},
      {"hc_fused_inject", &g_hc_fused_inject, {1, 0}},
      {"hc_token_k", &g_hc_token_k, {1, 2, 0}},
      {"hc_row_level", &g_hc_row_level, {1, 0}},
      {"pdl", &g_pdl, {1, 0}},
  };
  if (!key) return -1;
  for (const Key& k : kKeys) {
    if (std::strcmp(key, k.name) != 0) continue;
    bool ok = value == 0;
    for (int i = 0; !ok && k.allowed[i] != 0; ++i) ok = value == k.allowed[i];
    if (!ok) return -1;
    k.slot->store(value, std::memory_order_relaxed);
    return 0;
  }
  return -1;
}

// ---- group 1 -------------------------------------------------------------------------
int halo_b200_add(halo_b200_stream stream, float* y, const float* x, uint32_t n, char* err, size_t errlen) {
  EltArgs a;
  a.op = kOpAdd;
  a.seg[0] = {y, x, y, n};
  return RunElt(a, "halo_add", stream, err, errlen);
}

int halo_b200_axpy(halo_b200_stream stream, float* y, const float* x, float alpha, uint32_t n, char* err,
                   size_t errlen) {
  EltArgs a;
  a.op = kOpAxpy;
  a.seg[0] = {y, x, y, n};
  a.alpha = alpha;
  return RunElt(a, "halo_axpy", stream, err, errlen);
}

// short_rows_k1 forces one octet per thread on rows of <= 256 elements. The default layout is
// shared with the fused norm + RoPE kernel, so the separate kernels agree with the fused one
// bit for bit whenever rot <= d / 2 (the reference's fused-equals-separate property,
// tests/gpu/quant_gpu_test.cpp:2635-2749).
static int RmsnormTyped(halo_b200_stream stream, const void* x, int x_dtype, const float* w, void* y, int y_dtype,
                        uint32_t d, float eps, uint32_t w_stride, uint32_t w_period, int one_plus, uint32_t rows,
                        int short_rows_k1, char* err, size_t errlen) {
  NormArgs a;
  a.x = x;
  a.x_dtype = x_dtype;
  a.w = w;
  a.w_stride = w_stride;
  a.w_period = w_period;
  a.one_plus = one_plus;
  a.y = y;
  a.y_dtype = y_dtype;
  a.d = d;
  a.eps = eps;
  a.rows = rows;
  a.short_rows_k1 = short_rows_k1;
  REQUIRE(rows == 0 || y != nullptr, "halo_rmsnorm: y is null");
  return RunNorm(a, "halo_rmsnorm", stream, err, errlen);
}

int halo_b200_rmsnorm_ex(halo_b200_stream stream, const void* x, int x_dtype, const float* w, void* y, int y_dtype,
                         uint32_t d, float eps, uint32_t w_stride, uint32_t w_period, int one_plus, uint32_t rows,
                         char* err, size_t errlen) {
  return RmsnormTyped(stream, x, x_dtype, w, y, y_dtype, d, eps, w_stride, w_period, one_plus, rows, 0, err, errlen);
}

int halo_b200_rmsnorm(halo_b200_stream stream, const float* x, const float* w_all, float* y, uint32_t d, float eps,
                      uint32_t w_stride, uint32_t nvec, char* err, size_t errlen) {
  REQUIRE(w_all != nullptr, "halo_rmsnorm: w_all is null");
  // vector b uses gamma b * w_stride: a period of nvec rows
  return RmsnormTyped(stream, x, kF32, w_all, y, kF32, d, eps, w_stride, w_stride ? nvec : 1, 0, nvec, 0, err, errlen);
}

int halo_b200_rmsnorm_rows(halo_b200_stream stream, const float* x, const float* w_all, float* y, uint32_t d,
                           float eps, uint32_t w_stride, uint32_t w_period, uint32_t rows, char* err, size_t errlen) {
  REQUIRE(w_all != nullptr, "halo_rmsnorm_rows: w_all is null");
  REQUIRE(w_period > 0, "halo_rmsnorm_rows: w_period is 0");
  return RmsnormTyped(stream, x, kF32, w_all, y, kF32, d, eps, w_stride, w_period, 0, rows, 0, err, errlen);
}
int halo_b200_rmsnorm_rows_r16(halo_b200_stream stream, const uint16_t* x, const float* w_all, float* y, uint32_t d,
                               float eps, uint32_t w_stride, uint32_t w_period, uint32_t rows, char* err,
                               size_t errlen) {
  REQUIRE(w_all != nullptr, "halo_rmsnorm_rows_r16: w_all is null");
  REQUIRE(w_period > 0, "halo_rmsnorm_rows_r16: w_period is 0");
  return RmsnormTyped(stream, x, kF16, w_all, y, kF32, d, eps, w_stride, w_period, 0, rows, 0, err, errlen);
}
int halo_b200_rmsnorm_rows_rb(halo_b200_stream stream, const uint16_t* x, const float* w_all, float* y, uint32_t d,
                              float eps, uint32_t w_stride, uint32_t w_period, uint32_t rows, char* err,
                              size_t errlen) {
  REQUIRE(w_all != nullptr, "halo_rmsnorm_rows_rb: w_all is null");
  REQUIRE(w_period > 0, "halo_rmsnorm_rows_rb: w_period is 0");
  return RmsnormTyped(stream, x, kBF16, w_all, y, kF32, d, eps, w_stride, w_period, 0, rows, 0, err, errlen);
}

int halo_b200_rmsnorm_rows_h(halo_b200_stream stream, const void* x, int x_dtype, const float* w_all, float* y,
                             uint16_t* y16, uint32_t d, float eps, uint32_t w_stride, uint32_t w_period,
                             const float* iw, float* ipart, uint32_t irows, uint32_t y16_tokens, uint32_t rows,
                             char* err, size_t errlen) {
  REQUIRE(rows == 0 || (w_all && y && y16), "halo_rmsnorm_rows_h: null pointer");
  REQUIRE(w_period > 0, "halo_rmsnorm_rows_h: w_period is 0");
  if (iw) {
    // with the next projection's partial products: the grouped-norm kernel without a combine
    REQUIRE(w_period == 1 || w_stride == d, "halo_rmsnorm_rows_h: iw needs gamma rows d apart (w_stride == d)");
    REQUIRE(rows % w_period == 0, "halo_rmsnorm_rows_h: rows must be a multiple of w_period");
    HcArgs h{};
    h.res = const_cast<void*>(x);
    h.res_dtype = x_dtype;
    h.out_dtype = kF32;
    h.w = w_all;
    h.y = y;
    h.y_dtype = kF32;
    h.y16 = y16;
    h.y16_tokens = y16_tokens;
    h.iw = iw;
    h.ipart = ipart;
    h.irows = irows;
    h.hc = w_period;
    h.h = d;
    h.tokens = rows / w_period;
    h.eps = eps;
    return RunHc(h, "halo_rmsnorm_rows_h", stream, err, errlen);
  }
  NormArgs a;
  a.x = x;
  a.x_dtype = x_dtype;
  a.w = w_all;
  a.w_stride = w_stride;
  a.w_period = w_period;
  a.y = y;
  a.y_dtype = kF32;
  a.y16 = y16;
  a.y16_tokens = y16_tokens;
  a.kb_period = w_period;
  a.d = d;
  a.eps = eps;
  a.rows = rows;
  return RunNorm(a, "halo_rmsnorm_rows_h", stream, err, errlen);
}

int halo_b200_rmsnorm_y(halo_b200_stream stream, float* x, const float* w_all, uint32_t d, float eps,
                        uint32_t w_stride, uint32_t stride, uint32_t nvec, uint32_t batch, char* err, size_t errlen) {
  REQUIRE(w_all != nullptr, "halo_rmsnorm_y: w_all is null");
  NormArgs a;
  a.x = x;
  a.y = x;
  a.w = w_all;
  a.w_stride = w_stride;
  a.w_period = w_stride ? nvec : 1;  // vector v of every entry uses gamma v * w_stride
  a.d = d;
  a.eps = eps;
  a.rows = nvec * batch;
  a.rows_per_entry = nvec;
  a.entry_stride = stride;
  return RunNorm(a, "halo_rmsnorm_y", stream, err, errlen);
}

int halo_b200_add_rmsnorm(halo_b200_stream stream, void* res, const void* delta, int res_dtype, const float* w,
                          int one_plus, void* xn, int xn_dtype, uint8_t* xn_q8_0, int8_t* xq, float* xd, uint32_t d,
                          float eps, uint32_t rows, char* err, size_t errlen) {
  if (rows == 0) return Done(cudaSuccess, "halo_add_rmsnorm", err, errlen);
  REQUIRE(res != nullptr, "halo_add_rmsnorm: res is null");
  REQUIRE(xn || xn_q8_0 || xq, "halo_add_rmsnorm: no normalized output requested");
  NormArgs a;
  a.x = res;
  a.x_dtype = res_dtype;
  a.delta = delta;
  a.res = delta ? res : nullptr;
  a.w = w;
  a.one_plus = one_plus;
  a.y = xn;
  a.y_dtype = xn_dtype;
  a.q8_0 = xn_q8_0;
  a.xq = xq;
  a.xd = xd;
  a.d = d;
  a.eps = eps;
  a.rows = rows;
  return RunNorm(a, "halo_add_rmsnorm", stream, err, errlen);
}

int halo_b200_quantize_q8_rows(halo_b200_stream stream, const float* x, int8_t* xq, float* xd, uint32_t cols,
                               uint32_t rows, char* err, size_t errlen) {
  QuantArgs a;
  a.x = x;
  a.x_stride = cols;
  a.cols = cols;
  a.rows = rows;
  a.xq = xq;
  a.xd = xd;
  REQUIRE(rows == 0 || (xq && xd), "halo_quantize_q8_rows: null output");
  return RunQuant(a, "halo_quantize_q8_rows", stream, err, errlen);
}

int halo_b200_quantize_q8_kblocked(halo_b200_stream stream, const float* x, int8_t* xq, float* xd, uint32_t cols,
                                   uint32_t tokens, char* err, size_t errlen) {
  QuantArgs a;
  a.x = x;
  a.x_stride = cols;
  a.cols = cols;
  a.rows = tokens;
  a.xq = xq;
  a.xd = xd;
  a.kb_tokens = tokens;
  if (tokens == 0) return Done(cudaSuccess, "", err, errlen);
  REQUIRE(xq && xd, "halo_quantize_q8_kblocked: null output");
  return RunQuant(a, "halo_quantize_q8_kblocked", stream, err, errlen);
}

int halo_b200_q8x_cols(halo_b200_stream stream, const float* x, uint32_t xstride, uint32_t cols, int8_t* xq,
                       float* xs, int8_t* xq2, float* xs2, uint32_t batch, char* err, size_t errlen) {
  QuantArgs a;
  a.x = x;
  a.x_stride = xstride;
  a.cols = cols;
  a.rows = batch;
  a.xq = xq;
  a.xd = xs;
  a.xq2 = xq2;
  a.xd2 = xs2;
  REQUIRE(batch == 0 || (xq && xs), "halo_q8x_cols: null output");
  return RunQuant(a, "halo_q8x_cols", stream, err, errlen);
}

int halo_b200_hc_norm_q8x(halo_b200_stream stream, const float* res, const float* scale, const float* norm_w,
                          float* xn, uint32_t hc, uint32_t h, int8_t* xq, float* xs, int8_t* xq2, float* xs2,
                          uint32_t batch, char* err, size_t errlen) {
  QuantArgs a;
  a.x = res;
  a.x_stride = static_cast<uint64_t>(hc) * h;
  a.cols = hc * h;
  a.rows = batch;
  a.xq = xq;
  a.xd = xs;
  a.xq2 = xq2;
  a.xd2 = xs2;
  a.pre_scale = scale;
  a.pre_w = norm_w;
  a.pre_h = h;
  a.xn = xn;
  if (batch == 0 || a.cols == 0) return Done(cudaSuccess, "", err, errlen);
  REQUIRE(scale && norm_w && xn && xq && xs, "halo_hc_norm_q8x: null pointer");
  return RunQuant(a, "halo_hc_norm_q8x", stream, err, errlen);
}

int halo_b200_encode_q8_0_rows(halo_b200_stream stream, const void* x, int x_dtype, uint8_t* out, uint32_t cols,
                               uint32_t rows, char* err, size_t errlen) {
  QuantArgs a;
  a.x = x;
  a.x_dtype = x_dtype;
  a.x_stride = cols;
  a.cols = cols;
  a.rows = rows;
  a.q8_0 = out;
  REQUIRE(rows == 0 || out != nullptr, "halo_encode_q8_0_rows: out is null");
  return RunQuant(a, "halo_encode_q8_0_rows", stream, err, errlen);
}

// ---- group 2 -------------------------------------------------------------------------
int halo_b200_l2norm_ex(halo_b200_stream stream, const void* x, int x_dtype, void* y, int y_dtype, uint32_t d,
                        float eps, uint32_t rows, char* err, size_t errlen) {
  NormArgs a;
  a.x = x;
  a.x_dtype = x_dtype;
  a.y = y;
  a.y_dtype = y_dtype;
  a.d = d;
  a.eps = eps;
  a.rows = rows;
  a.l2 = 1;
  REQUIRE(rows == 0 || y != nullptr, "halo_l2norm: y is null");
  return RunNorm(a, "halo_l2norm", stream, err, errlen);
}

int halo_b200_l2norm(halo_b200_stream stream, float* x, uint32_t d, float eps, uint32_t nvec, char* err,
                     size_t errlen) {
  return halo_b200_l2norm_ex(stream, x, kF32, x, kF32, d, eps, nvec, err, errlen);
}

int halo_b200_gated_norm_ex(halo_b200_stream stream, const void* o, int o_dtype, const float* w, const void* z,
                            int z_dtype, void* y, int y_dtype, uint32_t d, float eps, uint32_t mode, uint32_t rows,
                            char* err, size_t errlen) {
  GatedArgs a;
  a.o = o;
  a.o_dtype = o_dtype;
  a.w = w;
  a.z = z;
  a.z_dtype = z_dtype;
  a.y = y;
  a.y_dtype = y_dtype;
  a.d = d;
  a.eps = eps;
  a.mode = mode;
  a.rows = rows;
  return RunGated(a, "halo_gated_norm", stream, err, errlen);
}

int halo_b200_gated_norm(halo_b200_stream stream, float* o, const float* w, const float* z, uint32_t d, float eps,
                         uint32_t mode, uint32_t rows, char* err, size_t errlen) {
  return halo_b200_gated_norm_ex(stream, o, kF32, w, z, kF32, o, kF32, d, eps, mode, rows, err, errlen);
}
int halo_b200_gated_norm_h(halo_b200_stream stream, const float* o, const float* w, const float* z, uint16_t* y16,
                           uint32_t d, float eps, uint32_t mode, uint32_t rows, char* err, size_t errlen) {
  return halo_b200_gated_norm_ex(stream, o, kF32, w, z, kF32, y16, kF16, d, eps, mode, rows, err, errlen);
}
int halo_b200_gated_norm_hz(halo_b200_stream stream, const float* o, const float* w, const uint16_t* z,
                            uint16_t* y16, uint32_t d, float eps, uint32_t mode, uint32_t rows, char* err,
                            size_t errlen) {
  return halo_b200_gated_norm_ex(stream, o, kF32, w, z, kF16, y16, kF16, d, eps, mode, rows, err, errlen);
}
int halo_b200_gated_norm_h128w(halo_b200_stream stream, const float* o, const float* w, const float* z,
                               uint16_t* y16, uint32_t rows, float eps, uint32_t mode, char* err, size_t errlen) {
  return halo_b200_gated_norm_ex(stream, o, kF32, w, z, kF32, y16, kF16, 128, eps, mode, rows, err, errlen);
}
int halo_b200_gated_norm_h128w_hh(halo_b200_stream stream, const uint16_t* o, const float* w, const uint16_t* z,
                                  uint16_t* y16, uint32_t rows, float eps, uint32_t mode, char* err, size_t errlen) {
  return halo_b200_gated_norm_ex(stream, o, kF16, w, z, kF16, y16, kF16, 128, eps, mode, rows, err, errlen);
}

// ---- group 3 -------------------------------------------------------------------------
int halo_b200_rope_ex(halo_b200_stream stream, void* q, uint32_t q_heads, void* k, uint32_t k_heads, int dtype,
                      uint32_t head_dim, uint32_t rotary_dim, float theta, uint32_t tokens, const uint32_t* params,
                      uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale, uint32_t* pos_out, char* err,
                      size_t errlen) {
  RopeArgs a;
  a.x = q;
  a.dtype = dtype;
  a.tokens = tokens;
  a.heads = q_heads;
  a.hd = head_dim;
  a.rot = rotary_dim;
  a.token_stride = static_cast<uint64_t>(q_heads) * head_dim;
  a.x2 = k_heads ? k : nullptr;
  a.heads2 = k ? k_heads : 0;
  a.token_stride2 = static_cast<uint64_t>(k_heads) * head_dim;
  a.pos.params = params;
  a.pos.pstride = pstride;
  a.pos.slot = slot;
  a.pos.pos0 = pos0;
  a.pos.scale = scale;
  a.pos_out = pos_out;
  return RunRope(a, theta, "halo_rope_neox", stream, err, errlen);
}

int halo_b200_rope_neox(halo_b200_stream stream, float* x, uint32_t head_dim, uint32_t rotary_dim, uint32_t pos,
                        float theta, uint32_t heads, char* err, size_t errlen) {
  return halo_b200_rope_ex(stream, x, heads, nullptr, 0, kF32, head_dim, rotary_dim, theta, 1, nullptr, 0, 0, pos, 1,
                           nullptr, err, errlen);
}

int halo_b200_rope_neox_rows(halo_b200_stream stream, float* x, uint32_t head_dim, uint32_t rotary_dim,
                             uint32_t pos0, uint32_t heads, float theta, uint32_t rows, char* err, size_t errlen) {
  REQUIRE(heads > 0, "halo_rope_neox_rows: heads is 0");
  // Row r is head r % heads of token r / heads. A trailing partial token (rows not a multiple
  // of heads) is rotated too, as the reference's per-row grid would.
  const uint32_t full = rows / heads, rest = rows % heads;
  int rc = halo_b200_rope_ex(stream, x, heads, nullptr, 0, kF32, head_dim, rotary_dim, theta, full, nullptr, 0, 0,
                             pos0, 1, nullptr, err, errlen);
  if (rc == 0 && rest)
    rc = halo_b200_rope_ex(stream, x + static_cast<size_t>(full) * heads * head_dim, rest, nullptr, 0, kF32, head_dim,
                           rotary_dim, theta, 1, nullptr, 0, 0, pos0 + full, 1, nullptr, err, errlen);
  return rc;
}

int halo_b200_rope_neox_p(halo_b200_stream stream, float* x, const uint32_t* params, uint32_t head_dim,
                          uint32_t rotary_dim, uint32_t slot, uint32_t scale, float theta, uint32_t heads, char* err,
                          size_t errlen) {
  REQUIRE(params != nullptr, "halo_rope_neox_p: params is null");
  return halo_b200_rope_ex(stream, x, heads, nullptr, 0, kF32, head_dim, rotary_dim, theta, 1, params, 0, slot, 0,
                           scale, nullptr, err, errlen);
}

int halo_b200_rope_neox_blocks(halo_b200_stream stream, float* x, uint32_t head_dim, uint32_t rotary_dim,
                               uint32_t b0, uint32_t ratio, float theta, uint32_t nblocks, char* err, size_t errlen) {
  // one head-sized row per pooled block, block b at (b0 + b) * ratio
  return halo_b200_rope_ex(stream, x, 1, nullptr, 0, kF32, head_dim, rotary_dim, theta, nblocks, nullptr, 0, 0, b0,
                           ratio, nullptr, err, errlen);
}

int halo_b200_rope_neox_p_y(halo_b200_stream stream, float* x, const uint32_t* params, uint32_t head_dim,
                            uint32_t rotary_dim, uint32_t slot, uint32_t scale, float theta, uint32_t stride,
                            uint32_t pstride, uint32_t heads, uint32_t batch, char* err, size_t errlen) {
  REQUIRE(params != nullptr, "halo_rope_neox_p_y: params is null");
  RopeArgs a;
  a.x = x;
  a.tokens = batch;  // one "token" per session entry
  a.heads = heads;
  a.hd = head_dim;
  a.rot = rotary_dim;
  a.token_stride = stride;
  a.pos.params = params;
  a.pos.pstride = pstride;
  a.pos.slot = slot;
  a.pos.scale = scale;
  return RunRope(a, theta, "halo_rope_neox_p_y", stream, err, errlen);
}

int halo_b200_split_qgate(halo_b200_stream stream, const float* qg, float* q, float* gate, uint32_t hd,
                          uint32_t rows, char* err, size_t errlen) {
  REQUIRE(rows == 0 || (qg && q && gate), "halo_split_qgate: null pointer");
  SplitArgs a;
  a.qg = qg;
  a.q = q;
  a.gate = gate;
  a.hd = hd;
  a.rows = rows;
  return Done(LaunchSplitQgate(a, S(stream)), "halo_split_qgate", err, errlen);
}

int halo_b200_split_qgate_y(halo_b200_stream stream, const float* qg, float* q, float* gate, uint32_t hd,
                            uint32_t qg_stride, uint32_t q_stride, uint32_t heads, uint32_t batch, char* err,
                            size_t errlen) {
  REQUIRE(heads * batch == 0 || (qg && q && gate), "halo_split_qgate_y: null pointer");
  SplitArgs a;
  a.qg = qg;
  a.q = q;
  a.gate = gate;
  a.hd = hd;
  a.rows = heads * batch;
  a.rows_per_entry = heads;
  a.qg_entry_stride = qg_stride;
  a.q_entry_stride = q_stride;
  return Done(LaunchSplitQgate(a, S(stream)), "halo_split_qgate_y", err, errlen);
}

int halo_b200_norm_rope_ex(halo_b200_stream stream, const void* in, int in_dtype, uint64_t in_row_stride, void* out,
                           int out_dtype, void* gate, void* cache, const float* w, int one_plus, float eps,
                           uint32_t d, uint32_t rotary_dim, uint32_t heads, uint32_t rows, float theta,
                           const uint32_t* params, uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale,
                           uint32_t* pos_out, char* err, size_t errlen) {
  NormRopeArgs a;
  a.in = in;
  a.in_dtype = in_dtype;
  a.in_row_stride = in_row_stride;
  a.out = out;
  a.out_dtype = out_dtype;
  a.gate = gate;
  a.cache = cache;
  a.w = w;
  a.one_plus = one_plus;
  a.eps = eps;
  a.d = d;
  a.rot = rotary_dim;
  a.heads = heads;
  a.rows = rows;
  a.pos.params = params;
  a.pos.pstride = pstride;
  a.pos.slot = slot;
  a.pos.pos0 = pos0;
  a.pos.scale = scale;
  a.pos_out = pos_out;
  return RunNormRope(a, theta, "halo_norm_rope", stream, err, errlen);
}

int halo_b200_norm_rope_qk_ex(halo_b200_stream stream, const void* q_in, uint64_t q_row_stride, void* q_out,
                              void* q_gate, const float* w_q, uint32_t q_heads, const void* k_in, void* k_out,
                              void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype, int out_dtype,
                              int one_plus, float eps, uint32_t d, uint32_t rotary_dim, uint32_t tokens, float theta,
                              const uint32_t* params, uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale,
                              uint32_t* pos_out, char* err, size_t errlen) {
  NormRopeArgs a = QkArgs(q_in, q_row_stride, q_out, q_gate, w_q, q_heads, k_in, k_out, k_cache, w_k, k_heads, in_dtype,
                          out_dtype, one_plus, eps, d, rotary_dim, tokens);
  a.pos.params = params;
  a.pos.pstride = pstride;
  a.pos.slot = slot;
  a.pos.pos0 = pos0;
  a.pos.scale = scale;
  a.pos_out = pos_out;
  return RunNormRope(a, theta, "halo_norm_rope_qk", stream, err, errlen);
}

int halo_b200_rope_table_ex(halo_b200_stream stream, float* table, uint32_t tokens, uint32_t rotary_dim, float theta,
                            const uint32_t* params, uint32_t pstride, uint32_t slot, uint32_t pos0, uint32_t scale,
                            uint32_t* pos_out, char* err, size_t errlen) {
  if (tokens == 0) return Done(cudaSuccess, "halo_rope_table", err, errlen);
  REQUIRE(table != nullptr, "halo_rope_table: table is null");
  REQUIRE(rotary_dim >= 2 && rotary_dim % 2 == 0, "halo_rope_table: rotary_dim %u must be even", rotary_dim);
  REQUIRE(Aligned(table, 4) && Aligned(params, 4) && Aligned(pos_out, 4), "halo_rope_table: pointer not aligned");
  InvFreq f;
  REQUIRE(FillInvFreq(&f, rotary_dim, theta), "halo_rope_table: rotary_dim %u exceeds %d", rotary_dim, 2 * kMaxRotHalf);
  RopeTableArgs a;
  a.table = table;
  a.tokens = tokens;
  a.rot = rotary_dim;
  a.pos.params = params;
  a.pos.pstride = pstride;
  a.pos.slot = slot;
  a.pos.pos0 = pos0;
  a.pos.scale = scale;
  a.pos_out = pos_out;
  return Done(LaunchRopeTable(a, f, S(stream)), "halo_rope_table", err, errlen);
}

int halo_b200_norm_rope_qk_table_ex(halo_b200_stream stream, const void* q_in, uint64_t q_row_stride, void* q_out,
                                    void* q_gate, const float* w_q, uint32_t q_heads, const void* k_in, void* k_out,
                                    void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype, int out_dtype,
                                    int one_plus, float eps, uint32_t d, uint32_t rotary_dim, uint32_t tokens,
                                    const float* table, char* err, size_t errlen) {
  REQUIRE(tokens == 0 || table != nullptr, "halo_norm_rope_qk_table: table is null");
  NormRopeArgs a = QkArgs(q_in, q_row_stride, q_out, q_gate, w_q, q_heads, k_in, k_out, k_cache, w_k, k_heads, in_dtype,
                          out_dtype, one_plus, eps, d, rotary_dim, tokens);
  a.table = table;
  return RunNormRope(a, 0.0f, "halo_norm_rope_qk_table", stream, err, errlen);
}

int halo_b200_split_qgate_norm_rope(halo_b200_stream stream, const float* qg, float* q, float* gate, const float* w,
                                    float eps, uint32_t rotary_dim, uint32_t pos0, uint32_t heads, float theta,
                                    uint32_t hd, uint32_t rows, char* err, size_t errlen) {
  REQUIRE(w != nullptr, "halo_split_qgate_norm_rope: w is null");
  return halo_b200_norm_rope_ex(stream, qg, kF32, 2ull * hd, q, kF32, gate, nullptr, w, 0, eps, hd, rotary_dim, heads,
                                rows, theta, nullptr, 0, 0, pos0, 1, nullptr, err, errlen);
}

int halo_b200_norm_rope_rows(halo_b200_stream stream, float* x, const float* w, float eps, uint32_t d,
                             uint32_t rotary_dim, uint32_t pos0, uint32_t heads, float theta, float* cache,
                             uint32_t rows, char* err, size_t errlen) {
  REQUIRE(w != nullptr, "halo_norm_rope_rows: w is null");
  return halo_b200_norm_rope_ex(stream, x, kF32, d, x, kF32, nullptr, cache, w, 0, eps, d, rotary_dim, heads, rows,
                                theta, nullptr, 0, 0, pos0, 1, nullptr, err, errlen);
}

// ---- group 4 -------------------------------------------------------------------------
int halo_b200_silu_mul_ex(halo_b200_stream stream, const void* g, const void* up, int in_dtype, void* y, int y_dtype,
                          uint64_t n, char* err, size_t errlen) {
  EltArgs a;
  a.op = kOpSiluMul;
  a.seg[0] = {g, up, y, n};
  a.in_dtype = in_dtype;
  a.y_dtype = y_dtype;
  return RunElt(a, "halo_silu_mul", stream, err, errlen);
}

int halo_b200_silu_mul_multi_ex(halo_b200_stream stream, uint32_t nseg, const void* const* g, const void* const* up,
                                void* const* y, const uint64_t* n, int in_dtype, int y_dtype, char* err,
                                size_t errlen) {
  REQUIRE(nseg >= 1 && nseg <= static_cast<uint32_t>(kMaxSegments), "halo_silu_mul_multi: 1..%d segments", kMaxSegments);
  REQUIRE(g && up && y && n, "halo_silu_mul_multi: null argument array");
  EltArgs a;
  a.op = kOpSiluMul;
  a.nseg = static_cast<int>(nseg);
  for (uint32_t i = 0; i < nseg; ++i) a.seg[i] = {g[i], up[i], y[i], n[i]};
  a.in_dtype = in_dtype;
  a.y_dtype = y_dtype;
  return RunElt(a, "halo_silu_mul_multi", stream, err, errlen);
}
int halo_b200_silu_mul(halo_b200_stream stream, float* g, const float* up, uint32_t n, char* err, size_t errlen) {
  return halo_b200_silu_mul_ex(stream, g, up, kF32, g, kF32, n, err, errlen);
}
int halo_b200_silu_mul_h(halo_b200_stream stream, const float* g, const float* up, uint16_t* y, uint32_t n, char* err,
                         size_t errlen) {
  return halo_b200_silu_mul_ex(stream, g, up, kF32, y, kF16, n, err, errlen);
}
int halo_b200_sigmoid_gate(halo_b200_stream stream, float* x, const float* gate, uint32_t n, char* err,
                           size_t errlen) {
  EltArgs a;
  a.op = kOpSigmoidGate;
  a.seg[0] = {x, gate, x, n};
  return RunElt(a, "halo_sigmoid_gate", stream, err, errlen);
}

// ---- group 5 -------------------------------------------------------------------------
int halo_b200_embed_q8_0_ex(halo_b200_stream stream, const uint8_t* w, uint64_t row_bytes, uint32_t vocab,
                            const uint32_t* ids, uint32_t id_stride, uint32_t id_slot, uint32_t tokens, void* out,
                            int out_dtype, uint32_t cols, char* err, size_t errlen) {
  REQUIRE(tokens == 0 || ids != nullptr, "halo_embed_q8_0: ids is null");
  EmbedArgs a;
  a.table = w;
  a.row_bytes = row_bytes;
  a.cols = cols;
  a.ids = ids;
  a.id_stride = id_stride;
  a.id_slot = id_slot;
  a.tokens = tokens;
  a.vocab = vocab;
  a.out = out;
  a.out_dtype = out_dtype;
  return RunEmbed(a, "halo_embed_q8_0", stream, err, errlen);
}

int halo_b200_matvec_q8_0_embed(halo_b200_stream stream, const uint8_t* w, float* out, uint32_t token, uint32_t cols,
                                uint64_t row_bytes, char* err, size_t errlen) {
  EmbedArgs a;
  a.table = w;
  a.row_bytes = row_bytes;
  a.cols = cols;
  a.token = token;
  a.out = out;
  return RunEmbed(a, "halo_matvec_q8_0_embed", stream, err, errlen);
}

int halo_b200_matvec_q8_0_embed_p(halo_b200_stream stream, const uint8_t* w, float* out, const uint32_t* params,
                                  uint32_t cols, uint64_t row_bytes, char* err, size_t errlen) {
  REQUIRE(params != nullptr, "halo_matvec_q8_0_embed_p: params is null");
  EmbedArgs a;
  a.table = w;
  a.row_bytes = row_bytes;
  a.cols = cols;
  a.ids = params;  // params[kHaloToken], slot 0 of the step parameters
  a.id_stride = 0;
  a.out = out;
  return RunEmbed(a, "halo_matvec_q8_0_embed_p", stream, err, errlen);
}

int halo_b200_matvec_q8_0_embed_rows(halo_b200_stream stream, const uint8_t* w, float* out, const uint32_t* params,
                                     uint32_t cols, uint64_t row_bytes, uint32_t tokens, char* err, size_t errlen) {
  REQUIRE(params != nullptr, "halo_matvec_q8_0_embed_rows: params is null");
  EmbedArgs a;
  a.table = w;
  a.row_bytes = row_bytes;
  a.cols = cols;
  a.ids = params;
  a.id_stride = 16;  // parameter rows are 16 uint32 apart, token in slot 0
  a.tokens = tokens;
  a.out = out;
  return RunEmbed(a, "halo_matvec_q8_0_embed_rows", stream, err, errlen);
}

// ---- hyper-connection residual ---------------------------------------------------------------
int halo_b200_hc_combine_norm_ex(halo_b200_stream stream, void* res, int res_dtype, const void* out, int out_dtype,
                                 const float* inject, const float* w_all, int one_plus, void* y, int y_dtype,
                                 uint16_t* y16, uint32_t y16_tokens, float* rscale, const float* iw, float* ipart,
                                 uint32_t irows, int8_t* yq, float* yd, uint32_t hc, uint32_t h, float eps,
                                 uint32_t tokens, char* err, size_t errlen) {
  HcArgs a{};
  a.res = res;
  a.res_dtype = res_dtype;
  a.out = out;
  a.out_dtype = out_dtype;
  a.inject = inject;
  a.w = w_all;
  a.one_plus = one_plus;
  a.y = y;
  a.y_dtype = y_dtype;
  a.y16 = y16;
  a.y16_tokens = y16_tokens;
  a.rscale = rscale;
  a.iw = iw;
  a.ipart = ipart;
  a.irows = irows;
  a.yq = yq;
  a.yd = yd;
  a.hc = hc;
  a.h = h;
  a.eps = eps;
  a.tokens = tokens;
  return RunHc(a, "halo_b200_hc_combine_norm_ex", stream, err, errlen);
}

int halo_b200_hc_combine_norm_moe_ex(halo_b200_stream stream, void* res, int res_dtype, const void* yp, int yp_dtype,
                                     const uint32_t* pos, const float* mw, const void* sx, int sx_dtype,
                                     const float* sg, uint32_t k, const float* inject, const float* w_all,
                                     int one_plus, void* y, int y_dtype, uint16_t* y16, uint32_t y16_tokens,
                                     float* rscale, const float* iw, float* ipart, uint32_t irows, uint32_t hc,
                                     uint32_t h, float eps, uint32_t tokens, char* err, size_t errlen) {
  REQUIRE(sx_dtype == kF32 || sx_dtype == yp_dtype, "halo_b200_hc_combine_norm_moe_ex: sx must be fp32 or of yp's type");
  HcArgs a{};
  a.res = res;
  a.res_dtype = res_dtype;
  a.yp = yp;
  a.out_dtype = yp_dtype;
  a.pos = pos;
  a.mw = mw;
  a.sx = sx;
  a.sx_is_f32 = sx_dtype == kF32;
  a.sg = sg;
  a.k = k;
  a.inject = inject;
  a.w = w_all;
  a.one_plus = one_plus;
  a.y = y;
  a.y_dtype = y_dtype;
  a.y16 = y16;
  a.y16_tokens = y16_tokens;
  a.rscale = rscale;
  a.iw = iw;
  a.ipart = ipart;
  a.irows = irows;
  a.hc = hc;
  a.h = h;
  a.eps = eps;
  a.tokens = tokens;
  return RunHc(a, "halo_b200_hc_combine_norm_moe_ex", stream, err, errlen);
}

int halo_b200_hc_combine_norm_rows(halo_b200_stream stream, void* res, int res_dtype, const float* out,
                                   const float* inject, const float* w_all, float* y, uint16_t* y16, uint32_t hc,
                                   uint32_t h, float eps, const float* iw, float* ipart, uint32_t irows,
                                   float* rscale, uint32_t y16_tokens, uint32_t rows, char* err, size_t errlen) {
  REQUIRE(hc > 0 && rows % hc == 0, "halo_hc_combine_norm_rows: the grid must hold hc rows per token");
  REQUIRE(rows == 0 || (out && inject), "halo_hc_combine_norm_rows: null pointer");
  return halo_b200_hc_combine_norm_ex(stream, res, res_dtype, out, kF32, inject, w_all, 0, y, kF32, y16, y16_tokens,
                                      rscale, iw, ipart, irows, nullptr, nullptr, hc, h, eps, rows / hc, err, errlen);
}

int halo_b200_hc_combine_norm_rows_q8(halo_b200_stream stream, float* res, const float* out, const float* inject,
                                      const float* w_all, float* y, uint16_t* y16, uint32_t hc, uint32_t h, float eps,
                                      const float* iw, float* ipart, uint32_t irows, float* rscale,
                                      uint32_t y16_tokens, int8_t* yq, float* yd, uint32_t rows, char* err,
                                      size_t errlen) {
  REQUIRE(hc > 0 && rows % hc == 0, "halo_hc_combine_norm_rows_q8: the grid must hold hc rows per token");
  REQUIRE(rows == 0 || (out && inject && yq && yd), "halo_hc_combine_norm_rows_q8: null pointer");
  return halo_b200_hc_combine_norm_ex(stream, res, kF32, out, kF32, inject, w_all, 0, y, kF32, y16, y16_tokens, rscale,
                                      iw, ipart, irows, yq, yd, hc, h, eps, rows / hc, err, errlen);
}

int halo_b200_hc_combine_norm_tok(halo_b200_stream stream, void* res, int res_dtype, const float* out,
                                  const float* inject, const float* w_all, uint16_t* y16, uint32_t h, float eps,
                                  const float* iw, float* ipart, uint32_t irows, float* rscale, uint32_t y16_tokens,
                                  uint32_t tokens, char* err, size_t errlen) {
  REQUIRE(tokens == 0 || (out && inject), "halo_hc_combine_norm_tok: null pointer");
  return halo_b200_hc_combine_norm_ex(stream, res, res_dtype, out, kF32, inject, w_all, 0, nullptr, kF32, y16,
                                      y16_tokens, rscale, iw, ipart, irows, nullptr, nullptr, 4, h, eps, tokens, err,
                                      errlen);
}

int halo_b200_hc_combine_norm_tok_moe(halo_b200_stream stream, void* res, int res_dtype, const uint16_t* yp,
                                      const uint32_t* pos, const float* mw, const float* sx, const float* sg,
                                      uint32_t k, const float* inject, const float* w_all, uint16_t* y16, uint32_t h,
                                      float eps, const float* iw, float* ipart, uint32_t irows, float* rscale,
                                      uint32_t y16_tokens, uint32_t tokens, char* err, size_t errlen) {
  REQUIRE(tokens == 0 || (yp && inject), "halo_hc_combine_norm_tok_moe: null pointer");
  return halo_b200_hc_combine_norm_moe_ex(stream, res, res_dtype, yp, kF16, pos, mw, sx, kF32, sg, k, inject, w_all, 0,
                                          nullptr, kF32, y16, y16_tokens, rscale, iw, ipart, irows, 4, h, eps, tokens,
                                          err, errlen);
}

int halo_b200_hc_combine_rows_ex(halo_b200_stream stream, void* res, int res_dtype, const void* out, int out_dtype,
                                 const float* inject, uint32_t hc, uint32_t h, uint32_t tokens, char* err,
                                 size_t errlen) {
  HcEltArgs a{};
  a.op = kHcCombine;
  a.a = res;
  a.a_dtype = res_dtype;
  a.b = out;
  a.b_dtype = out_dtype;
  a.c = inject;
  a.hc = hc;
  a.h = h;
  a.tokens = tokens;
  return RunHcElt(a, "halo_hc_combine_rows", stream, err, errlen);
}

int halo_b200_hc_combine_rows(halo_b200_stream stream, void* res, int res_dtype, const float* out, const float* inject,
                              uint32_t hc, uint32_t h, uint32_t tokens, char* err, size_t errlen) {
  return halo_b200_hc_combine_rows_ex(stream, res, res_dtype, out, kF32, inject, hc, h, tokens, err, errlen);
}

int halo_b200_broadcast_rows_ex(halo_b200_stream stream, void* res, int res_dtype, const void* x, int x_dtype,
                                uint32_t hc, uint32_t h, uint32_t tokens, char* err, size_t errlen) {
  HcEltArgs a{};
  a.op = kHcBroadcast;
  a.a = res;
  a.a_dtype = res_dtype;
  a.b = x;
  a.b_dtype = x_dtype;
  a.hc = hc;
  a.h = h;
  a.tokens = tokens;
  return RunHcElt(a, "halo_broadcast_rows", stream, err, errlen);
}

int halo_b200_broadcast_rows(halo_b200_stream stream, void* res, int res_dtype, const float* x, uint32_t hc,
                             uint32_t h, uint32_t tokens, char* err, size_t errlen) {
  return halo_b200_broadcast_rows_ex(stream, res, res_dtype, x, kF32, hc, h, tokens, err, errlen);
}

int halo_b200_hc_mix_rows_ex(halo_b200_stream stream, const void* xn, const void* gate, void* mixed, int dtype,
                             uint32_t hc, uint32_t h, uint32_t tokens, char* err, size_t errlen) {
  HcEltArgs a{};
  a.op = kHcMix;
  a.a = mixed;
  a.a_dtype = dtype;
  a.b = xn;
  a.b_dtype = dtype;
  a.c = gate;
  a.hc = hc;
  a.h = h;
  a.tokens = tokens;
  return RunHcElt(a, "halo_hc_mix_rows", stream, err, errlen);
}

int halo_b200_hc_mix_rows(halo_b200_stream stream, const float* xn, const float* gate, float* mixed, uint32_t hc,
                          uint32_t h, uint32_t tokens, char* err, size_t errlen) {
  return halo_b200_hc_mix_rows_ex(stream, xn, gate, mixed, kF32, hc, h, tokens, err, errlen);
}

int halo_b200_axpy_sigmoid_rows(halo_b200_stream stream, float* y, const float* x, const float* g, uint32_t n,
                                uint32_t tokens, char* err, size_t errlen) {
  HcEltArgs a{};
  a.op = kAxpySigmoidRows;
  a.a = y;
  a.a_dtype = kF32;
  a.b = x;
  a.b_dtype = kF32;
  a.c = g;
  a.hc = 1;
  a.h = n;
  a.tokens = tokens;
  return RunHcElt(a, "halo_axpy_sigmoid_rows", stream, err, errlen);
}

int halo_b200_inject_reduce(halo_b200_stream stream, const float* ipart, float* inject, uint32_t hc, uint32_t irows,
                            uint32_t tokens, char* err, size_t errlen) {
  if (tokens == 0 || irows == 0) return Done(cudaSuccess, "halo_inject_reduce", err, errlen);
  HcEltArgs a{};
  a.op = kInjectReduce;
  a.a = inject;
  a.a_dtype = kF32;
  a.b = ipart;
  a.b_dtype = kF32;
  a.hc = hc;
  a.h = 1;
  a.irows = irows;
  a.tokens = tokens;
  return RunHcElt(a, "halo_inject_reduce", stream, err, errlen);
}

int halo_b200_res_to_f32(halo_b200_stream stream, float* y, const void* x, int x_dtype, uint32_t n, char* err,
                         size_t errlen) {
  REQUIRE(x_dtype == kF16 || x_dtype == kBF16, "halo_res_to_f32: x must be fp16 or bf16");
  return halo_b200_broadcast_rows_ex(stream, y, kF32, x, x_dtype, 1, n, 1, err, errlen);
}

int halo_b200_hc_norm_scales(halo_b200_stream stream, const float* res, float* scale, uint32_t h, float eps,
                             uint32_t rows, char* err, size_t errlen) {
  REQUIRE(rows == 0 || scale != nullptr, "halo_hc_norm_scales: scale is null");
  NormArgs a;
  a.x = res;
  a.rscale = scale;
  a.d = h;
  a.eps = eps;
  a.rows = rows;
  return RunNorm(a, "halo_hc_norm_scales", stream, err, errlen);
}


// ---- DeltaNet causal conv + SiLU + L2 norm ------------------------------------------------------
int halo_b200_conv_l2norm_ex(halo_b200_stream stream, const void* in, int in_dtype, const float* state, const float* w,
                             void* out, int out_dtype, uint32_t channels, uint32_t kern, uint32_t l2_channels,
                             uint32_t d, float eps, uint32_t tokens, char* err, size_t errlen) {
  ConvArgs a{};
  a.in = in;
  a.in_dtype = in_dtype;
  a.state = const_cast<float*>(state);
  a.w = w;
  a.out = out;
  a.out_dtype = out_dtype;
  a.channels = channels;
  a.kern = kern;
  a.l2_channels = l2_channels;
  a.d = d;
  a.eps = eps;
  a.tokens = tokens;
  return RunConv(a, false, "halo_conv_l2norm_prefill", stream, err, errlen);
}

int halo_b200_conv_state_advance(halo_b200_stream stream, const void* in, int in_dtype, float* state,
                                 uint32_t channels, uint32_t kern, uint32_t tokens, char* err, size_t errlen) {
  ConvArgs a{};
  a.in = in;
  a.in_dtype = in_dtype;
  a.out_dtype = kF32;
  a.state = state;
  a.channels = channels;
  a.kern = kern;
  a.tokens = tokens;
  return RunConv(a, true, "halo_conv_state_advance", stream, err, errlen);
}

int halo_b200_conv_l2norm_prefill(halo_b200_stream stream, const float* in, const float* state, const float* w,
                                  float* out, uint32_t channels, uint32_t kern, uint32_t l2_channels, float eps,
                                  uint32_t d, uint32_t tokens, char* err, size_t errlen) {
  return halo_b200_conv_l2norm_ex(stream, in, kF32, state, w, out, kF32, channels, kern, l2_channels, d, eps, tokens, err,
                                  errlen);
}

int halo_b200_conv_l2norm_prefill8(halo_b200_stream stream, const void* in, int in_dtype, const float* state,
                                   const float* w, void* out, int out_dtype, uint32_t channels, uint32_t tokens,
                                   uint32_t l2_channels, float eps, uint32_t d, char* err, size_t errlen) {
  return halo_b200_conv_l2norm_ex(stream, in, in_dtype, state, w, out, out_dtype, channels, 4, l2_channels, d, eps, tokens,
                                  err, errlen);
}

int halo_b200_conv_l2norm(halo_b200_stream stream, const float* in, float* state, const float* w, float* out,
                          uint32_t channels, uint32_t kern, uint32_t l2_channels, float eps, uint32_t d, char* err,
                          size_t errlen) {
  ConvArgs a{};
  a.in = in;
  a.in_dtype = kF32;
  a.state = state;
  a.w = w;
  a.out = out;
  a.out_dtype = kF32;
  a.channels = channels;
  a.kern = kern;
  a.l2_channels = l2_channels;
  a.d = d;
  a.eps = eps;
  a.tokens = 1;
  a.entries = 1;
  return RunConvStep(a, "halo_conv_l2norm", stream, err, errlen);
}

int halo_b200_conv_l2norm_y(halo_b200_stream stream, const float* in, const uint64_t* tab, uint32_t tstride,
                            uint32_t tslot, const float* w, float* out, uint32_t channels, uint32_t kern,
                            uint32_t l2_channels, float eps, uint32_t stride, uint32_t d, uint32_t entries, char* err,
                            size_t errlen) {
  ConvArgs a{};
  a.in = in;
  a.in_dtype = kF32;
  a.w = w;
  a.out = out;
  a.out_dtype = kF32;
  a.channels = channels;
  a.kern = kern;
  a.l2_channels = l2_channels;
  a.d = d;
  a.eps = eps;
  a.tokens = 1;
  a.entries = entries;
  a.entry_stride = stride;
  a.state_tab = tab;
  a.tstride = tstride;
  a.tslot = tslot;
  REQUIRE(entries == 0 || tab != nullptr, "halo_conv_l2norm_y: the state table is null");
  return RunConvStep(a, "halo_conv_l2norm_y", stream, err, errlen);
}

int halo_b200_conv_step(halo_b200_stream stream, const float* in, float* state, const float* w, float* out,
                        uint32_t channels, uint32_t kern, char* err, size_t errlen) {
  return halo_b200_conv_l2norm(stream, in, state, w, out, channels, kern, 0, 0.0f, 128, err, errlen);
}


// ---- row copies and conversions around the attention block ------------------------------------
int halo_b200_copy_at(halo_b200_stream stream, void* dst, int dst_dtype, const float* src, const uint32_t* params,
                      uint32_t slot, uint32_t stride, uint32_t n, char* err, size_t errlen) {
  REQUIRE(n == 0 || params != nullptr, "halo_copy_at: params is null");
  REQUIRE(dst_dtype == kF32 || dst_dtype == kF16 || dst_dtype == kBF16, "halo_copy_at: unknown dtype");
  HcEltArgs a{};
  a.op = kHcBroadcast;
  a.a = dst;
  a.a_dtype = dst_dtype;
  a.b = src;
  a.b_dtype = kF32;
  a.hc = 1;
  a.h = n;
  a.tokens = 1;
  a.at_params = params;
  a.at_slot = slot;
  a.at_stride = stride;
  return RunHcElt(a, "halo_copy_at", stream, err, errlen);
}

int halo_b200_copy_at_y(halo_b200_stream stream, const uint64_t* tab, uint32_t tstride, uint32_t tslot, int dst_dtype,
                        const float* src, const uint32_t* params, uint32_t slot, uint32_t stride, uint32_t n,
                        uint32_t src_stride, uint32_t pstride, uint32_t entries, char* err, size_t errlen) {
  if (entries == 0 || n == 0) return Done(cudaSuccess, "", err, errlen);
  REQUIRE(tab && src && params, "halo_copy_at_y: null pointer");
  REQUIRE(dst_dtype == kF32 || dst_dtype == kF16 || dst_dtype == kBF16, "halo_copy_at_y: unknown dtype");
  REQUIRE(Aligned(tab, 8) && Aligned(src, 4) && Aligned(params, 4), "halo_copy_at_y: pointer not aligned to its element type");
  REQUIRE(entries <= 65535u, "halo_copy_at_y: more than 65535 entries");
  CopyAtArgs a{};
  a.tab = tab;
  a.tstride = tstride;
  a.tslot = tslot;
  a.dst_dtype = dst_dtype;
  a.src = src;
  a.params = params;
  a.slot = slot;
  a.stride = stride;
  a.n = n;
  a.src_stride = src_stride;
  a.pstride = pstride;
  a.entries = entries;
  return Done(LaunchCopyAtEntries(a, S(stream)), "halo_copy_at_y", err, errlen);
}

int halo_b200_copy(halo_b200_stream stream, float* dst, const float* src, uint32_t n, char* err, size_t errlen) {
  return halo_b200_broadcast_rows_ex(stream, dst, kF32, src, kF32, 1, n, 1, err, errlen);
}

int halo_b200_f16_rows(halo_b200_stream stream, const float* x, uint16_t* y, uint32_t n, char* err, size_t errlen) {
  return halo_b200_broadcast_rows_ex(stream, y, kF16, x, kF32, 1, n, 1, err, errlen);
}

int halo_b200_scale_silu(halo_b200_stream stream, const float* x, void* y, int y_dtype, float scale, uint32_t n,
                         char* err, size_t errlen) {
  REQUIRE(y_dtype == kF32 || y_dtype == kF16, "halo_scale_silu: y must be fp32 or fp16");
  HcEltArgs a{};
  a.op = kScaleSilu;
  a.a = y;
  a.a_dtype = y_dtype;
  a.b = x;
  a.b_dtype = kF32;
  a.hc = 1;
  a.h = n;
  a.tokens = 1;
  a.alpha = scale;
  return RunHcElt(a, "halo_scale_silu", stream, err, errlen);
}


int halo_b200_stage_timeouts(unsigned int* count, char* err, size_t errlen) {
  REQUIRE(count != nullptr, "halo_b200_stage_timeouts: count is null");
  unsigned int conv = 0, rope = 0;
  cudaError_t e = ReadConvStageTimeouts(&conv);
  if (e == cudaSuccess) e = ReadRopeStageTimeouts(&rope);
  *count = conv + rope;
  return Done(e, "halo_b200_stage_timeouts", err, errlen);
}

int halo_b200_conv_stage_timeouts(unsigned int* count, char* err, size_t errlen) {
  return halo_b200_stage_timeouts(count, err, errlen);
}


// ---- MoE combine -----------------------------------------------------------------------------------
int halo_b200_moe_combine_ex(halo_b200_stream stream, const void* yp, int yp_dtype, const uint32_t* pos, const float* mw,
                             const void* sx, int sx_dtype, const float* sg, void* out, int out_dtype, uint32_t k,
                             uint32_t n, uint32_t tokens, char* err, size_t errlen) {
  REQUIRE(sx == nullptr || sx_dtype == kF32 || sx_dtype == yp_dtype, "halo_b200_moe_combine_ex: sx must be fp32 or of yp's type");
  MoeCombineArgs a{};
  a.yp = yp;
  a.yp_dtype = yp_dtype;
  a.pos = pos;
  a.mw = mw;
  a.sx = sx;
  a.sx_is_f32 = sx_dtype == kF32;
  a.sg = sg;
  a.out = out;
  a.out_dtype = out_dtype;
  a.k = k;
  a.n = n;
  a.tokens = tokens;
  return RunMoeCombine(a, "halo_moe_combine", stream, err, errlen);
}

int halo_b200_moe_combine_grouped(halo_b200_stream stream, const uint16_t* yp, const uint32_t* pos, const float* w,
                                  float* out, uint32_t k, uint32_t n, uint32_t tokens, char* err, size_t errlen) {
  return halo_b200_moe_combine_ex(stream, yp, kF16, pos, w, nullptr, kF32, nullptr, out, kF32, k, n, tokens, err, errlen);
}

int halo_b200_moe_combine_shared(halo_b200_stream stream, const uint16_t* yp, const uint32_t* pos, const float* w,
                                 const float* x, const float* g, float* out, uint32_t k, uint32_t n, uint32_t tokens,
                                 char* err, size_t errlen) {
  REQUIRE(tokens == 0 || (x && g), "halo_moe_combine_shared: null pointer");
  return halo_b200_moe_combine_ex(stream, yp, kF16, pos, w, x, kF32, g, out, kF32, k, n, tokens, err, errlen);
}

int halo_b200_moe_combine(halo_b200_stream stream, const float* part, const float* weights, float* out, uint32_t slots,
                          uint32_t n, char* err, size_t errlen) {
  return halo_b200_moe_combine_ex(stream, part, kF32, nullptr, weights, nullptr, kF32, nullptr, out, kF32, slots, n, 1, err,
                                  errlen);
}

int halo_b200_axpy_slot(halo_b200_stream stream, float* y, const float* x, const float* weights, uint32_t slot,
                        uint32_t n, char* err, size_t errlen) {
  REQUIRE(n == 0 || weights != nullptr, "halo_axpy_slot: weights is null");
  MoeCombineArgs a{};
  a.yp = x;
  a.yp_dtype = kF32;
  a.mw = weights ? weights + slot : nullptr;
  a.out = y;
  a.out_dtype = kF32;
  a.k = 1;
  a.n = n;
  a.tokens = 1;
  a.accumulate = 1;
  return RunMoeCombine(a, "halo_axpy_slot", stream, err, errlen);
}


}  // extern "C"
