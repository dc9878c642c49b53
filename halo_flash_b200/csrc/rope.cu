// Partial NEOX rotary embedding for sm_100a, standalone and fused behind the
// per-head RMSNorm. Replaces halo_rope_neox, _rows, _p, _blocks, _p_y,
// halo_split_qgate(_y), halo_split_qgate_norm_rope and halo_norm_rope_rows
// (src/kernels/core.hip:275-311, 356-443; src/kernels/batch_decode.hip:1679-1697);
// arithmetic follows src/model/cpu_ops.cpp:168-185.
//
// The angle must be bit-identical to the CPU operator's: a one-ulp difference in
// the inverse frequency becomes 1e-2 rad at position 262143. So the host computes
// pow(theta, -2 i / rot) with the CPU's libm and passes the table as a kernel
// argument; the device does the single fp32 multiply float(pos) * freq and a
// full-range sincosf.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "stage.cuh"

namespace halo_b200 {
namespace {

__device__ __forceinline__ uint32_t token_pos(const PosSpec& p, uint32_t t) {
  const uint32_t base = p.params ? p.params[static_cast<size_t>(t) * p.pstride + p.slot] : p.pos0 + t;
  return base * p.scale;
}

// Standalone, in place. A CTA owns `tpc` consecutive tokens: it first fills a
// shared (cos, sin) table of tpc x rot/2 entries - one sincosf per token and
// frequency instead of one per head - then rotates every head of both tensors.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kBlock) rope_kernel(const RopeArgs a, const __grid_constant__ InvFreq f,
                                                     const unsigned tpc) {
  pdl_begin();
  extern __shared__ float2 cs[];  // [tpc][half]
  const uint32_t half = a.rot / 2;
  const uint32_t t0 = blockIdx.x * tpc;
  for (uint32_t idx = threadIdx.x; idx < tpc * half; idx += kBlock) {
    const uint32_t t = t0 + idx / half, i = idx % half;
    if (t < a.tokens) {
      const uint32_t pos = token_pos(a.pos, t);
      const float angle = __fmul_rn(static_cast<float>(pos), f.f[i]);
      float sn, c;
      sincosf(angle, &sn, &c);
      cs[idx] = make_float2(c, sn);
      if (i == 0 && a.pos_out) a.pos_out[t] = pos;
    }
  }
  __syncthreads();
  const uint32_t heads_all = a.heads + a.heads2;
  const uint32_t per_head = VEC ? half / 8 : half;
  const uint32_t per_token = heads_all * per_head;
  for (uint32_t item = threadIdx.x; item < tpc * per_token; item += kBlock) {
    const uint32_t tl = item / per_token, r = item % per_token;
    const uint32_t t = t0 + tl;
    if (t >= a.tokens) break;
    const uint32_t h = r / per_head, p = r % per_head;
    T* v = h < a.heads ? static_cast<T*>(a.x) + static_cast<size_t>(t) * a.token_stride + static_cast<size_t>(h) * a.hd
                       : static_cast<T*>(a.x2) + static_cast<size_t>(t) * a.token_stride2 +
                             static_cast<size_t>(h - a.heads) * a.hd;
    const float2* tab = cs + tl * half;
    if constexpr (VEC) {
      float lo[8], hi[8];
      load8(v + p * 8, lo);
      load8(v + half + p * 8, hi);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 t2 = tab[p * 8 + i];
        const float x0 = lo[i], x1 = hi[i];
        lo[i] = x0 * t2.x - x1 * t2.y;
        hi[i] = x0 * t2.y + x1 * t2.x;
      }
      store8(v + p * 8, lo);
      store8(v + half + p * 8, hi);
    } else {
      const float2 t2 = tab[p];
      const float x0 = to_f32(v[p]), x1 = to_f32(v[p + half]);
      v[p] = from_f32<T>(x0 * t2.x - x1 * t2.y);
      v[p + half] = from_f32<T>(x0 * t2.y + x1 * t2.x);
    }
  }
}

// RMSNorm (shared gamma) + RoPE on rows of d <= 256 (one row = one head of one token), for one
// tensor or for Q and K in one launch (the first CTAs take Q's rows, the rest K's: which tensor
// a CTA works on is uniform, so nothing is selected per row). A CTA owns one pass of consecutive
// rows - kBlock / g thread groups x ROWS rows, 32 or 64 rows at d = 256 - so the grid has
// thousands of short-lived CTAs and no tail. It first fills shared cos and signed-sin tables
// for the few tokens those rows belong to - one sincosf per token and frequency instead of one
// per head and lane - then every group loads its rows up front. A group of g lanes (g <= 32,
// shuffles only) owns a row; lane `lir` holds octets lir and (K == 2) lir + g. The sum of squares
// is formed exactly as the standalone norm kernel forms it for the same row length, so fused
// equals norm-then-rope bit for bit. Rotation: lane lir < half/8 holds the first halves of 8
// pairs, lane lir + half/8 their partners, both in the k = 0 octet (the launcher picks K == 2 only
// when rot <= d / 2); the two exchange their normalized values with one shuffle per element and
// each computes own * cos + other * (-/+ sin): the CPU operator's a*c - b*s and a*s + b*c, term
// for term. FULL: every row of the CTA exists and d == 8 K g, so nothing is predicated.
__device__ __forceinline__ uint32_t div_magic(uint32_t n, uint32_t d, uint32_t magic) {
  return magic ? __umulhi(n, magic) : n / d;
}

// Rotate the 8 values of `x` (first or second halves of 8 pairs) given their partners `o`, the
// 8 cosines (c0, c1) and the 8 signed sines (s0, s1): x = x * cos + o * sin. Scalar multiplies
// and adds, each rounded separately (-fmad=false), exactly as the standalone rope kernel and the
// CPU operator compute a*c - b*s and a*s + b*c; a packed mul/add pair was seen to contract into
// an FMA. Everything stays in named registers: arrays indexed here ended up in local memory.
__device__ __forceinline__ void rotate8(Oct& x, const Oct& o, const float4 c0, const float4 c1, const float4 s0,
                                        const float4 s1) {
  x.p[0].x = x.p[0].x * c0.x + o.p[0].x * s0.x;
  x.p[0].y = x.p[0].y * c0.y + o.p[0].y * s0.y;
  x.p[1].x = x.p[1].x * c0.z + o.p[1].x * s0.z;
  x.p[1].y = x.p[1].y * c0.w + o.p[1].y * s0.w;
  x.p[2].x = x.p[2].x * c1.x + o.p[2].x * s1.x;
  x.p[2].y = x.p[2].y * c1.y + o.p[2].y * s1.y;
  x.p[3].x = x.p[3].x * c1.z + o.p[3].x * s1.z;
  x.p[3].y = x.p[3].y * c1.w + o.p[3].y * s1.w;
}
__device__ __forceinline__ float4 scale4(float4 v, float s) { return make_float4(v.x * s, v.y * s, v.z * s, v.w * s); }
__device__ __forceinline__ Oct shuffle_oct(const Oct& x, unsigned src_lane) {
  Oct o;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o.p[i].x = __shfl_sync(kFullMask, x.p[i].x, src_lane);
    o.p[i].y = __shfl_sync(kFullMask, x.p[i].y, src_lane);
  }
  return o;
}

struct RopeCta {
  const void* in;
  uint64_t in_row_stride;
  void* out;
  void* gate;
  void* cache;
  const float* w;
  uint32_t heads, rows, magic;
};

template <typename IT, typename OT, int K, int ROWS, bool FULL, bool GT>
__device__ __forceinline__ void norm_rope_body(const RopeCta t, const NormRopeArgs& a, const InvFreq& f,
                                               const unsigned lg, const uint32_t cta, const float inv_d,
                                               float* smem) {
  const uint32_t half = a.rot / 2;
  const unsigned slots = kBlock >> lg;
  const uint32_t r0 = cta * (slots * ROWS);  // first row of this CTA within its tensor
  uint32_t r1 = r0 + slots * ROWS;
  if (!FULL && r1 > t.rows) r1 = t.rows;
  const uint32_t tok0 = GT ? 0u : div_magic(r0, t.heads, t.magic);
  const uint32_t ntok = GT ? 0u : div_magic(r1 - 1, t.heads, t.magic) - tok0 + 1;
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const unsigned g = 1u << lg;
  const unsigned lir = threadIdx.x & (g - 1);
  const unsigned slot = threadIdx.x >> lg;
  const unsigned octs = a.d >> 3;
  const unsigned hp = a.rot / 16;  // lanes per half of the rotated span
  const bool rotates = lir < 2 * hp;
  const bool low = lir < hp;
  const unsigned src_lane = lane - lir + (rotates ? (low ? lir + hp : lir - hp) : lir);
  const unsigned fbase = (low ? lir : lir - hp) * 8;

  Raw<IT> raw[ROWS][K];
  const IT* src0 = static_cast<const IT*>(t.in) + static_cast<size_t>(r0 + slot) * t.in_row_stride;
  const size_t src_step = static_cast<size_t>(slots) * t.in_row_stride;
#pragma unroll
  for (int u = 0; u < ROWS; ++u) {
    const IT* src = src0 + u * src_step;
    const bool row_ok = FULL || r0 + u * slots + slot < r1;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      if (FULL || (row_ok && j < octs)) raw[u][k] = raw_load(src + j * 8);
      else raw[u][k] = Raw<IT>{};
    }
  }
  if (t.gate) {  // the gate halves of q|gate rows: copied through, after the main loads are out
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
      const IT* src = src0 + u * src_step + a.d;
      IT* gdst = static_cast<IT*>(t.gate) + static_cast<size_t>(r0 + u * slots + slot) * a.d;
      const bool row_ok = FULL || r0 + u * slots + slot < r1;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        if (FULL || (row_ok && j < octs)) oct_store(gdst + j * 8, oct_load(src + j * 8));
      }
    }
  }
  Oct gm[K];
  if (t.w) {  // 1 KiB of gamma, fetched while the rows are in flight
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      gm[k] = (FULL || j < octs) ? oct_load_cached(t.w + j * 8) : oct_zero();
      if (a.one_plus) {
        const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) gm[k].p[i] = __fadd2_rn(one, gm[k].p[i]);
      }
    }
  }
  const float* lane_cos;
  const float* lane_sin;
  uint32_t tok_step;  // floats between two tokens' table rows
  if constexpr (GT) {
    // precomputed table in global memory (L2-resident)
    lane_cos = a.table + fbase;
    lane_sin = a.table + half + fbase;
    tok_step = a.rot;
  } else {
    // The tables are filled while the row loads issued above are in flight.
    float* cosv = smem;                // [ntok][half]
    float* sinv = smem + ntok * half;  // [ntok][half]
    for (uint32_t tl = warp; tl < ntok; tl += kBlock / 32) {
      const uint32_t tok = tok0 + tl;
      const uint32_t pos = token_pos(a.pos, tok);
      for (uint32_t i = lane; i < half; i += 32) {
        const float angle = __fmul_rn(static_cast<float>(pos), f.f[i]);
        float sn, c;
        sincosf(angle, &sn, &c);
        cosv[tl * half + i] = c;
        sinv[tl * half + i] = sn;
      }
      // the CTA holding a token's first row of the first tensor reports its position
      if (lane == 0 && a.pos_out && t.in == a.in && tok * t.heads >= r0) a.pos_out[tok] = pos;
    }
    __syncthreads();
    lane_cos = cosv + fbase;
    lane_sin = sinv + fbase;
    tok_step = half;
  }
  const float sign = low ? -1.0f : 1.0f;  // first halves take -sin, second halves +sin

#pragma unroll
  for (int u = 0; u < ROWS; ++u) {
    const uint32_t row = r0 + u * slots + slot;
    const bool row_ok = FULL || row < r1;
    Oct x[K];
#pragma unroll
    for (int k = 0; k < K; ++k) x[k] = raw_unpack(raw[u][k]);
    if (t.w) {  // the norm kernel's arithmetic for a row of this length, step for step
      float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int k = 0; k < K; ++k) acc = oct_sumsq(x[k], acc);
      const float ss = group_sum_narrow(acc.x + acc.y, g);
      const float scale = rsqrtf(__fmaf_rn(ss, inv_d, a.eps));
#pragma unroll
      for (int k = 0; k < K; ++k) x[k] = oct_mul(oct_scale(x[k], scale), gm[k]);
    }
    const uint32_t tl = row_ok ? div_magic(row, t.heads, t.magic) - tok0 : 0;
    const float* tc = lane_cos + static_cast<size_t>(tl) * tok_step;
    const float* ts = lane_sin + static_cast<size_t>(tl) * tok_step;
    const Oct o = shuffle_oct(x[0], src_lane);
    if (rotates) {
      float4 c0, c1, s0, s1;
      // plain loads in both cases: the global table was written by the kernel before this one, which may still
      // have been running when this grid was scheduled (programmatic dependent launch), so it is not read-only for
      // this kernel's lifetime and must not go through the non-coherent path
      c0 = *reinterpret_cast<const float4*>(tc), c1 = *reinterpret_cast<const float4*>(tc + 4);
      s0 = *reinterpret_cast<const float4*>(ts), s1 = *reinterpret_cast<const float4*>(ts + 4);
      rotate8(x[0], o, c0, c1, scale4(s0, sign), scale4(s1, sign));  // +-sin is exact
    }
    OT* dst = static_cast<OT*>(t.out) + static_cast<size_t>(row) * a.d;
    OT* cdst = t.cache ? static_cast<OT*>(t.cache) + static_cast<size_t>(row) * a.d : nullptr;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      if (FULL || (row_ok && j < octs)) {
        oct_store(dst + j * 8, x[k]);
        if (cdst) oct_store(cdst + j * 8, x[k]);
      }
    }
  }
}

template <typename IT, typename OT, int K, int ROWS, bool GT>
__global__ void __launch_bounds__(kBlock, K * ROWS >= 8 ? 2 : 3) norm_rope_kernel(const NormRopeArgs a, const __grid_constant__ InvFreq f,
                                                             const unsigned lg, const uint32_t ctas1,
                                                             const float inv_d, const uint32_t magic1,
                                                             const uint32_t magic2) {
  pdl_trigger_early();
  extern __shared__ float rope_smem[];
  const unsigned slots = kBlock >> lg;
  const bool second = blockIdx.x >= ctas1;
  RopeCta t;
  if (!second) t = RopeCta{a.in, a.in_row_stride, a.out, a.gate, a.cache, a.w, a.heads, a.rows, magic1};
  else t = RopeCta{a.in2, a.in_row_stride2, a.out2, nullptr, a.cache2, a.w2, a.heads2,
                   ((a.rows + a.heads - 1) / a.heads) * a.heads2, magic2};
  const uint32_t cta = second ? blockIdx.x - ctas1 : blockIdx.x;
  const bool full = (a.d >> 3) == (static_cast<unsigned>(K) << lg) && (cta + 1) * (slots * ROWS) <= t.rows;
  // ahead of the wait for the kernel before this one: a hint to L2 for the CTA's rows where they are one dense span
  // (plain rows, or q|gate rows whose gate halves the CTA copies through anyway)
  if (HALO_PF_ROPE_GENERAL != 0 && threadIdx.x == 0 && full &&
      (t.in_row_stride == a.d || (t.gate && t.in_row_stride == 2 * static_cast<uint64_t>(a.d))) &&
      (t.in_row_stride * sizeof(IT)) % 16 == 0) {
    const size_t span = static_cast<size_t>(slots * ROWS) * t.in_row_stride;
    prefetch_l2_span(static_cast<const IT*>(t.in) + cta * span, static_cast<unsigned>(span * sizeof(IT)));
  }
  pdl_wait_and_trigger();
  if (full) norm_rope_body<IT, OT, K, ROWS, true, GT>(t, a, f, lg, cta, inv_d, rope_smem);
  else norm_rope_body<IT, OT, K, ROWS, false, GT>(t, a, f, lg, cta, inv_d, rope_smem);
}

__device__ __forceinline__ Oct oct_from(float4 a, float4 b) {
  Oct o;
  o.p[0] = make_float2(a.x, a.y), o.p[1] = make_float2(a.z, a.w);
  o.p[2] = make_float2(b.x, b.y), o.p[3] = make_float2(b.z, b.w);
  return o;
}

// The lean fused kernels for the common case: Q (and K) rows that fill whole CTA passes, gammas
// present, rotation table given, no q|gate split and no cache copy. One row per thread group, K
// octets per lane (4 at d = 256: eight lanes own a row and the 64 rotated dims are the first octet
// of each, so every lane of the warp takes part in the exchange), operands as plain arguments,
// nothing predicated; which tensor a pass works on is uniform. The gammas (1 + w applied once) are
// staged in shared memory in the lanes' read order. Same arithmetic, bit for bit, as the general
// kernel above.
struct RopeLeanArgs {  // scalar fields on purpose: indexing a parameter array by tensor copies it to local memory
  const void *in0, *in1;
  void *out0, *out1;
  const float *w0, *w1;
  uint32_t heads0, heads1, magic0, magic1;
  uint32_t ctas0;  // passes (CTAs of the direct kernel, tiles of the staged one) that belong to tensor 0
  uint32_t tiles;  // staged kernel: passes in all
  uint32_t d, rot, lg;
  float eps, inv_d;
  const float* table;
};

constexpr int kLeanCtas(int K) { return K == 4 ? 4 : (K == 2 ? 5 : 6); }

// Element e of a gamma row goes to float4 slot (2 k + e / 4 % 2) g + l of its octet j = k g + l: a lane's two
// 16-byte reads per octet are then contiguous across the lanes of its group (no bank conflicts).
template <bool ONEPLUS>
__device__ __forceinline__ void stage_gamma(float* gs, const float* w, unsigned d, unsigned lg) {
  const unsigned g = 1u << lg;
  for (unsigned e = threadIdx.x; e < d; e += kBlock) {
    const unsigned j = e >> 3, k = j >> lg, l = j & (g - 1), h = (e >> 2) & 1u;
    const float wv = __ldg(w + e);
    gs[((((k << 1) + h) << lg) + l) * 4 + (e & 3u)] = ONEPLUS ? 1.0f + wv : wv;
  }
}

// This token's eight cosines and eight sines for a lane of the rotated span. Plain (coherent) loads: the table
// was written by an earlier kernel of the stream that may still have been running when this grid was scheduled
// (programmatic dependent launch), so it is not read-only for this kernel's lifetime and must not go through
// the non-coherent path.
struct CosSin {
  float4 c0, c1, t0, t1;
};
__device__ __forceinline__ CosSin load_cos_sin(const float* table, uint32_t token, unsigned rot, unsigned lir, unsigned hp) {
  const float* tc = table + static_cast<size_t>(token) * rot + ((lir < hp ? lir : lir - hp) << 3);
  const float* ts = tc + (rot >> 1);
  CosSin r;
  r.c0 = *reinterpret_cast<const float4*>(tc), r.c1 = *reinterpret_cast<const float4*>(tc + 4);
  r.t0 = *reinterpret_cast<const float4*>(ts), r.t1 = *reinterpret_cast<const float4*>(ts + 4);
  return r;
}

// One row held as K octets per lane -> normalized and scaled by the staged gamma. Returns nothing: x is updated.
template <int K>
__device__ __forceinline__ void norm_row(Oct (&x)[K], const float* gs, const unsigned lg, const unsigned lir,
                                         const float eps, const float inv_d) {
  const unsigned g = 1u << lg;
  float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int k = 0; k < K; ++k) acc = oct_sumsq(x[k], acc);
  const float ss = group_sum_narrow(acc.x + acc.y, g);
  const float scale = rsqrtf(__fmaf_rn(ss, inv_d, eps));
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const Oct gm = oct_from(*reinterpret_cast<const float4*>(gs + ((((2 * k) << lg) + lir) << 2)),
                            *reinterpret_cast<const float4*>(gs + ((((2 * k + 1) << lg) + lir) << 2)));
    x[k] = oct_mul(oct_scale(x[k], scale), gm);
  }
}

// Partners of the rotated span exchange their first octet (all 32 lanes call) and rotate.
__device__ __forceinline__ void rotate_row(Oct& x0, const unsigned lir, const unsigned lane, const unsigned hp,
                                           const CosSin& cs) {
  const bool rotates = lir < 2 * hp;
  const bool low = lir < hp;
  const unsigned src_lane = lane - lir + (rotates ? (low ? lir + hp : lir - hp) : lir);
  const Oct o = shuffle_oct(x0, src_lane);
  if (rotates) {
    const float sign = low ? -1.0f : 1.0f;  // first halves take -sin, second halves +sin (exact)
    rotate8(x0, o, cs.c0, cs.c1, scale4(cs.t0, sign), scale4(cs.t1, sign));
  }
}

template <typename IT, typename OT, int K, bool ONEPLUS>
__global__ void __launch_bounds__(kBlock, kLeanCtas(K)) norm_rope_lean_kernel(const RopeLeanArgs a) {
  pdl_begin();
  __shared__ __align__(16) float gs[8 * K * 32];  // d <= 8 K g, g <= 32
  const bool sel = blockIdx.x >= a.ctas0;
  const uint32_t cta = blockIdx.x - (sel ? a.ctas0 : 0u);
  const unsigned lg = a.lg, g = 1u << lg;
  const unsigned lane = threadIdx.x & 31u;
  const unsigned lir = threadIdx.x & (g - 1);
  const uint32_t row = cta * (kBlock >> lg) + (threadIdx.x >> lg);
  const size_t off = static_cast<size_t>(row) * a.d;
  const IT* src = static_cast<const IT*>(sel ? a.in1 : a.in0) + off;
  Raw<IT> rx[K];
#pragma unroll
  for (int k = 0; k < K; ++k) rx[k] = raw_load(src + (((k << lg) + lir) << 3));
  stage_gamma<ONEPLUS>(gs, sel ? a.w1 : a.w0, a.d, lg);  // while the rows are in flight
  __syncthreads();
  const unsigned hp = a.rot >> 4;  // lanes per half of the rotated span
  Oct x[K];
#pragma unroll
  for (int k = 0; k < K; ++k) x[k] = raw_unpack(rx[k]);
  norm_row<K>(x, gs, lg, lir, a.eps, a.inv_d);
  // this token's cos / sin are requested only now: they come from L1 / L2 (a few KB shared by the rows of a token),
  // and holding them in registers while the row is in flight would cost a resident CTA per SM
  CosSin cs = {};
  if (lir < 2 * hp)
    cs = load_cos_sin(a.table, div_magic(row, sel ? a.heads1 : a.heads0, sel ? a.magic1 : a.magic0), a.rot, lir, hp);
  rotate_row(x[0], lir, lane, hp, cs);
  OT* dst = static_cast<OT*>(sel ? a.out1 : a.out0) + off;
#pragma unroll
  for (int k = 0; k < K; ++k) oct_store(dst + (((k << lg) + lir) << 3), x[k]);
}

// The same rows through persistent CTAs that STAGE them: a pass of kBlock / g rows is one contiguous span of
// the tensor (16 KiB at d = 256, bf16), fetched by ONE bulk asynchronous copy into one of two shared-memory
// buffers and counted on an mbarrier. While the CTA normalizes and rotates pass n out of one buffer the copy
// engine fills the other with pass n + 1: bytes in flight cost no registers and the load latency of a pass
// hides behind the arithmetic of the one before, which the direct kernel above (every CTA loads, waits,
// computes, stores, exits) cannot do. Passes are dealt round-robin: CTA c takes c, c + grid, c + 2 grid, ...
// over the passes of tensor 0 followed by those of tensor 1. Results leave with ordinary 16-byte stores, in
// place or not. Every wait is bounded; a wait that runs out is counted and ends the CTA (see stage_wait).
__device__ unsigned int g_stage_timeouts = 0;

template <typename T, int K, bool ONEPLUS>
__global__ void __launch_bounds__(kBlock, 4) norm_rope_staged_kernel(const RopeLeanArgs a) {
  // This persistent kernel lets its successor be scheduled at once whatever its grid (at most four CTAs per SM, below
  // kEarlyTriggerCtas): its launches always fill the GPU, so nothing can pile up behind it (7.4 against 8.4 us at 2048
  // tokens, 12.4 against 13.5 at 4096, with the trigger after the wait).
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t rope_stage[];
  __shared__ __align__(8) unsigned long long bars[2];
  const unsigned lg = a.lg, g = 1u << lg;
  const unsigned rows_per_pass = kBlock >> lg;
  const unsigned pass_elems = rows_per_pass * a.d;
  const unsigned pass_bytes = pass_elems * static_cast<unsigned>(sizeof(T));  // a multiple of 16: d % 8 == 0
  T* bufs = reinterpret_cast<T*>(rope_stage);
  float* gs = reinterpret_cast<float*>(rope_stage + 2 * static_cast<size_t>(pass_bytes));  // [2 tensors][d]
  const unsigned lane = threadIdx.x & 31u, lir = threadIdx.x & (g - 1), slot = threadIdx.x >> lg;
  const unsigned hp = a.rot >> 4;

  auto pass_src = [&](uint32_t p) {
    const bool second = p >= a.ctas0;
    return static_cast<const T*>(second ? a.in1 : a.in0) + static_cast<size_t>(second ? p - a.ctas0 : p) * pass_elems;
  };
  // thread 0 asks the copy engine for pass `p` into buffer `b`
  auto request = [&](uint32_t p, unsigned b) {
    const unsigned bar = smem_addr(&bars[b]);
    stage_expect(bar, pass_bytes);
    stage_copy(smem_addr(bufs + b * pass_elems), pass_src(p), pass_bytes, bar);
  };
  uint32_t p = blockIdx.x;
  const uint32_t stride = gridDim.x;
  // before the wait for the kernel ahead: the barriers, and a hint to L2 for the CTA's first pass
  if (threadIdx.x == 0) {
    stage_init(bars, 2);
    if (HALO_PF_ROPE_STAGED != 0 && p < a.tiles) prefetch_l2_span(pass_src(p), pass_bytes);
  }
  pdl_wait_and_trigger();
  if (p >= a.tiles) return;  // uniform: the whole CTA has no pass
  __syncthreads();
  if (threadIdx.x == 0) {
    request(p, 0);
    if (p + stride < a.tiles) request(p + stride, 1);
  }
  stage_gamma<ONEPLUS>(gs, a.w0, a.d, lg);
  if (a.w1) stage_gamma<ONEPLUS>(gs + a.d, a.w1, a.d, lg);
  __syncthreads();

  for (uint32_t n = 0; p < a.tiles; ++n, p += stride) {
    const unsigned b = n & 1u;
    const bool sel = p >= a.ctas0;
    const uint32_t row = (sel ? p - a.ctas0 : p) * rows_per_pass + slot;
    // this token's cos / sin are requested before the wait: they arrive while the pass is read and reduced
    CosSin cs = {};
    if (lir < 2 * hp)
      cs = load_cos_sin(a.table, div_magic(row, sel ? a.heads1 : a.heads0, sel ? a.magic1 : a.magic0), a.rot, lir, hp);
    // buffer b's (n / 2)-th use: phase parity (n / 2) & 1
    const unsigned done = stage_wait(smem_addr(&bars[b]), (n >> 1) & 1u);
    if (!__syncthreads_and(static_cast<int>(done))) {
      // Never seen. Nothing more is requested, and the copies that may still be in flight into this CTA's shared
      // memory (this buffer, and the other one's next use) get one more bounded wait before the CTA leaves.
      stage_wait(smem_addr(&bars[b]), (n >> 1) & 1u);
      if (p + stride < a.tiles) stage_wait(smem_addr(&bars[b ^ 1u]), ((n + 1) >> 1) & 1u);
      if (threadIdx.x == 0) atomicAdd(&g_stage_timeouts, 1u);
      return;
    }
    const T* mine = bufs + b * pass_elems + slot * a.d;
    Oct x[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const uint4 u = *reinterpret_cast<const uint4*>(mine + (((k << lg) + lir) << 3));
      if constexpr (std::is_same_v<T, bf16>) x[k] = oct_unpack_bf16(u);
      else x[k] = oct_unpack_f16(u);
    }
    norm_row<K>(x, gs + (sel ? a.d : 0u), lg, lir, a.eps, a.inv_d);
    rotate_row(x[0], lir, lane, hp, cs);
    T* dst = static_cast<T*>(sel ? a.out1 : a.out0) + static_cast<size_t>(row) * a.d;
#pragma unroll
    for (int k = 0; k < K; ++k) oct_store(dst + (((k << lg) + lir) << 3), x[k]);
    __syncthreads();  // every thread has read buffer b: refill it with the pass after next
    if (threadIdx.x == 0 && p + 2 * stride < a.tiles) request(p + 2 * stride, b);
  }
}

// One thread per (token, frequency): the rotation table of a step, shared by every layer.
__global__ void __launch_bounds__(kBlock) rope_table_kernel(const RopeTableArgs a, const __grid_constant__ InvFreq f) {
  pdl_begin();
  const uint32_t half = a.rot / 2;
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x;
  const uint32_t t = static_cast<uint32_t>(idx / half), i = static_cast<uint32_t>(idx % half);
  if (t >= a.tokens) return;
  const uint32_t pos = token_pos(a.pos, t);
  const float angle = __fmul_rn(static_cast<float>(pos), f.f[i]);
  float sn, c;
  sincosf(angle, &sn, &c);
  a.table[static_cast<size_t>(t) * a.rot + i] = c;
  a.table[static_cast<size_t>(t) * a.rot + half + i] = sn;
  if (i == 0 && a.pos_out) a.pos_out[t] = pos;
}

template <typename T>
__global__ void __launch_bounds__(kBlock) split_qgate_kernel(const SplitArgs a) {
  pdl_begin();
  const size_t total = static_cast<size_t>(a.rows) * a.hd;
  const T* qg = static_cast<const T*>(a.qg);
  T* q = static_cast<T*>(a.q);
  T* gate = static_cast<T*>(a.gate);
  for (size_t idx = static_cast<size_t>(blockIdx.x) * kBlock + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * kBlock) {
    const uint32_t row = static_cast<uint32_t>(idx / a.hd), i = static_cast<uint32_t>(idx % a.hd);
    size_t in_off = static_cast<size_t>(row) * 2 * a.hd, out_off = static_cast<size_t>(row) * a.hd;
    if (a.rows_per_entry) {
      const uint32_t e = row / a.rows_per_entry, r = row % a.rows_per_entry;
      in_off = static_cast<size_t>(e) * a.qg_entry_stride + static_cast<size_t>(r) * 2 * a.hd;
      out_off = static_cast<size_t>(e) * a.q_entry_stride + static_cast<size_t>(r) * a.hd;
    }
    q[out_off + i] = qg[in_off + i];
    gate[out_off + i] = qg[in_off + a.hd + i];
  }
}

template <typename T>
cudaError_t LaunchRopeT(const RopeArgs& a, const InvFreq& f, cudaStream_t s) {
  const uint32_t half = a.rot / 2;
  const uint32_t per_token = (a.heads + a.heads2) * (a.vec ? half / 8 : half);
  // Enough tokens per CTA for about two items per thread, bounded by the table size.
  unsigned tpc = per_token ? (2 * kBlock + per_token - 1) / per_token : 1;
  if (tpc < 1) tpc = 1;
  if (tpc > 64) tpc = 64;
  if (tpc > a.tokens) tpc = a.tokens;
  const unsigned grid = (a.tokens + tpc - 1) / tpc;
  const size_t smem = static_cast<size_t>(tpc) * half * sizeof(float2);
  if (a.vec) LaunchKernel(rope_kernel<T, true>, grid, kBlock, smem, s, a, f, tpc);
  else LaunchKernel(rope_kernel<T, false>, grid, kBlock, smem, s, a, f, tpc);
  return cudaGetLastError();
}

uint32_t Magic(uint32_t divisor, uint64_t max_n) {
  // floor(n / d) == umulhi(n, ceil(2^32 / d)) whenever n * d < 2^32; 0 = use a real division
  return (divisor > 1 && max_n * divisor < (1ull << 32)) ? static_cast<uint32_t>(((1ull << 32) + divisor - 1) / divisor)
                                                          : 0u;
}

template <typename IT, typename OT, int K>
void LaunchLeanRope(const RopeLeanArgs& l, unsigned grid, bool one_plus, bool staged, cudaStream_t s) {
  if constexpr (std::is_same_v<IT, OT> && sizeof(IT) == 2 && K >= 2) {
    if (staged) {
      // two pass buffers + the two gamma rows; persistent CTAs, four per SM
      const unsigned pass_bytes = (kBlock >> l.lg) * l.d * static_cast<unsigned>(sizeof(IT));
      const size_t smem = 2 * static_cast<size_t>(pass_bytes) + 2 * static_cast<size_t>(l.d) * sizeof(float);
      const unsigned pgrid = l.tiles < 148u * 4u ? l.tiles : 148u * 4u;
      if (one_plus) LaunchKernel(norm_rope_staged_kernel<IT, K, true>, pgrid, kBlock, smem, s, l);
      else LaunchKernel(norm_rope_staged_kernel<IT, K, false>, pgrid, kBlock, smem, s, l);
      return;
    }
  }
  if (one_plus) LaunchKernel(norm_rope_lean_kernel<IT, OT, K, true>, grid, kBlock, 0, s, l);
  else LaunchKernel(norm_rope_lean_kernel<IT, OT, K, false>, grid, kBlock, 0, s, l);
}

template <typename IT, typename OT>
cudaError_t LaunchNormRopeT(const NormRopeArgs& a, const InvFreq& f, cudaStream_t s) {
  const unsigned octs = a.d / 8;
  // Two octets per lane halve the instructions per row; the rotated span must then sit in
  // the first octet of the lanes (rot <= d / 2), which holds for 64-of-256 and 16-of-64.
  int k = (octs >= 2 && a.rot * 2 <= a.d) ? 2 : 1;
  // Rows of 256: four octets per lane, eight lanes per row (the layout the standalone norm kernel picks for
  // such rows, so fused equals separate bit for bit); the rotated span must be the first octet of the lanes.
  if (octs == 32 && a.rot * 4 <= a.d && a.lean_k != 2) k = 4;
  if (a.lean_k == 1 && octs <= 32) k = 1;
  unsigned g = 1, lg = 0;
  while (g * k < octs) g <<= 1, ++lg;
  const unsigned rows_in_flight = k == 4 ? 1u : (a.rows_per_group ? static_cast<unsigned>(a.rows_per_group) : 2u);
  const unsigned rows_per_cta = kBlock / g * rows_in_flight;
  const unsigned tokens = (a.rows + a.heads - 1) / a.heads;
  const uint64_t rows2 = static_cast<uint64_t>(tokens) * a.heads2;
  if (rows2 > 0xFFFFFFFFull) return cudaErrorInvalidValue;
  const unsigned ctas1 = (a.rows + rows_per_cta - 1) / rows_per_cta;
  const unsigned ctas2 = static_cast<unsigned>((rows2 + rows_per_cta - 1) / rows_per_cta);
  const unsigned min_heads = a.heads2 && a.heads2 < a.heads ? a.heads2 : a.heads;
  const unsigned max_tok = rows_per_cta / min_heads + 2;  // tokens a CTA's rows can touch
  const size_t smem = a.table ? 0 : 2 * static_cast<size_t>(max_tok) * (a.rot / 2) * sizeof(float);
  if (smem > 48u * 1024u) return cudaErrorInvalidValue;
  const float inv_d = 1.0f / static_cast<float>(a.d);
  const uint32_t m1 = Magic(a.heads, a.rows), m2 = a.heads2 ? Magic(a.heads2, rows2) : 0u;
  const unsigned grid = ctas1 + ctas2;
  const unsigned rpc1 = kBlock / g;  // rows per CTA of the lean kernel (one row per thread group)
  const bool lean = a.table && octs == static_cast<unsigned>(k) * g && a.w && a.gate == nullptr && a.cache == nullptr &&
                    a.cache2 == nullptr && a.in_row_stride == a.d && a.rows % rpc1 == 0 &&
                    (a.heads2 == 0 || (a.w2 && a.in_row_stride2 == a.d && rows2 % rpc1 == 0)) && !a.force_general;
  if (lean) {
    RopeLeanArgs l = {};
    l.in0 = a.in, l.out0 = a.out, l.w0 = a.w, l.heads0 = a.heads, l.magic0 = m1;
    l.in1 = a.in2, l.out1 = a.out2, l.w1 = a.w2, l.heads1 = a.heads2 ? a.heads2 : 1, l.magic1 = m2;
    l.ctas0 = a.rows / rpc1;
    l.d = a.d, l.rot = a.rot, l.lg = lg, l.eps = a.eps, l.inv_d = inv_d, l.table = a.table;
    const unsigned lgrid = l.ctas0 + static_cast<unsigned>(rows2 / rpc1);
    l.tiles = lgrid;
    // staged (bulk copies into shared memory, persistent CTAs) where the launch has several passes per CTA slot
    // and a pass with its gammas fits the default 48 KiB of dynamic shared memory
    const size_t pass_bytes = static_cast<size_t>(rpc1) * a.d * sizeof(IT);
    const bool staged = a.staged != 0 && std::is_same_v<IT, OT> && sizeof(IT) == 2 && k >= 2 && lgrid > 148u * 4u &&
                        2 * pass_bytes + 2 * a.d * sizeof(float) <= 48u * 1024u;
    if (k == 4) LaunchLeanRope<IT, OT, 4>(l, lgrid, a.one_plus != 0, staged, s);
    else if (k == 2) LaunchLeanRope<IT, OT, 2>(l, lgrid, a.one_plus != 0, staged, s);
    else LaunchLeanRope<IT, OT, 1>(l, lgrid, a.one_plus != 0, false, s);
    return cudaGetLastError();
  }
  if (k == 4) {
    if (a.table) LaunchKernel(norm_rope_kernel<IT, OT, 4, 1, true>, grid, kBlock, 0, s, a, f, lg, ctas1, inv_d, m1, m2);
    else LaunchKernel(norm_rope_kernel<IT, OT, 4, 1, false>, grid, kBlock, smem, s, a, f, lg, ctas1, inv_d, m1, m2);
    return cudaGetLastError();
  }
  if (a.table) {
    if (k == 2 && rows_in_flight == 4) LaunchKernel(norm_rope_kernel<IT, OT, 2, 4, true>, grid, kBlock, 0, s, a, f, lg, ctas1, inv_d, m1, m2);
    else if (k == 2) LaunchKernel(norm_rope_kernel<IT, OT, 2, 2, true>, grid, kBlock, 0, s, a, f, lg, ctas1, inv_d, m1, m2);
    else LaunchKernel(norm_rope_kernel<IT, OT, 1, 2, true>, grid, kBlock, 0, s, a, f, lg, ctas1, inv_d, m1, m2);
  } else {
    if (k == 2 && rows_in_flight == 4) LaunchKernel(norm_rope_kernel<IT, OT, 2, 4, false>, grid, kBlock, smem, s, a, f, lg, ctas1, inv_d, m1, m2);
    else if (k == 2) LaunchKernel(norm_rope_kernel<IT, OT, 2, 2, false>, grid, kBlock, smem, s, a, f, lg, ctas1, inv_d, m1, m2);
    else LaunchKernel(norm_rope_kernel<IT, OT, 1, 2, false>, grid, kBlock, smem, s, a, f, lg, ctas1, inv_d, m1, m2);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t LaunchRope(const RopeArgs& a, const InvFreq& f, cudaStream_t s) {
  if (a.tokens == 0 || a.heads + a.heads2 == 0 || a.rot < 2) return cudaSuccess;
  switch (a.dtype) {
    case kF32: return LaunchRopeT<float>(a, f, s);
    case kF16: return LaunchRopeT<f16>(a, f, s);
    case kBF16: return LaunchRopeT<bf16>(a, f, s);
  }
  return cudaErrorInvalidValue;
}

cudaError_t LaunchNormRope(const NormRopeArgs& a, const InvFreq& f, cudaStream_t s) {
  if (a.rows == 0) return cudaSuccess;
  const int key = a.in_dtype * 3 + a.out_dtype;
  switch (key) {
    case kF32 * 3 + kF32: return LaunchNormRopeT<float, float>(a, f, s);
    case kF32 * 3 + kBF16: return LaunchNormRopeT<float, bf16>(a, f, s);
    case kF32 * 3 + kF16: return LaunchNormRopeT<float, f16>(a, f, s);
    case kBF16 * 3 + kBF16: return LaunchNormRopeT<bf16, bf16>(a, f, s);
    case kBF16 * 3 + kF32: return LaunchNormRopeT<bf16, float>(a, f, s);
    case kF16 * 3 + kF16: return LaunchNormRopeT<f16, f16>(a, f, s);
  }
  return cudaErrorInvalidValue;
}

cudaError_t ReadRopeStageTimeouts(unsigned int* out) {
  return cudaMemcpyFromSymbol(out, g_stage_timeouts, sizeof(unsigned int));
}

cudaError_t LaunchRopeTable(const RopeTableArgs& a, const InvFreq& f, cudaStream_t s) {
  const uint64_t n = static_cast<uint64_t>(a.tokens) * (a.rot / 2);
  if (n == 0) return cudaSuccess;
  const uint64_t grid = (n + kBlock - 1) / kBlock;
  if (grid > 0x7FFFFFFFull) return cudaErrorInvalidValue;
  LaunchKernel(rope_table_kernel, static_cast<unsigned>(grid), kBlock, 0, s, a, f);
  return cudaGetLastError();
}

cudaError_t LaunchSplitQgate(const SplitArgs& a, cudaStream_t s) {
  const size_t total = static_cast<size_t>(a.rows) * a.hd;
  if (total == 0) return cudaSuccess;
  size_t grid = (total + kBlock - 1) / kBlock;
  if (grid > 148u * 16u) grid = 148u * 16u;
  switch (a.dtype) {
    case kF32: LaunchKernel(split_qgate_kernel<float>, static_cast<unsigned>(grid), kBlock, 0, s, a); break;
    case kF16: LaunchKernel(split_qgate_kernel<f16>, static_cast<unsigned>(grid), kBlock, 0, s, a); break;
    case kBF16: LaunchKernel(split_qgate_kernel<bf16>, static_cast<unsigned>(grid), kBlock, 0, s, a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace halo_b200
