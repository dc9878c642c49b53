// Hyper-connection residual ops for sm_100a. The residual of Flash-Next is hc streams of h
// values per token; after every block the block output is scattered into all streams with
// weights 2 sigmoid(inject / hc), and the next mixer normalizes each stream on its own
// (grouped RMSNorm) under one [hc h] gamma. Replaces halo_hc_combine_norm_rows(_r16, _rb, _q8),
// halo_hc_combine_norm_tok(_moe, _moev)(_r16, _rb), halo_hc_combine(_rows), halo_broadcast(_rows),
// halo_hc_mix(_rows), halo_axpy_sigmoid(_rows), halo_inject_reduce, halo_res_to_f32_*
// (src/kernels/core.hip:601-625, 1130-1133, 4105-4496, 4634-4714); arithmetic follows
// src/model/reference.cpp:151-202 (GroupedNorm, HcMix, HcCombine) and 558-578 (expert sum).
//
// hc_combine_norm_kernel: one pass over the residual. A group of g threads owns either a whole
// token (HC = hc streams, the block-output row is loaded, or built from the experts, once) or
// one (token, stream) row (HC = 1, any hc). Thread `lir` holds octets lir, lir + g, ... of every
// stream it owns; the streams stay in registers between the combine, the sums of squares and
// the normalized stores, so each residual byte crosses HBM once per direction.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace halo_b200 {
namespace {

// 1 / (1 + exp(-x)) with the IEEE division (src/model/cpu_ops.cpp:158-160): used for the
// per-row and per-token scalars, whose error would multiply a whole row.
__device__ __forceinline__ float sigmoid_ieee(float x) { return 1.0f / (1.0f + expf(-x)); }

// x + o * a with the product and the sum rounded separately (dst[i] += block_out[i] * w,
// reference.cpp:196): an fp32 residual then equals the CPU operator's bit for bit.
__device__ __forceinline__ Oct oct_axpy_unfused(const Oct& x, const Oct& o, float a) {
  Oct r;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    r.p[i] = make_float2(__fadd_rn(x.p[i].x, __fmul_rn(o.p[i].x, a)), __fadd_rn(x.p[i].y, __fmul_rn(o.p[i].y, a)));
  return r;
}

// The same update for a 16-bit residual: the sum is rounded to 16 bits when it is stored, so the
// product is not rounded on its own and the update is one packed FMA per two values (a quarter of the
// instructions; the bf16 kernel is bound by instruction issue). With a == 1 (zero logits) it is still
// the exact rounded sum x + o.
template <typename RT>
__device__ __forceinline__ Oct oct_combine(const Oct& x, const Oct& o, float a) {
  if constexpr (std::is_same_v<RT, float>) {
    return oct_axpy_unfused(x, o, a);
  } else {
    const float2 a2 = make_float2(a, a);
    Oct r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.p[i] = __ffma2_rn(o.p[i], a2, x.p[i]);
    return r;
  }
}

template <typename T>
__device__ __forceinline__ Raw<T> raw_zero() {
  Raw<T> r;
  if constexpr (std::is_same_v<T, float>) {
    r.a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    r.b = r.a;
  } else {
    r.u = make_uint4(0u, 0u, 0u, 0u);
  }
  return r;
}

// The combined values in the residual's own type: what is stored, and what the norm reads back. A
// 16-bit residual is kept packed (4 registers per octet instead of 8) across the reduction.
__device__ __forceinline__ Raw<float> raw_pack(const Oct& o, float) {
  Raw<float> r;
  r.a = make_float4(o.p[0].x, o.p[0].y, o.p[1].x, o.p[1].y);
  r.b = make_float4(o.p[2].x, o.p[2].y, o.p[3].x, o.p[3].y);
  return r;
}
__device__ __forceinline__ Raw<bf16> raw_pack(const Oct& o, bf16) {
  Raw<bf16> r;
  r.u = oct_pack_bf16(o);
  return r;
}
__device__ __forceinline__ Raw<f16> raw_pack(const Oct& o, f16) {
  Raw<f16> r;
  r.u = oct_pack_f16(o);
  return r;
}
__device__ __forceinline__ void raw_store(float* p, const Raw<float>& r) {
  reinterpret_cast<float4*>(p)[0] = r.a;
  reinterpret_cast<float4*>(p)[1] = r.b;
}
__device__ __forceinline__ void raw_store(bf16* p, const Raw<bf16>& r) { *reinterpret_cast<uint4*>(p) = r.u; }
__device__ __forceinline__ void raw_store(f16* p, const Raw<f16>& r) { *reinterpret_cast<uint4*>(p) = r.u; }

// Resident CTAs per SM the register allocation is held to, from the registers a thread keeps live
// across the reduction (4 per 16-bit octet, 8 per fp32 octet): the kernel waits on HBM, and bytes in
// flight per SM (CTAs x loads per thread) decide its bandwidth.
constexpr int HcMinCtas(int octets, int rt_size) {
  if (rt_size == 2) return octets <= 4 ? 4 : (octets <= 5 ? 3 : 2);
  return octets <= 2 ? 4 : (octets <= 4 ? 3 : (octets <= 5 ? 2 : 1));
}

// HC: streams per thread group (hc, or 1 = one row per group). K: octets per stream per thread.
// MOE: the block output is sum_slot mw * yp[pos] + sigmoid(sg) * sx instead of a stored row.
// LEAN: the common call - a stored block output combined into full tiles (every group exists, every
// thread's octets lie inside the row) with y as the only normalized output - compiled without the
// predicates and without the code of the other outputs (the kernel is bound by instruction issue).
template <typename RT, typename OT, typename YT, int HC, int K, bool MOE, bool LEAN = false>
__global__ void __launch_bounds__(kBlock, HcMinCtas(HC* K, sizeof(RT)))
    hc_combine_norm_kernel(const HcArgs a, const unsigned lg, const float inv_h) {
  pdl_trigger_early();
  if constexpr (LEAN) {  // full tiles: the CTA's groups are one contiguous span of the residual and one of the block output
    if (HALO_PF_HC != 0 && threadIdx.x == 0) {
      const size_t rspan = static_cast<size_t>(kBlock >> lg) * (HC == 1 ? 1u : a.hc) * a.h;
      prefetch_l2_span(static_cast<const RT*>(a.res) + blockIdx.x * rspan, static_cast<unsigned>(rspan * sizeof(RT)));
      if constexpr (HC != 1) {
        const size_t ospan = static_cast<size_t>(kBlock >> lg) * a.h;
        prefetch_l2_span(static_cast<const OT*>(a.out) + blockIdx.x * ospan, static_cast<unsigned>(ospan * sizeof(OT)));
      }
    }
  }
  pdl_wait_and_trigger();
  __shared__ float red[kBlock / 32][HC];
  __shared__ float part[kBlock / 32][HC][8];
  const unsigned g = 1u << lg;
  const unsigned lir = threadIdx.x & (g - 1), lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t grp = blockIdx.x * (kBlock >> lg) + (threadIdx.x >> lg);
  const bool grp_ok = LEAN || grp < (HC == 1 ? a.tokens * a.hc : a.tokens);
  const uint32_t t = HC == 1 ? grp / a.hc : grp;
  const uint32_t s0 = HC == 1 ? grp - t * a.hc : 0u;
  const unsigned octs = a.h >> 3;
  const size_t row0 = (static_cast<size_t>(t) * a.hc + s0) * a.h;
  RT* res = static_cast<RT*>(a.res) + row0;
  const bool combine = LEAN || MOE || a.inject != nullptr;  // false: grouped norm only, the residual is not written

  // scatter weights a_s = 2 sigmoid(inject / hc): lane s of every min(g, 32)-lane segment computes
  // stream s's (first of all, so the logit's load and the exp overlap the row loads below), the others
  // fetch it with a shuffle once the rows have arrived
  const unsigned seg = g < 32u ? g : 32u;
  const unsigned sub = lane & (seg - 1);
  float a_mine = 0.0f;
  if (sub < HC && grp_ok && combine)
    a_mine = 2.0f * sigmoid_ieee(a.inject[static_cast<size_t>(t) * a.hc + s0 + sub] / static_cast<float>(a.hc));
  // every load of the residual and of the block output is issued before any is consumed
  Raw<RT> rr[HC][K];
#pragma unroll
  for (int s = 0; s < HC; ++s)
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      rr[s][k] = (LEAN || (grp_ok && j < octs)) ? raw_load(res + static_cast<size_t>(s) * a.h + j * 8) : raw_zero<RT>();
    }
  Oct o[K];
  if constexpr (!MOE) {
    const OT* out = static_cast<const OT*>(a.out) + static_cast<size_t>(t) * a.h;
    Raw<OT> ro[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      ro[k] = (LEAN || (combine && grp_ok && j < octs)) ? raw_load(out + j * 8) : raw_zero<OT>();
    }
#pragma unroll
    for (int k = 0; k < K; ++k) o[k] = raw_unpack(ro[k]);
  } else {
#pragma unroll
    for (int k = 0; k < K; ++k) o[k] = oct_zero();
    if (grp_ok) {
      // slots in order, then the shared expert: out += weight * down (reference.cpp:558-578)
      const uint32_t* pp = a.pos + static_cast<size_t>(t) * a.k;
      const float* ww = a.mw + static_cast<size_t>(t) * a.k;
#pragma unroll(K == 1 ? 2 : 5)
      for (uint32_t slot = 0; slot < a.k; ++slot) {
        const OT* yr = static_cast<const OT*>(a.yp) + static_cast<size_t>(pp[slot]) * a.h;
        const float ws = ww[slot];
        Raw<OT> ry[K];
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const unsigned j = (k << lg) + lir;
          ry[k] = j < octs ? raw_load(yr + j * 8) : raw_zero<OT>();
        }
#pragma unroll
        for (int k = 0; k < K; ++k) o[k] = oct_axpy_unfused(o[k], raw_unpack(ry[k]), ws);
      }
      const float gs = sigmoid_ieee(a.sg[t]);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        if (j < octs) {
          const size_t off = static_cast<size_t>(t) * a.h + j * 8;
          const Oct x = a.sx_is_f32 ? oct_load(static_cast<const float*>(a.sx) + off)
                                    : oct_load(static_cast<const OT*>(a.sx) + off);
          o[k] = oct_axpy_unfused(o[k], x, gs);
        }
      }
    }
  }

  float as[HC];
#pragma unroll
  for (int s = 0; s < HC; ++s) as[s] = __shfl_sync(kFullMask, a_mine, (lane - sub) + s);

  Raw<RT> kept[HC][K];
  float ss[HC];
#pragma unroll
  for (int s = 0; s < HC; ++s) {
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      // stored in the residual's type; the norm reads the residual as stored (core.hip:4132-4135)
      kept[s][k] = raw_pack(oct_combine<RT>(raw_unpack(rr[s][k]), o[k], as[s]), RT{});
      if (LEAN || (combine && grp_ok && j < octs)) raw_store(res + static_cast<size_t>(s) * a.h + j * 8, kept[s][k]);
      acc = oct_sumsq(raw_unpack(kept[s][k]), acc);
    }
    ss[s] = acc.x + acc.y;
  }
#pragma unroll
  for (int s = 0; s < HC; ++s)
#pragma unroll
    for (unsigned of = 16; of > 0; of >>= 1)
      if (of < g) ss[s] += __shfl_xor_sync(kFullMask, ss[s], of);
  const unsigned wpg = g >> 5, first = wpg ? (warp / wpg) * wpg : 0u;
  if (g > 32u) {
    // second stage, the HC sums sharing one barrier: every lane fetches the partial of warp
    // first + (lane mod wpg) and a butterfly over wpg lanes leaves the total in all of them
    // (4 shared loads and 3 shuffle steps per sum instead of a loop over the group's warps)
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < HC; ++s) red[warp][s] = ss[s];
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < HC; ++s) {
      float tsum = red[first + (lane & (wpg - 1))][s];
#pragma unroll
      for (unsigned of = 4; of > 0; of >>= 1)
        if (of < wpg) tsum += __shfl_xor_sync(kFullMask, tsum, of);
      ss[s] = tsum;
    }
  }

#pragma unroll
  for (int s = 0; s < HC; ++s) {
    const float scale = rsqrtf(__fmaf_rn(ss[s], inv_h, a.eps));
    if (a.rscale && grp_ok && lir == 0) a.rscale[static_cast<size_t>(t) * a.hc + s0 + s] = scale;
    const float* w = a.w + static_cast<size_t>(s0 + s) * a.h;
    Oct v[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      const bool ok = LEAN || (grp_ok && j < octs);
      Oct gm = ok ? oct_load_cached(w + j * 8) : oct_zero();
      if (a.one_plus) {
        const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) gm.p[i] = __fadd2_rn(one, gm.p[i]);
      }
      v[k] = oct_mul(oct_scale(raw_unpack(kept[s][k]), scale), gm);
      const size_t dense = row0 + static_cast<size_t>(s) * a.h + j * 8;
      if (LEAN || (ok && a.y)) oct_store(static_cast<YT*>(a.y) + dense, v[k]);
      if (LEAN || (a.y16 == nullptr && a.yq == nullptr)) continue;
      const uint32_t c = (s0 + s) * a.h + j * 8;  // column within the token's hc h values
      const size_t blocked = (static_cast<size_t>(c >> 6) * a.y16_tokens + t) * 64 + (c & 63u);
      if (ok && a.y16) oct_store(static_cast<f16*>(a.y16) + (a.y16_tokens ? blocked : dense), v[k]);
      if (a.yq) {  // int8 copy per 32 values = the 4 lanes of a quad (all lanes shuffle)
        float arr[8];
        oct_to_array(v[k], arr);
        const float qs = div127(quad_amax(arr));
        const uint2 codes = i8_codes(arr, qs);
        if (ok) {
          *reinterpret_cast<uint2*>(a.yq + blocked) = codes;
          if ((j & 3u) == 0) a.yd[static_cast<size_t>(c >> 5) * a.y16_tokens + t] = qs;
        }
      }
    }
    if (!LEAN && a.iw) {
      // partial products of this normalized stream with the next projection's fp32 rows;
      // halo_inject_reduce (kInjectReduce) sums them over the streams
      float ip[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        float2 acc = make_float2(0.0f, 0.0f);
        if (r < static_cast<int>(a.irows)) {
          const float* iwr = a.iw + (static_cast<size_t>(r) * a.hc + s0 + s) * a.h;
#pragma unroll
          for (int k = 0; k < K; ++k) {
            const unsigned j = (k << lg) + lir;
            if (grp_ok && j < octs) {
              const Oct wv = oct_load_cached(iwr + j * 8);
#pragma unroll
              for (int i = 0; i < 4; ++i) acc = __ffma2_rn(v[k].p[i], wv.p[i], acc);
            }
          }
        }
        float sum = acc.x + acc.y;
#pragma unroll
        for (unsigned of = 16; of > 0; of >>= 1)
          if (of < g) sum += __shfl_xor_sync(kFullMask, sum, of);
        ip[r] = sum;
      }
      if (g > 32u) {
        if (lane == 0) {
#pragma unroll
          for (int r = 0; r < 8; ++r) part[warp][s][r] = ip[r];
        }
      } else if (grp_ok && lir == 0) {
        float* dst = a.ipart + (static_cast<size_t>(t) * a.hc + s0 + s) * a.irows;
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < static_cast<int>(a.irows)) dst[r] = ip[r];
      }
    }
  }
  if (!LEAN && a.iw && g > 32u) {
    __syncthreads();
    if (lir < HC * 8u && grp_ok) {
      const unsigned s = lir >> 3, r = lir & 7u;
      if (r < a.irows) {
        float tsum = 0.0f;
        for (unsigned i = 0; i < wpg; ++i) tsum += part[first + i][s][r];
        a.ipart[(static_cast<size_t>(t) * a.hc + s0 + s) * a.irows + r] = tsum;
      }
    }
  }
}

// Any h, any alignment: one CTA per (token, stream) row, scalar accesses, the row is re-read
// after the reduction. Correctness path for shapes the vector kernel refuses (no expert sum).
template <typename RT, typename OT, typename YT>
__global__ void __launch_bounds__(kBlock) hc_combine_norm_scalar_kernel(const HcArgs a) {
  pdl_begin();
  __shared__ float scratch[kBlock / 32];
  __shared__ float bcast[2];
  const uint32_t row = blockIdx.x, t = row / a.hc, s = row - t * a.hc;
  RT* res = static_cast<RT*>(a.res) + static_cast<size_t>(row) * a.h;
  const OT* out = static_cast<const OT*>(a.out) + static_cast<size_t>(t) * a.h;
  if (threadIdx.x == 0) bcast[0] = 2.0f * sigmoid_ieee(a.inject[row] / static_cast<float>(a.hc));
  __syncthreads();
  const float as = bcast[0];
  float ss = 0.0f;
  for (uint32_t i = threadIdx.x; i < a.h; i += kBlock) {
    float x = std::is_same_v<RT, float> ? __fadd_rn(to_f32(res[i]), __fmul_rn(to_f32(out[i]), as))
                                        : __fmaf_rn(to_f32(out[i]), as, to_f32(res[i]));  // as oct_combine
    res[i] = from_f32<RT>(x);
    x = to_f32(res[i]);
    ss = __fmaf_rn(x, x, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tsum = 0.0f;
    for (int i = 0; i < kBlock / 32; ++i) tsum += scratch[i];
    bcast[1] = rsqrtf(__fmaf_rn(tsum, 1.0f / static_cast<float>(a.h), a.eps));
    if (a.rscale) a.rscale[row] = bcast[1];
  }
  __syncthreads();
  const float scale = bcast[1];
  const float* w = a.w + static_cast<size_t>(s) * a.h;
  float ip[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  for (uint32_t i = threadIdx.x; i < a.h; i += kBlock) {
    const float gm = a.one_plus ? 1.0f + w[i] : w[i];
    const float y = (to_f32(res[i]) * scale) * gm;
    const uint32_t c = s * a.h + i;
    const size_t dense = static_cast<size_t>(row) * a.h + i;
    if (a.y) static_cast<YT*>(a.y)[dense] = from_f32<YT>(y);
    if (a.y16)
      static_cast<f16*>(a.y16)[a.y16_tokens ? (static_cast<size_t>(c >> 6) * a.y16_tokens + t) * 64 + (c & 63u) : dense] =
          __float2half_rn(y);
    if (a.iw)
      for (uint32_t r = 0; r < a.irows; ++r)
        ip[r] = __fmaf_rn(y, a.iw[(static_cast<size_t>(r) * a.hc + s) * a.h + i], ip[r]);
  }
  if (a.iw) {
    for (uint32_t r = 0; r < a.irows; ++r) {
      __syncthreads();
      const float wsum = warp_sum(ip[r]);
      if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = wsum;
      __syncthreads();
      if (threadIdx.x == 0) {
        float tsum = 0.0f;
        for (int i = 0; i < kBlock / 32; ++i) tsum += scratch[i];
        a.ipart[static_cast<size_t>(row) * a.irows + r] = tsum;
      }
    }
  }
}

// ---- elementwise stream ops -------------------------------------------------------------
// One CTA works on one token: thread j handles octet j of the token's h columns for every
// stream, so per-token scalars (scatter weights, the shared-expert gate) are computed once
// per CTA and each [h] row is loaded once however many streams use it.
template <typename AT, typename BT, int OP>
__global__ void __launch_bounds__(kBlock) hc_elt_vec_kernel(const HcEltArgs a, const uint32_t chunks) {
  pdl_trigger_early();
  __shared__ float sc[8];
  const uint32_t t = blockIdx.x / chunks, chunk = blockIdx.x - t * chunks;
  if constexpr (HALO_PF_HC_ELT != 0) {
    // ahead of the wait for the kernel before this one: hints to L2 for the rows this CTA reads, one thread per row
    const unsigned c0 = chunk * kBlock * 8u;
    if (c0 < a.h && threadIdx.x <= 2 * a.hc) {
      const unsigned elems = a.h - c0 < kBlock * 8u ? a.h - c0 : kBlock * 8u;
      const size_t row = static_cast<size_t>(t) * a.h + c0, rows = static_cast<size_t>(t) * a.hc * a.h + c0;
      const unsigned s = threadIdx.x;
      if constexpr (OP == kHcMix) {
        if (s < a.hc) prefetch_l2_span(static_cast<const BT*>(a.b) + rows + static_cast<size_t>(s) * a.h, elems * static_cast<unsigned>(sizeof(BT)));
        else if (s < 2 * a.hc) prefetch_l2_span(static_cast<const BT*>(a.c) + rows + static_cast<size_t>(s - a.hc) * a.h, elems * static_cast<unsigned>(sizeof(BT)));
      } else {
        if (s == 0) prefetch_l2_span(static_cast<const BT*>(a.b) + row, elems * static_cast<unsigned>(sizeof(BT)));
        else if (OP == kHcCombine && s <= a.hc) prefetch_l2_span(static_cast<const AT*>(a.a) + rows + static_cast<size_t>(s - 1) * a.h, elems * static_cast<unsigned>(sizeof(AT)));
        else if (OP == kAxpySigmoidRows && s == 1) prefetch_l2_span(static_cast<const AT*>(a.a) + row, elems * static_cast<unsigned>(sizeof(AT)));
      }
    }
  }
  pdl_wait_and_trigger();
  const unsigned j = chunk * kBlock + threadIdx.x;
  const unsigned octs = a.h >> 3;
  const bool ok = j < octs;
  const float fhc = static_cast<float>(a.hc);
  if constexpr (OP == kHcCombine) {
    if (threadIdx.x < a.hc)
      sc[threadIdx.x] = 2.0f * sigmoid_ieee(static_cast<const float*>(a.c)[static_cast<size_t>(t) * a.hc + threadIdx.x] / fhc);
    __syncthreads();
    if (!ok) return;
    const Oct o = oct_load(static_cast<const BT*>(a.b) + static_cast<size_t>(t) * a.h + j * 8);
    AT* res = static_cast<AT*>(a.a) + static_cast<size_t>(t) * a.hc * a.h + j * 8;
    for (uint32_t s = 0; s < a.hc; ++s) {
      AT* p = res + static_cast<size_t>(s) * a.h;
      oct_store(p, oct_combine<AT>(oct_load(p), o, sc[s]));
    }
  } else if constexpr (OP == kHcBroadcast) {
    if (!ok) return;
    const Oct x = oct_load(static_cast<const BT*>(a.b) + static_cast<size_t>(t) * a.h + j * 8);
    AT* res = static_cast<AT*>(a.a) + static_cast<size_t>(t) * a.hc * a.h + j * 8;
    if (a.at_params) res += static_cast<size_t>(a.at_params[a.at_slot]) * a.at_stride;  // row append (halo_copy_at)
    for (uint32_t s = 0; s < a.hc; ++s) oct_store(res + static_cast<size_t>(s) * a.h, x);
  } else if constexpr (OP == kScaleSilu) {
    if (!ok) return;
    Oct x = oct_scale(oct_load(static_cast<const BT*>(a.b) + static_cast<size_t>(t) * a.h + j * 8), a.alpha);
#pragma unroll
    for (int i = 0; i < 4; ++i) x.p[i] = silu2_f(x.p[i]);
    oct_store(static_cast<AT*>(a.a) + static_cast<size_t>(t) * a.h + j * 8, x);
  } else if constexpr (OP == kHcMix) {
    if (!ok) return;
    const size_t base = static_cast<size_t>(t) * a.hc * a.h + j * 8;
    Oct acc = oct_zero();
    for (uint32_t s = 0; s < a.hc; ++s) {
      const Oct x = oct_load(static_cast<const BT*>(a.b) + base + static_cast<size_t>(s) * a.h);
      const Oct gt = oct_load(static_cast<const BT*>(a.c) + base + static_cast<size_t>(s) * a.h);
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // product and sum rounded separately (reference.cpp:183)
        const float2 sg = sigmoid2_f(gt.p[i]);
        acc.p[i] = make_float2(__fadd_rn(acc.p[i].x, __fmul_rn(x.p[i].x, sg.x)),
                               __fadd_rn(acc.p[i].y, __fmul_rn(x.p[i].y, sg.y)));
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc.p[i] = make_float2(__fdiv_rn(acc.p[i].x, fhc), __fdiv_rn(acc.p[i].y, fhc));
    oct_store(static_cast<AT*>(a.a) + static_cast<size_t>(t) * a.h + j * 8, acc);
  } else {  // kAxpySigmoidRows
    if (threadIdx.x == 0) sc[0] = sigmoid_ieee(static_cast<const float*>(a.c)[t]);
    __syncthreads();
    if (!ok) return;
    AT* y = static_cast<AT*>(a.a) + static_cast<size_t>(t) * a.h + j * 8;
    const Oct x = oct_load(static_cast<const BT*>(a.b) + static_cast<size_t>(t) * a.h + j * 8);
    oct_store(y, oct_axpy_unfused(oct_load(y), x, sc[0]));
  }
}

// One thread per output element, any h and alignment.
template <typename AT, typename BT>
__global__ void __launch_bounds__(kBlock) hc_elt_scalar_kernel(const HcEltArgs a) {
  pdl_begin();
  const float fhc = static_cast<float>(a.hc);
  const bool per_token = a.op == kHcMix || a.op == kAxpySigmoidRows || a.op == kScaleSilu;
  const size_t n = static_cast<size_t>(a.tokens) * (per_token ? 1u : a.hc) * a.h;
  const size_t at = a.at_params ? static_cast<size_t>(a.at_params[a.at_slot]) * a.at_stride : 0;
  for (size_t idx = static_cast<size_t>(blockIdx.x) * kBlock + threadIdx.x; idx < n;
       idx += static_cast<size_t>(gridDim.x) * kBlock) {
    if (a.op == kScaleSilu) {
      static_cast<AT*>(a.a)[idx] = from_f32<AT>(silu_f(__fmul_rn(to_f32(static_cast<const BT*>(a.b)[idx]), a.alpha)));
    } else if (a.op == kHcMix) {
      const size_t t = idx / a.h, i = idx % a.h;
      float acc = 0.0f;
      for (uint32_t s = 0; s < a.hc; ++s) {
        const size_t k = (t * a.hc + s) * a.h + i;
        acc = __fadd_rn(acc, __fmul_rn(to_f32(static_cast<const BT*>(a.b)[k]), sigmoid_f(to_f32(static_cast<const BT*>(a.c)[k]))));
      }
      static_cast<AT*>(a.a)[idx] = from_f32<AT>(__fdiv_rn(acc, fhc));
    } else if (a.op == kAxpySigmoidRows) {
      const float gs = sigmoid_ieee(static_cast<const float*>(a.c)[idx / a.h]);
      AT* y = static_cast<AT*>(a.a) + idx;
      *y = from_f32<AT>(__fadd_rn(to_f32(*y), __fmul_rn(to_f32(static_cast<const BT*>(a.b)[idx]), gs)));
    } else {
      const size_t per = static_cast<size_t>(a.hc) * a.h;
      const size_t t = idx / per, r = idx % per;
      const float x = to_f32(static_cast<const BT*>(a.b)[t * a.h + r % a.h]);
      AT* p = static_cast<AT*>(a.a) + idx + at;
      if (a.op == kHcBroadcast) {
        *p = from_f32<AT>(x);
      } else {
        const float as = 2.0f * sigmoid_ieee(static_cast<const float*>(a.c)[t * a.hc + r / a.h] / fhc);
        *p = from_f32<AT>(std::is_same_v<AT, float> ? __fadd_rn(to_f32(*p), __fmul_rn(x, as)) : __fmaf_rn(x, as, to_f32(*p)));
      }
    }
  }
}

// inject[t][r] = sum over streams, in order, of ipart[(t hc + s) irows + r] (core.hip:4486-4496).
__global__ void __launch_bounds__(kBlock) inject_reduce_kernel(const HcEltArgs a) {
  pdl_begin();
  const uint32_t idx = blockIdx.x * kBlock + threadIdx.x;
  if (idx >= a.tokens * a.irows) return;
  const uint32_t t = idx / a.irows, r = idx - t * a.irows;
  const float* ip = static_cast<const float*>(a.b);
  float acc = 0.0f;
  for (uint32_t s = 0; s < a.hc; ++s) acc = __fadd_rn(acc, ip[(static_cast<size_t>(t) * a.hc + s) * a.irows + r]);
  static_cast<float*>(a.a)[idx] = acc;
}

// ---- inject partial products as a pass of their own -------------------------------------------------
// ipart[t][s][r] = <y[t][s][:], iw[r][s h ..]>. Inside the combine kernel every token re-reads all
// irows x hc x h weights from L2 (131 KB per token at irows 4, H 2048: 537 MB per 4096 tokens, which cost more
// than the combine itself). Here a CTA works on ONE stream with one thread per octet of its h columns; the
// thread keeps its 8 columns of up to 4 weight rows in registers for the whole launch and walks over tokens,
// four at a time. The normalized values must be the fp32 ones the combine kernel had in registers (an fp16 or
// bf16 copy would change the products), so the pass reads either an fp32 y or - as the reference's mix epilogue
// does (src/kernels/core.hip:4097-4099) - rebuilds y = (res * rscale) * gamma from the stored residual, the row
// scales and the gammas, with the combine kernel's own two multiplies: the same bits, 16 KB per token at H 2048
// for a bf16 residual. The
// 4 tokens x 4 rows = 16 partial sums of a thread are reduced over the warp by a transposing butterfly (16
// shuffles for 16 values instead of 80), over the CTA's warps through shared memory with one barrier per batch.
// More than 4 rows: one launch per 4 rows (the second reads y from L2).
__device__ __forceinline__ float warp_reduce16(const float (&v)[16], unsigned lane) {
  // after the step with stride m, a lane holds the values whose index agrees with its lane bits >= m
  float w8[8], w4[4], w2[2];
  const bool b3 = lane & 8u, b2 = lane & 4u, b1 = lane & 2u, b0 = lane & 1u;
#pragma unroll
  for (int i = 0; i < 8; ++i) w8[i] = (b3 ? v[i + 8] : v[i]) + __shfl_xor_sync(kFullMask, b3 ? v[i] : v[i + 8], 8);
#pragma unroll
  for (int i = 0; i < 4; ++i) w4[i] = (b2 ? w8[i + 4] : w8[i]) + __shfl_xor_sync(kFullMask, b2 ? w8[i] : w8[i + 4], 4);
#pragma unroll
  for (int i = 0; i < 2; ++i) w2[i] = (b1 ? w4[i + 2] : w4[i]) + __shfl_xor_sync(kFullMask, b1 ? w4[i] : w4[i + 2], 2);
  float r = (b0 ? w2[1] : w2[0]) + __shfl_xor_sync(kFullMask, b0 ? w2[0] : w2[1], 1);
  return r + __shfl_xor_sync(kFullMask, r, 16);  // value (lane & 15), summed over all 32 lanes
}

constexpr int kInjTokens = 4, kInjRows = 4;

template <typename ST, bool REBUILD, int BLOCK>
__global__ void __launch_bounds__(BLOCK) hc_inject_kernel(const HcArgs a, const ST* __restrict__ src, const uint32_t r0) {
  pdl_begin();
  __shared__ float part[2][4][16][32];  // [buffer][batch of the group][value][warp]
  const uint32_t s = blockIdx.x % a.hc, chunk = blockIdx.x / a.hc, chunks = gridDim.x / a.hc;
  const unsigned octs = a.h >> 3, j = threadIdx.x, lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const unsigned warps = (blockDim.x + 31) >> 5;
  const bool live = j < octs;
  const uint32_t nr = a.irows - r0 < static_cast<uint32_t>(kInjRows) ? a.irows - r0 : static_cast<uint32_t>(kInjRows);
  Oct w[kInjRows];
#pragma unroll
  for (int r = 0; r < kInjRows; ++r)
    w[r] = (live && static_cast<uint32_t>(r) < nr)
               ? oct_load_cached(a.iw + (static_cast<size_t>(r0 + r) * a.hc + s) * a.h + j * 8)
               : oct_zero();
  Oct gm = oct_zero();
  if (REBUILD && live) {
    gm = oct_load_cached(a.w + static_cast<size_t>(s) * a.h + j * 8);
    if (a.one_plus) {
      const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
      for (int i = 0; i < 4; ++i) gm.p[i] = __fadd2_rn(one, gm.p[i]);
    }
  }
  const size_t col_off = static_cast<size_t>(s) * a.h + j * 8;
  const size_t tok_step = static_cast<size_t>(a.hc) * a.h;
  const uint32_t batches = (a.tokens + kInjTokens - 1) / kInjTokens;
  // the rows of the next batch are requested before this batch is computed
  auto fetch = [&](uint32_t bt, Raw<ST> (&dst)[kInjTokens]) {
    const uint32_t t0 = bt * kInjTokens;
#pragma unroll
    for (int u = 0; u < kInjTokens; ++u) {
      if (live && bt < batches && t0 + u < a.tokens) dst[u] = raw_load(src + col_off + static_cast<size_t>(t0 + u) * tok_step);
      else dst[u] = raw_zero<ST>();
    }
  };
  // sums the warps' partials of the group of (up to four) batches ending with the CTA's batch number `last`
  // and writes them: thread b * 16 + v takes value v = u * 4 + r of the group's batch b
  auto flush = [&](uint32_t last) {
    __syncthreads();
    for (uint32_t idx = threadIdx.x; idx < 64; idx += blockDim.x) {
      const uint32_t b = idx >> 4, val = idx & 15u, first = last & ~3u;
      if (first + b <= last) {
        const uint32_t t = (chunk + (first + b) * chunks) * kInjTokens + (val >> 2), r = val & 3u;
        float sum = 0.0f;
        for (unsigned wi = 0; wi < warps; ++wi) sum += part[(last >> 2) & 1u][b][val][wi];
        if (t < a.tokens && r < nr) a.ipart[(static_cast<size_t>(t) * a.hc + s) * a.irows + r0 + r] = sum;
      }
    }
    // the other buffer is written by the next group; this one again only after the next flush's barrier
  };
  Raw<ST> nxt[kInjTokens];
  fetch(chunk, nxt);
  uint32_t n = 0;
  for (uint32_t bt = chunk; bt < batches; bt += chunks, ++n) {
    const uint32_t t0 = bt * kInjTokens;
    Raw<ST> raw[kInjTokens];
#pragma unroll
    for (int u = 0; u < kInjTokens; ++u) raw[u] = nxt[u];
    fetch(bt + chunks, nxt);
    float scale[kInjTokens];
    if constexpr (REBUILD) {
#pragma unroll
      for (int u = 0; u < kInjTokens; ++u)
        scale[u] = t0 + u < a.tokens ? a.rscale[static_cast<size_t>(t0 + u) * a.hc + s] : 0.0f;
    }
    float v[16];
#pragma unroll
    for (int u = 0; u < kInjTokens; ++u) {
      Oct x = raw_unpack(raw[u]);
      if constexpr (REBUILD) x = oct_mul(oct_scale(x, scale[u]), gm);  // the combine kernel's y, bit for bit
#pragma unroll
      for (int r = 0; r < kInjRows; ++r) {
        float2 acc = __fmul2_rn(x.p[0], w[r].p[0]);
        acc = __ffma2_rn(x.p[1], w[r].p[1], acc);
        acc = __ffma2_rn(x.p[2], w[r].p[2], acc);
        acc = __ffma2_rn(x.p[3], w[r].p[3], acc);
        v[u * kInjRows + r] = acc.x + acc.y;
      }
    }
    const float total = warp_reduce16(v, lane);
    if (lane < 16) part[(n >> 2) & 1u][n & 3u][lane][warp] = total;
    if ((n & 3u) == 3u) flush(n);  // the CTA meets once per four batches
  }
  if ((n & 3u) != 0u) flush(n - 1);  // the last, partial group (n is now the number of batches done)
}

template <typename ST, bool REBUILD>
cudaError_t LaunchHcInject(const HcArgs& a, const ST* src, cudaStream_t s) {
  const unsigned threads = (a.h / 8 + 31) / 32 * 32;
  const uint32_t batches = (a.tokens + kInjTokens - 1) / kInjTokens;
  uint32_t chunks = (148u * (threads <= 256 ? 3u : (threads <= 512 ? 2u : 1u))) / a.hc;
  if (chunks < 1) chunks = 1;
  if (chunks > batches) chunks = batches;
  for (uint32_t r0 = 0; r0 < a.irows; r0 += kInjRows) {
    cudaError_t e;
    if (threads <= 256) e = LaunchKernel(hc_inject_kernel<ST, REBUILD, 256>, chunks * a.hc, threads, 0, s, a, src, r0);
    else if (threads <= 512) e = LaunchKernel(hc_inject_kernel<ST, REBUILD, 512>, chunks * a.hc, threads, 0, s, a, src, r0);
    else e = LaunchKernel(hc_inject_kernel<ST, REBUILD, 1024>, chunks * a.hc, threads, 0, s, a, src, r0);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// The combine + norm without the partial products, then the pass above. Possible when the fp32 normalized
// values can be had again: from an fp32 y, or from the stored residual and the row scales.
bool InjectAsSecondPass(const HcArgs& a) {
  return a.iw && !a.fused_inject && a.vec && ((a.y && a.y_dtype == kF32) || a.rscale) &&
         a.h <= 8192u;  // one thread per octet, <= 1024 threads
}

struct HcShape {
  int hc;  // streams per group: a.hc (token level) or 1 (row level)
  int k;
  unsigned lg;
};

// Token level when hc is 4 and a token's streams fit 4 x (1 or 2) octets per thread with at most a
// quarter of the lanes idle (always, if it fits, when the block output is built from the experts:
// rebuilding it per stream would gather every expert row four times); else one row per group
// with the (g, K) of least padding (K = 2 preferred among equals, as the plain row norm found best).
HcShape PickHcShape(const HcArgs& a) {
  const unsigned octs = a.h / 8;
  HcShape sh{};
  if (a.hc == 4 && !a.row_level && octs >= 4) {
    for (unsigned k = (a.token_k == 2 ? 2u : 1u); k <= 2; ++k) {
      const unsigned need = (octs + k - 1) / k;
      unsigned g = 4;
      while (g < need) g <<= 1;
      if (g > 256u) continue;
      if ((g * k - octs) * 4 <= g * k || a.yp) {
        sh.hc = 4;
        sh.k = static_cast<int>(k);
        while ((1u << sh.lg) < g) ++sh.lg;
        return sh;
      }
    }
  }
  static const int kKs[] = {2, 1, 3, 4, 5, 8};
  unsigned best_waste = ~0u;
  for (int k : kKs)
    for (unsigned g = 4; g <= 256u; g <<= 1) {
      if (g * k < octs) continue;
      const unsigned waste = g * k - octs;
      if (waste < best_waste) {
        best_waste = waste;
        sh.hc = 1;
        sh.k = k;
        sh.lg = 0;
        while ((1u << sh.lg) < g) ++sh.lg;
      }
      break;  // larger g only adds padding for this k
    }
  return sh;
}

template <typename RT, typename OT, typename YT, bool MOE>
cudaError_t LaunchHcT(const HcArgs& a, cudaStream_t s) {
  if (!a.vec) {
    if constexpr (MOE) return cudaErrorInvalidValue;
    else return LaunchKernel(hc_combine_norm_scalar_kernel<RT, OT, YT>, a.tokens * a.hc, kBlock, 0, s, a);
  }
  const HcShape sh = PickHcShape(a);
  if (sh.k == 0) return cudaErrorInvalidValue;
  const unsigned per_cta = kBlock >> sh.lg;
  const unsigned groups = sh.hc == 1 ? a.tokens * a.hc : a.tokens;
  const unsigned grid = (groups + per_cta - 1) / per_cta;
  const float inv_h = 1.0f / static_cast<float>(a.h);
  // the lean form: see the kernel
  const bool lean = !MOE && a.out && a.inject && a.y && !a.y16 && !a.yq && !a.iw &&
                    a.h / 8 == (static_cast<unsigned>(sh.k) << sh.lg) && groups % per_cta == 0;
#define HALO_HC_LEAN(HCV, KV)                                                                                      \
  if constexpr (!MOE) {                                                                                            \
    if (lean && sh.hc == HCV && sh.k == KV)                                                                        \
      return LaunchKernel(hc_combine_norm_kernel<RT, OT, YT, HCV, KV, false, true>, grid, kBlock, 0, s, a, sh.lg, inv_h); \
  }
  HALO_HC_LEAN(4, 1)
  HALO_HC_LEAN(1, 2)
  HALO_HC_LEAN(1, 5)
#undef HALO_HC_LEAN
#define HALO_HC_CASE(HCV, KV) \
  if (sh.hc == HCV && sh.k == KV) \
    return LaunchKernel(hc_combine_norm_kernel<RT, OT, YT, HCV, KV, MOE>, grid, kBlock, 0, s, a, sh.lg, inv_h)
  HALO_HC_CASE(4, 1);
  HALO_HC_CASE(4, 2);
  HALO_HC_CASE(1, 1);
  HALO_HC_CASE(1, 2);
  HALO_HC_CASE(1, 3);
  HALO_HC_CASE(1, 4);
  HALO_HC_CASE(1, 5);
  HALO_HC_CASE(1, 8);
#undef HALO_HC_CASE
  return cudaErrorInvalidValue;
}

template <typename RT, typename OT, typename YT>
cudaError_t LaunchHcM(const HcArgs& a, cudaStream_t s) {
  return a.yp ? LaunchHcT<RT, OT, YT, true>(a, s) : LaunchHcT<RT, OT, YT, false>(a, s);
}

template <typename AT, typename BT>
cudaError_t LaunchHcEltT(const HcEltArgs& a, cudaStream_t s) {
  if (a.vec && a.hc <= 8) {
    const uint32_t chunks = (a.h / 8 + kBlock - 1) / kBlock;
    const unsigned grid = a.tokens * chunks;
    switch (a.op) {
      case kHcCombine: return LaunchKernel(hc_elt_vec_kernel<AT, BT, kHcCombine>, grid, kBlock, 0, s, a, chunks);
      case kHcBroadcast: return LaunchKernel(hc_elt_vec_kernel<AT, BT, kHcBroadcast>, grid, kBlock, 0, s, a, chunks);
      case kHcMix: return LaunchKernel(hc_elt_vec_kernel<AT, BT, kHcMix>, grid, kBlock, 0, s, a, chunks);
      case kScaleSilu: return LaunchKernel(hc_elt_vec_kernel<AT, BT, kScaleSilu>, grid, kBlock, 0, s, a, chunks);
      default: return LaunchKernel(hc_elt_vec_kernel<AT, BT, kAxpySigmoidRows>, grid, kBlock, 0, s, a, chunks);
    }
  }
  const bool per_token = a.op == kHcMix || a.op == kAxpySigmoidRows || a.op == kScaleSilu;
  const size_t n = static_cast<size_t>(a.tokens) * (per_token ? 1u : a.hc) * a.h;
  size_t grid = (n + kBlock - 1) / kBlock;
  if (grid > 148u * 32u) grid = 148u * 32u;
  return LaunchKernel(hc_elt_scalar_kernel<AT, BT>, static_cast<unsigned>(grid), kBlock, 0, s, a);
}

// ---- MoE combine -------------------------------------------------------------------------------------
// One thread per octet of a token's n columns; the k expert rows of the token are requested together (up to
// 16 loads in flight per thread), then summed in slot order with the product and the sum rounded
// separately, then the gated shared expert is added (src/model/reference.cpp:558-578).
// KR: expert rows in flight per thread; EXACT: k is a multiple of KR, so no slot of the unrolled batches is
// predicated (with k = 10 in batches of 8 the second batch issued eight slots' instructions for two rows: 22.7 M
// warp instructions per 4096 tokens, half of them predicated off).
template <typename YT, typename OT, int KR, bool EXACT>
__global__ void __launch_bounds__(kBlock, sizeof(YT) == 2 ? 4 : 2) moe_combine_kernel(const MoeCombineArgs a, const uint32_t chunks, const uint32_t ahead) {
  pdl_begin();
  __shared__ float gate;
  const uint32_t t = blockIdx.x / chunks, chunk = blockIdx.x - t * chunks;
  const unsigned j = chunk * kBlock + threadIdx.x;
  if (a.sx) {
    if (threadIdx.x == 0) gate = sigmoid_ieee(a.sg[t]);
    __syncthreads();
  }
  // One wave of resident CTAs ahead: thread s < k looks up expert row s of the token `ahead` tokens later now, and
  // hints this CTA's chunk of it to L2 once the CTA's own loads are on their way (below). A gather is two dependent
  // round trips (index, then row) per one-shot CTA, and CTAs that start together wait together; the hint turns the
  // second trip of the later CTA into an L2 hit and keeps HBM busy meanwhile.
  const uint32_t t_ahead = t + ahead;
  const bool hint = HALO_PF_MOE != 0 && ahead != 0 && threadIdx.x <= a.k && t_ahead < a.tokens;
  size_t row_ahead = 0;
  if (hint && threadIdx.x < a.k)
    row_ahead = a.pos ? a.pos[static_cast<size_t>(t_ahead) * a.k + threadIdx.x] : static_cast<size_t>(t_ahead) * a.k + threadIdx.x;
  if (j >= (a.n >> 3)) return;
  const YT* yp = static_cast<const YT*>(a.yp) + j * 8;
  const float* ww = a.mw + static_cast<size_t>(t) * a.k;
  Oct acc = oct_zero();
  OT* out = static_cast<OT*>(a.out) + static_cast<size_t>(t) * a.n + j * 8;
  if (a.accumulate) acc = oct_load(out);
  // At most eight expert rows in flight per thread (128 bytes of 16-bit rows): with sixteen the kernel held 89
  // registers and two CTAs per SM, and spent its time waiting on the index -> row dependency with too little in flight.
  constexpr int kRows = KR;
  for (uint32_t s0 = 0; s0 < a.k; s0 += kRows) {
    Raw<YT> rows[kRows];
    float wv[kRows];
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const uint32_t s = s0 + u;
      if (EXACT || s < a.k) {
        const size_t r = a.pos ? a.pos[static_cast<size_t>(t) * a.k + s] : static_cast<size_t>(t) * a.k + s;
        rows[u] = raw_load(yp + r * a.n);
        wv[u] = ww[s];
      }
    }
    if (s0 == 0 && hint) {  // the chunk's span of the row: 16-byte aligned, a multiple of 16 bytes (n % 8 == 0)
      const unsigned c0 = chunk * kBlock * 8u;
      const unsigned elems = a.n - c0 < kBlock * 8u ? a.n - c0 : kBlock * 8u;
      if (threadIdx.x < a.k) {
        prefetch_l2_span(static_cast<const YT*>(a.yp) + row_ahead * a.n + c0, elems * static_cast<unsigned>(sizeof(YT)));
      } else if (a.sx) {
        const size_t off = static_cast<size_t>(t_ahead) * a.n + c0;
        if (a.sx_is_f32) prefetch_l2_span(static_cast<const float*>(a.sx) + off, elems * 4u);
        else prefetch_l2_span(static_cast<const YT*>(a.sx) + off, elems * static_cast<unsigned>(sizeof(YT)));
      }
    }
#pragma unroll
    for (int u = 0; u < kRows; ++u)
      if (EXACT || s0 + u < a.k) acc = oct_axpy_unfused(acc, raw_unpack(rows[u]), wv[u]);
  }
  if (a.sx) {
    const size_t off = static_cast<size_t>(t) * a.n + j * 8;
    const Oct x = a.sx_is_f32 ? oct_load(static_cast<const float*>(a.sx) + off) : oct_load(static_cast<const YT*>(a.sx) + off);
    acc = oct_axpy_unfused(acc, x, gate);
  }
  oct_store(out, acc);
}

template <typename YT, typename OT>
__global__ void __launch_bounds__(kBlock) moe_combine_scalar_kernel(const MoeCombineArgs a) {
  pdl_begin();
  const size_t total = static_cast<size_t>(a.tokens) * a.n;
  for (size_t idx = static_cast<size_t>(blockIdx.x) * kBlock + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * kBlock) {
    const size_t t = idx / a.n, i = idx % a.n;
    OT* out = static_cast<OT*>(a.out) + idx;
    float acc = a.accumulate ? to_f32(*out) : 0.0f;
    for (uint32_t s = 0; s < a.k; ++s) {
      const size_t r = a.pos ? a.pos[t * a.k + s] : t * a.k + s;
      acc = __fadd_rn(acc, __fmul_rn(a.mw[t * a.k + s], to_f32(static_cast<const YT*>(a.yp)[r * a.n + i])));
    }
    if (a.sx) {
      const float x = a.sx_is_f32 ? static_cast<const float*>(a.sx)[idx] : to_f32(static_cast<const YT*>(a.sx)[idx]);
      acc = __fadd_rn(acc, __fmul_rn(sigmoid_ieee(a.sg[t]), x));
    }
    *out = from_f32<OT>(acc);
  }
}

template <typename YT, typename OT>
cudaError_t LaunchMoeCombineT(const MoeCombineArgs& a, cudaStream_t s) {
  if (a.vec) {
    const uint32_t chunks = (a.n / 8 + kBlock - 1) / kBlock;
    // tokens in one wave of resident CTAs (the kernel's launch bounds: 4 CTAs per SM for 16-bit rows, 2 for fp32)
    const uint32_t ahead = (kSms * (sizeof(YT) == 2 ? 4u : 2u) + chunks - 1) / chunks;
    const unsigned grid = a.tokens * chunks;
    if (a.k % 8 == 0) return LaunchKernel(moe_combine_kernel<YT, OT, 8, true>, grid, kBlock, 0, s, a, chunks, ahead);
    if (a.k % 5 == 0) return LaunchKernel(moe_combine_kernel<YT, OT, 5, true>, grid, kBlock, 0, s, a, chunks, ahead);
    if (a.k % 6 == 0) return LaunchKernel(moe_combine_kernel<YT, OT, 6, true>, grid, kBlock, 0, s, a, chunks, ahead);
    if (a.k % 4 == 0) return LaunchKernel(moe_combine_kernel<YT, OT, 4, true>, grid, kBlock, 0, s, a, chunks, ahead);
    return LaunchKernel(moe_combine_kernel<YT, OT, 8, false>, grid, kBlock, 0, s, a, chunks, ahead);
  }
  size_t grid = (static_cast<size_t>(a.tokens) * a.n + kBlock - 1) / kBlock;
  if (grid > 148u * 32u) grid = 148u * 32u;
  return LaunchKernel(moe_combine_scalar_kernel<YT, OT>, static_cast<unsigned>(grid), kBlock, 0, s, a);
}

}  // namespace

cudaError_t LaunchMoeCombine(const MoeCombineArgs& a, cudaStream_t s) {
  if (a.tokens == 0 || a.n == 0) return cudaSuccess;
  const int y = a.yp_dtype, o = a.out_dtype;
  if (y == kF16 && o == kF32) return LaunchMoeCombineT<f16, float>(a, s);
  if (y == kF32 && o == kF32) return LaunchMoeCombineT<float, float>(a, s);
  if (y == kBF16 && o == kBF16) return LaunchMoeCombineT<bf16, bf16>(a, s);
  if (y == kBF16 && o == kF32) return LaunchMoeCombineT<bf16, float>(a, s);
  if (y == kF16 && o == kF16) return LaunchMoeCombineT<f16, f16>(a, s);
  return cudaErrorInvalidValue;
}

// (res, out, y) type triples: the reference's (fp32 | fp16 | bf16 residual, fp32 block output and
// fp32 y) and the all-16-bit forms of a bf16 / fp16 engine.
namespace {
cudaError_t LaunchHcTyped(const HcArgs& a, cudaStream_t s);
}

cudaError_t LaunchHcCombineNorm(const HcArgs& a, cudaStream_t s) {
  if (a.tokens == 0 || a.hc == 0 || a.h == 0) return cudaSuccess;
  if (!InjectAsSecondPass(a)) return LaunchHcTyped(a, s);
  HcArgs first = a;
  first.iw = nullptr;
  first.ipart = nullptr;
  first.irows = 0;
  const cudaError_t e = LaunchHcTyped(first, s);
  if (e != cudaSuccess) return e;
  if (a.rscale) {  // rebuild from the residual: 2 bytes per value for a 16-bit residual
    switch (a.res_dtype) {
      case kF32: return LaunchHcInject<float, true>(a, static_cast<const float*>(a.res), s);
      case kF16: return LaunchHcInject<f16, true>(a, static_cast<const f16*>(a.res), s);
      default: return LaunchHcInject<bf16, true>(a, static_cast<const bf16*>(a.res), s);
    }
  }
  return LaunchHcInject<float, false>(a, static_cast<const float*>(a.y), s);
}

namespace {
cudaError_t LaunchHcTyped(const HcArgs& a, cudaStream_t s) {
  const int r = a.res_dtype, o = a.out_dtype, y = a.y_dtype;
  if (r == kF32 && o == kF32 && y == kF32) return LaunchHcM<float, float, float>(a, s);
  if (r == kF16 && o == kF32 && y == kF32) return LaunchHcM<f16, float, float>(a, s);
  if (r == kBF16 && o == kF32 && y == kF32) return LaunchHcM<bf16, float, float>(a, s);
  if (r == kF32 && o == kF16 && y == kF32) return LaunchHcM<float, f16, float>(a, s);
  if (r == kF16 && o == kF16 && y == kF32) return LaunchHcM<f16, f16, float>(a, s);
  if (r == kBF16 && o == kF16 && y == kF32) return LaunchHcM<bf16, f16, float>(a, s);
  if (r == kBF16 && o == kBF16 && y == kBF16) return LaunchHcM<bf16, bf16, bf16>(a, s);
  if (r == kF16 && o == kF16 && y == kF16) return LaunchHcM<f16, f16, f16>(a, s);
  return cudaErrorInvalidValue;
}
}  // namespace

namespace {
// One thread per element: the destinations come from a table in device memory, so nothing about their
// alignment is known at launch.
template <typename AT>
__global__ void __launch_bounds__(kBlock) copy_at_entries_kernel(const CopyAtArgs a) {
  pdl_begin();
  const uint32_t e = blockIdx.y;
  AT* dst = reinterpret_cast<AT*>(a.tab[static_cast<size_t>(e) * a.tstride + a.tslot]) +
            static_cast<size_t>(a.params[static_cast<size_t>(e) * a.pstride + a.slot]) * a.stride;
  const float* src = a.src + static_cast<size_t>(e) * a.src_stride;
  for (uint32_t i = blockIdx.x * kBlock + threadIdx.x; i < a.n; i += gridDim.x * kBlock) dst[i] = from_f32<AT>(src[i]);
}
}  // namespace

cudaError_t LaunchCopyAtEntries(const CopyAtArgs& a, cudaStream_t s) {
  if (a.entries == 0 || a.n == 0) return cudaSuccess;
  if (a.entries > 65535u) return cudaErrorInvalidValue;
  unsigned gx = (a.n + kBlock - 1) / kBlock;
  if (gx > 148u * 8u) gx = 148u * 8u;
  const dim3 grid(gx, a.entries);
  switch (a.dst_dtype) {
    case kF32: return LaunchKernel(copy_at_entries_kernel<float>, grid, kBlock, 0, s, a);
    case kF16: return LaunchKernel(copy_at_entries_kernel<f16>, grid, kBlock, 0, s, a);
    case kBF16: return LaunchKernel(copy_at_entries_kernel<bf16>, grid, kBlock, 0, s, a);
  }
  return cudaErrorInvalidValue;
}

cudaError_t LaunchHcElt(const HcEltArgs& a, cudaStream_t s) {
  if (a.tokens == 0 || a.h == 0) return cudaSuccess;
  if (a.op == kInjectReduce) {
    if (a.irows == 0) return cudaSuccess;
    return LaunchKernel(inject_reduce_kernel, (a.tokens * a.irows + kBlock - 1) / kBlock, kBlock, 0, s, a);
  }
  const int x = a.a_dtype, b = a.b_dtype;
  if (x == kF32 && b == kF32) return LaunchHcEltT<float, float>(a, s);
  if (x == kF16 && b == kF32) return LaunchHcEltT<f16, float>(a, s);
  if (x == kBF16 && b == kF32) return LaunchHcEltT<bf16, float>(a, s);
  if (x == kBF16 && b == kBF16) return LaunchHcEltT<bf16, bf16>(a, s);
  if (x == kF16 && b == kF16) return LaunchHcEltT<f16, f16>(a, s);
  if (x == kF32 && b == kF16) return LaunchHcEltT<float, f16>(a, s);
  if (x == kF32 && b == kBF16) return LaunchHcEltT<float, bf16>(a, s);
  return cudaErrorInvalidValue;
}

}  // namespace halo_b200
