// Row norms for sm_100a: RMSNorm, residual-add + RMSNorm, L2 norm, gated RMSNorm,
// with the Q8 re-quantise epilogues. Replaces halo-flash's halo_rmsnorm*,
// halo_l2norm, halo_gated_norm*, halo_quantize_q8_* epilogue and the add+norm
// fusion of halo_hc_combine_norm_rows (src/kernels/core.hip:247-273, 495-510,
// 4045-4077, 4105-4210, 4502-4632); arithmetic follows src/model/cpu_ops.cpp:134-156.
//
// Layout: a row of d elements is split into octets (8 consecutive elements, one
// 16-byte load for 16-bit types, two for fp32). A group of g threads (g a power
// of two, 1..256) owns one row; thread `lir` of the group holds octets
// lir, lir + g, ... (K of them, compile-time), so every warp-wide load
// instruction covers one contiguous 512-byte (16-bit) or 1 KiB (fp32) span.
// The whole row stays in registers between the sum of squares and the scaled
// store: each activation byte crosses HBM exactly once per direction. g <= 32
// reduces with shuffles only; g > 32 adds one shared-memory stage.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "norm_lean.cuh"

namespace halo_b200 {
namespace {

template <typename T>
__device__ __forceinline__ T* at(void* p, size_t off) { return static_cast<T*>(p) + off; }
template <typename T>
__device__ __forceinline__ const T* at(const void* p, size_t off) { return static_cast<const T*>(p) + off; }

// Epilogues on one normalized octet `v` (columns [c0, c0 + 8) of row `row`); all 32
// lanes of the warp call (quad shuffles), `ok` marks lanes that hold real data.
__device__ __forceinline__ void q8_epilogues(const NormArgs& a, const float (&v)[8], uint32_t row, uint32_t c0, bool ok) {
  const float amax = quad_amax(v);
  if (a.q8_0) {
    uint16_t dbits;
    const uint2 codes = q8_0_codes(v, amax, &dbits);
    if (ok) {
      uint8_t* blk = a.q8_0 + static_cast<size_t>(row) * (a.d / 32) * 34 + static_cast<size_t>(c0 / 32) * 34;
      if ((c0 & 31u) == 0) *reinterpret_cast<uint16_t*>(blk) = dbits;
      store_codes_u16(blk + 2 + (c0 & 31u), codes);
    }
  }
  if (a.xq) {
    const float scale = div127(amax);
    const uint2 codes = i8_codes(v, scale);
    if (ok) {
      if (a.kb_tokens) {
        const uint32_t t = row / a.kb_period, c = (row % a.kb_period) * a.d + c0;
        *reinterpret_cast<uint2*>(a.xq + (static_cast<size_t>(c / 64) * a.kb_tokens + t) * 64 + c % 64) = codes;
        if ((c0 & 31u) == 0) a.xd[static_cast<size_t>(c / 32) * a.kb_tokens + t] = scale;
      } else {
        *reinterpret_cast<uint2*>(a.xq + static_cast<size_t>(row) * a.d + c0) = codes;
        if ((c0 & 31u) == 0) a.xd[static_cast<size_t>(row) * (a.d / 32) + c0 / 32] = scale;
      }
    }
  }
}

// R rows per thread group (R > 1 only for short rows, K == 1): row u of group `slot` is
// row0 + u * (groups per CTA), so neighbouring groups still read neighbouring rows.
// FULL: every row of the grid exists and every thread's octets lie inside the row, so no
// load or store is predicated (the launcher checks d == 8 K g and rows % (rows per CTA) == 0).
// These kernels are bound by instruction issue as much as by HBM: the arithmetic is packed
// fp32x2, offsets are shifts, and rare features hide behind warp-uniform branches.
template <typename XT, typename YT, int K, int R, bool ADD, bool FULL>
__device__ __forceinline__ void norm_rows_body(const NormArgs& a, const unsigned lg, const float inv_d,
                                               float* scratch) {
  const unsigned g = 1u << lg;
  const unsigned lir = threadIdx.x & (g - 1);
  const unsigned rpc = kBlock >> lg;
  const uint32_t row0 = blockIdx.x * (rpc * R) + (threadIdx.x >> lg);
  const unsigned octs = a.d >> 3;

  Oct v[R][K];
  size_t dense[R], xoff[R];
  bool row_ok[R];
  // Every load of the thread is issued before any is consumed.
#pragma unroll
  for (int u = 0; u < R; ++u) {
    const uint32_t row = row0 + u * rpc;
    row_ok[u] = FULL || row < a.rows;
    dense[u] = static_cast<size_t>(row) * a.d;
    xoff[u] = dense[u];
    if (a.rows_per_entry)
      xoff[u] = static_cast<size_t>(row / a.rows_per_entry) * a.entry_stride +
                static_cast<size_t>(row % a.rows_per_entry) * a.d;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      if (FULL || (row_ok[u] && j < octs)) v[u][k] = oct_load(at<XT>(a.x, xoff[u] + j * 8));
      else v[u][k] = oct_zero();
    }
  }
  if constexpr (ADD) {
    Oct dl[R][K];
#pragma unroll
    for (int u = 0; u < R; ++u)
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        if (FULL || (row_ok[u] && j < octs)) dl[u][k] = oct_load(at<XT>(a.delta, dense[u] + j * 8));
        else dl[u][k] = oct_zero();
      }
#pragma unroll
    for (int u = 0; u < R; ++u)
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        v[u][k] = oct_add(v[u][k], dl[u][k]);
        // stored in the residual's type; the norm then reads the residual as stored
        if (FULL || (row_ok[u] && j < octs)) oct_store_round(at<XT>(a.res, xoff[u] + j * 8), v[u][k]);
      }
  }

  // Gammas do not depend on the reduction: for long rows (one row per group, at most two
  // octets per thread) they are fetched before it, so the L2 round trip overlaps the
  // shuffle / barrier instead of following it. Short rows re-read a gamma that sits in L1.
  constexpr bool kEarlyGamma = K <= 2 && R == 1;
  Oct gm[kEarlyGamma ? K : 1];
  if constexpr (kEarlyGamma) {
    if (a.w) {
      const float* wrow = a.w + (a.w_period > 1 ? static_cast<size_t>(row0 % a.w_period) * a.w_stride : 0);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        if (FULL || (row_ok[0] && j < octs)) gm[k] = oct_load_cached(wrow + j * 8);
        else gm[k] = oct_zero();
        if (a.one_plus) {
          const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
          for (int i = 0; i < 4; ++i) gm[k].p[i] = __fadd2_rn(one, gm[k].p[i]);
        }
      }
    }
  }

  const bool epi = a.q8_0 != nullptr || a.xq != nullptr;
#pragma unroll
  for (int u = 0; u < R; ++u) {
    const uint32_t row = row0 + u * rpc;
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < K; ++k) acc = oct_sumsq(v[u][k], acc);
    const float ss = group_sum(acc.x + acc.y, g, scratch);
    const float scale = a.l2 ? rsqrtf(ss + a.eps) : rsqrtf(__fmaf_rn(ss, inv_d, a.eps));
    if (a.rscale && row_ok[u] && lir == 0) a.rscale[row] = scale;
    const float* wrow = nullptr;
    if (!kEarlyGamma && a.w)
      wrow = a.w + (a.w_period > 1 ? static_cast<size_t>(row % a.w_period) * a.w_stride : 0);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      const bool ok = FULL || (row_ok[u] && j < octs);
      v[u][k] = oct_scale(v[u][k], scale);
      if constexpr (kEarlyGamma) {
        if (a.w) v[u][k] = oct_mul(v[u][k], gm[k]);
      } else if (wrow) {
        Oct gl = ok ? oct_load_cached(wrow + j * 8) : oct_zero();
        if (a.one_plus) {
          const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
          for (int i = 0; i < 4; ++i) gl.p[i] = __fadd2_rn(one, gl.p[i]);
        }
        v[u][k] = oct_mul(v[u][k], gl);
      }
      if (ok) {
        if (a.y) oct_store(at<YT>(a.y, xoff[u] + j * 8), v[u][k]);
        if (a.y16) {
          size_t o16 = dense[u] + j * 8;
          if (a.y16_tokens) {
            const uint32_t t = row / a.kb_period, c = (row % a.kb_period) * a.d + j * 8;
            o16 = (static_cast<size_t>(c / 64) * a.y16_tokens + t) * 64 + c % 64;
          }
          oct_store(at<f16>(a.y16, o16), v[u][k]);
        }
      }
      if (epi) {
        float arr[8];
        oct_to_array(v[u][k], arr);
        q8_epilogues(a, arr, row, j * 8, ok);
      }
    }
  }
}

// Resident CTAs per SM the register allocation is held to: the kernels wait on HBM most of
// the time, so for short per-thread rows more warps in flight beat a few saved instructions.
// `live` = octets a thread holds in fp32 across the reduction (8 registers each).
constexpr int MinCtas(int live) { return live <= 1 ? 6 : (live <= 2 ? 5 : (live <= 4 ? 3 : 1)); }

// The general kernel: every feature, every load and store predicated.
template <typename XT, typename YT, int K, int R, bool ADD>
__global__ void __launch_bounds__(kBlock, MinCtas(K * R)) norm_rows_kernel(const NormArgs a, const unsigned lg,
                                                                          const float inv_d) {
  pdl_begin();
  __shared__ float scratch[kBlock / 32];
  norm_rows_body<XT, YT, K, R, ADD, false>(a, lg, inv_d, scratch);
}

// Any d, any alignment: one CTA per row, scalar accesses, the row is re-read
// after the reduction. Correctness path for shapes the vector kernel refuses.
template <typename XT, typename YT, bool ADD>
__global__ void __launch_bounds__(kBlock) norm_rows_scalar_kernel(const NormArgs a) {
  pdl_begin();
  __shared__ float scratch[kBlock / 32];
  __shared__ float total;
  const uint32_t row = blockIdx.x;
  const size_t dense = static_cast<size_t>(row) * a.d;
  const size_t xoff = a.rows_per_entry
                          ? static_cast<size_t>(row / a.rows_per_entry) * a.entry_stride +
                                static_cast<size_t>(row % a.rows_per_entry) * a.d
                          : dense;
  const XT* x = at<XT>(a.x, xoff);
  float ss = 0.0f;
  for (uint32_t i = threadIdx.x; i < a.d; i += kBlock) {
    float xv = to_f32(x[i]);
    if constexpr (ADD) {
      xv = xv + to_f32(at<XT>(a.delta, dense)[i]);
      at<XT>(a.res, xoff)[i] = from_f32<XT>(xv);
      xv = round_through<XT>(xv);
    }
    ss += xv * xv;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    for (int i = 0; i < kBlock / 32; ++i) t += scratch[i];
    total = t;
  }
  __syncthreads();
  ss = total;
  const float scale = a.l2 ? 1.0f / sqrtf(ss + a.eps) : 1.0f / sqrtf(ss / static_cast<float>(a.d) + a.eps);
  if (a.rscale && threadIdx.x == 0) a.rscale[row] = scale;
  const float* wrow = a.w ? a.w + static_cast<size_t>(row % a.w_period) * a.w_stride : nullptr;
  const XT* src = ADD ? at<XT>(static_cast<const void*>(a.res), xoff) : x;
  const bool epi = a.q8_0 != nullptr || a.xq != nullptr;  // api.cu guarantees d % 32 == 0 then
  const uint32_t lane = threadIdx.x & 31u;
  for (uint32_t base = threadIdx.x - lane; base < a.d; base += kBlock) {
    const uint32_t i = base + lane;
    const bool ok = i < a.d;
    float v = ok ? to_f32(src[i]) : 0.0f;
    if (wrow) {
      const float gm = ok ? wrow[i] : 0.0f;
      v = v * scale * (a.one_plus ? 1.0f + gm : gm);
    } else {
      v = v * scale;
    }
    if (ok) {
      if (a.y) at<YT>(a.y, xoff)[i] = from_f32<YT>(v);
      if (a.y16) {
        size_t o16 = dense + i;
        if (a.y16_tokens) {
          const uint32_t t = row / a.kb_period, c = (row % a.kb_period) * a.d + i;
          o16 = (static_cast<size_t>(c / 64) * a.y16_tokens + t) * 64 + c % 64;
        }
        at<f16>(a.y16, o16)[0] = __float2half_rn(v);
      }
    }
    if (epi) {
      const float amax = warp_max(fabsf(v));
      if (a.q8_0) {
        const f16 dh = __float2half_rn(amax / 127.0f);
        const float d = __half2float(dh);
        float q = 0.0f;
        if (d > 0.0f) q = fminf(fmaxf(rintf(v / d), -127.0f), 127.0f);
        uint8_t* blk = a.q8_0 + static_cast<size_t>(row) * (a.d / 32) * 34 + static_cast<size_t>(i / 32) * 34;
        if (ok) {
          if (lane == 0) *reinterpret_cast<uint16_t*>(blk) = __half_as_ushort(dh);
          blk[2 + lane] = static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(q)));
        }
      }
      if (a.xq) {
        const float qs = amax / 127.0f;
        const int8_t code = static_cast<int8_t>(qs > 0.0f ? static_cast<int>(rintf(v / qs)) : 0);
        if (ok) {
          if (a.kb_tokens) {
            const uint32_t t = row / a.kb_period, c = (row % a.kb_period) * a.d + i;
            a.xq[(static_cast<size_t>(c / 64) * a.kb_tokens + t) * 64 + c % 64] = code;
            if (lane == 0) a.xd[static_cast<size_t>(c / 32) * a.kb_tokens + t] = qs;
          } else {
            a.xq[static_cast<size_t>(row) * a.d + i] = code;
            if (lane == 0) a.xd[static_cast<size_t>(row) * (a.d / 32) + i / 32] = qs;
          }
        }
      }
    }
  }
}

// ---- gated RMSNorm: y = ((o * scale) * w) * gate(z) ----------------------------------------
template <typename OT, typename ZT, typename YT, int K, int R, bool FULL>
__device__ __forceinline__ void gated_norm_body(const GatedArgs& a, const unsigned lg, const float inv_d,
                                                float* scratch) {
  const unsigned g = 1u << lg;
  const unsigned lir = threadIdx.x & (g - 1);
  const unsigned rpc = kBlock >> lg;
  const uint32_t row0 = blockIdx.x * (rpc * R) + (threadIdx.x >> lg);
  const unsigned octs = a.d >> 3;
  // All loads first, kept as raw bits (4 registers per 16-bit octet) until each row is processed.
  Raw<OT> ro[R][K];
  Raw<ZT> rz[R][K];
#pragma unroll
  for (int u = 0; u < R; ++u) {
    const uint32_t row = row0 + u * rpc;
    const size_t off = static_cast<size_t>(row) * a.d;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      if (FULL || (row < a.rows && j < octs)) {
        ro[u][k] = raw_load(at<OT>(a.o, off + j * 8));
        rz[u][k] = raw_load(at<ZT>(a.z, off + j * 8));
      } else {
        ro[u][k] = Raw<OT>{};
        rz[u][k] = Raw<ZT>{};
      }
    }
  }
  Oct gm[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned j = (k << lg) + lir;
    gm[k] = (FULL || j < octs) ? oct_load_cached(a.w + j * 8) : oct_zero();
  }
#pragma unroll
  for (int u = 0; u < R; ++u) {
    const uint32_t row = row0 + u * rpc;
    Oct v[K], zz[K];
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      v[k] = raw_unpack(ro[u][k]);
      acc = oct_sumsq(v[k], acc);
    }
    // The gate does not depend on the reduction: its exp2 / reciprocal work is independent of the
    // shuffles below and overlaps them. The product keeps the CPU operator's order,
    // ((o * scale) * w) * gate.
#pragma unroll
    for (int k = 0; k < K; ++k) zz[k] = raw_unpack(rz[u][k]);
    if (a.mode == 0) {
#pragma unroll
      for (int k = 0; k < K; ++k)
#pragma unroll
        for (int i = 0; i < 4; ++i) zz[k].p[i] = silu2_f(zz[k].p[i]);
    } else {
#pragma unroll
      for (int k = 0; k < K; ++k)
#pragma unroll
        for (int i = 0; i < 4; ++i) zz[k].p[i] = sigmoid2_f(zz[k].p[i]);
    }
    const float ss = group_sum(acc.x + acc.y, g, scratch);
    const float scale = rsqrtf(__fmaf_rn(ss, inv_d, a.eps));
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      if (FULL || (row < a.rows && j < octs)) {
        const Oct r = oct_mul(oct_mul(oct_scale(v[k], scale), gm[k]), zz[k]);
        oct_store(at<YT>(a.y, static_cast<size_t>(row) * a.d + j * 8), r);
      }
    }
  }
}

template <typename OT, typename ZT, typename YT, int K, int R, bool FULL>
__global__ void __launch_bounds__(kBlock, K >= 4 ? 2 : (K * R <= 2 ? 4 : 3)) gated_norm_kernel(const GatedArgs a, const unsigned lg,
                                                                               const float inv_d) {
  pdl_begin();
  __shared__ float scratch[kBlock / 32];
  gated_norm_body<OT, ZT, YT, K, R, FULL>(a, lg, inv_d, scratch);
}

// The lean gated norm for the common case (every row exists, d == 8 g, one octet per thread):
// operands as plain arguments, nothing predicated, no code for other shapes. On the 32 x 128
// DeltaNet heads of 4096 tokens it runs in 16.5 us where the general kernel needs 19.8.
struct GatedLeanArgs {
  const void* o;
  const void* z;
  const float* w;
  void* y;
  uint32_t d, lg, mode;
  float eps, inv_d;
};

template <typename OT, typename ZT, typename YT>
__global__ void __launch_bounds__(kBlock) gated_norm_lean_kernel(const GatedLeanArgs a) {
  pdl_trigger_early();
  // (only the first wave: the rows of every later CTA were hinted by the look-ahead of an earlier one, below)
  if (HALO_PF_GATED != 0 && threadIdx.x == 0 && (HALO_PF_AHEAD_GATED == 0 || blockIdx.x < HALO_PF_AHEAD_GATED * kSms * 8u)) {
    const size_t span = static_cast<size_t>(kBlock >> a.lg) * a.d;
    prefetch_l2_span(static_cast<const OT*>(a.o) + blockIdx.x * span, static_cast<unsigned>(span * sizeof(OT)));
    prefetch_l2_span(static_cast<const ZT*>(a.z) + blockIdx.x * span, static_cast<unsigned>(span * sizeof(ZT)));
  }
  pdl_wait_and_trigger();
  const unsigned lg = a.lg, g = 1u << lg;
  const unsigned lir = threadIdx.x & (g - 1);
  const uint32_t row = blockIdx.x * (kBlock >> lg) + (threadIdx.x >> lg);
  const size_t off = static_cast<size_t>(row) * a.d + (lir << 3);
  const Raw<OT> ro = raw_load(static_cast<const OT*>(a.o) + off);
  const Raw<ZT> rz = raw_load(static_cast<const ZT*>(a.z) + off);
  constexpr unsigned kAhead = HALO_PF_AHEAD_GATED * kSms * 8u;
  if constexpr (kAhead != 0) {
    if (threadIdx.x == 0 && blockIdx.x + kAhead < gridDim.x) {
      const size_t span = static_cast<size_t>(kBlock >> lg) * a.d;
      prefetch_l2_span(static_cast<const OT*>(a.o) + (blockIdx.x + kAhead) * span, static_cast<unsigned>(span * sizeof(OT)));
      prefetch_l2_span(static_cast<const ZT*>(a.z) + (blockIdx.x + kAhead) * span, static_cast<unsigned>(span * sizeof(ZT)));
    }
  }
  const Oct gm = oct_load_cached(a.w + (lir << 3));
  const Oct v = raw_unpack(ro);
  Oct zz = raw_unpack(rz);
  const float2 acc = oct_sumsq(v, make_float2(0.0f, 0.0f));
  if (a.mode == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) zz.p[i] = silu2_f(zz.p[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) zz.p[i] = sigmoid2_f(zz.p[i]);
  }
  const float ss = group_sum_narrow(acc.x + acc.y, g);
  const float scale = rsqrtf(__fmaf_rn(ss, a.inv_d, a.eps));
  oct_store(static_cast<YT*>(a.y) + off, oct_mul(oct_mul(oct_scale(v, scale), gm), zz));
}

template <typename OT, typename ZT, typename YT>
__global__ void __launch_bounds__(kBlock) gated_norm_scalar_kernel(const GatedArgs a) {
  pdl_begin();
  __shared__ float scratch[kBlock / 32];
  __shared__ float total;
  const size_t off = static_cast<size_t>(blockIdx.x) * a.d;
  const OT* o = at<OT>(a.o, off);
  const ZT* z = at<ZT>(a.z, off);
  float ss = 0.0f;
  for (uint32_t i = threadIdx.x; i < a.d; i += kBlock) {
    const float xv = to_f32(o[i]);
    ss += xv * xv;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    for (int i = 0; i < kBlock / 32; ++i) t += scratch[i];
    total = t;
  }
  __syncthreads();
  const float scale = 1.0f / sqrtf(total / static_cast<float>(a.d) + a.eps);
  for (uint32_t i = threadIdx.x; i < a.d; i += kBlock) {
    const float zf = to_f32(z[i]);
    const float gate = a.mode == 0 ? silu_f(zf) : sigmoid_f(zf);
    at<YT>(a.y, off)[i] = from_f32<YT>(to_f32(o[i]) * scale * a.w[i] * gate);
  }
}

// few_rows: the launch cannot fill the GPU (a decode step). It then lasts as long as one warp's chain of
// dependent instructions (about 10 cycles each), so rows are spread over as many threads as they have
// octets, one octet per thread: 1.55 -> 1.2 us for the add + norm of 8 rows of 2048. Not applied where
// the caller pinned a layout (want_k1: the layout shared with the fused norm + RoPE kernel).
Shape PickShape(unsigned octs, unsigned rows, int want_g, unsigned min_g, int want_k1, bool few_rows_ok = false) {
  unsigned g;
  const bool few_rows = few_rows_ok && static_cast<uint64_t>(rows) * octs <= 148u * 256u;
  if (want_g > 0) {
    g = static_cast<unsigned>(want_g);
  } else if (few_rows) {
    g = 1;
    while (g < octs && g < 256u) g <<= 1;
  } else if (octs <= 32) {
    // Short rows (one head), shuffles only. Two octets per thread measured faster than one
    // (13.8 vs 14.8 us for the 16 x 128 q/k L2 norm at 4096 tokens) and faster than several
    // rows per group; want_k1 keeps one octet per thread, the layout of the fused norm + RoPE
    // kernel, for callers that need the two to agree bit for bit.
    g = 1;
    while ((want_k1 ? g : 2 * g) < octs) g <<= 1;
    // rows of 256 (a GQA head): eight lanes with four octets each, the layout of the fused norm + RoPE kernel
    if (!want_k1 && octs == 32) g = 8;
  } else {
    // Two octets per thread keep registers low (many resident CTAs, many loads in flight)
    // and the gammas prefetchable; measured best at d = 2048 (g = 128) on B200.
    g = 64;
    while (g < 256 && octs > 2 * g) g <<= 1;
  }
  if (g < min_g) g = min_g;
  unsigned k = (octs + g - 1) / g, kp = 1;
  while (kp < k) kp <<= 1;
  Shape sh;
  sh.lg = 0;
  while ((1u << sh.lg) < g) ++sh.lg;
  sh.k = static_cast<int>(kp);
  sh.r = 1;
  sh.rows_per_cta = kBlock / g;
  sh.full = octs == kp * g && rows % sh.rows_per_cta == 0;
  return sh;
}

// Rows of 3 g or 5 g octets with g = 64, 128 or 256 threads (H = 1536, 2560, 3072, 5120, ...): three or five octets
// per thread in the lean kernel, where the general kernel pads the row to a power of two (at H = 2560 it runs 256
// threads x 2 octets with 37 % of the lanes idle: 17.2 us = 0.75 of measured for the add + norm of 4096 rows).
bool PickOddShape(unsigned octs, unsigned rows, size_t elem_size, Shape* sh) {
  for (int k : {3, 5}) {
    if (octs % k != 0) continue;
    if (k == 5 && elem_size == 4) continue;  // fp32 rows at five octets per thread measured slower than the general kernel (19.8 against 17.1 us)
    const unsigned g = octs / k;
    if (g < 64 || g > 256 || (g & (g - 1)) != 0 || rows % (kBlock / g) != 0) continue;
    sh->lg = 0;
    while ((1u << sh->lg) < g) ++sh->lg;
    sh->k = k, sh->r = 1, sh->rows_per_cta = kBlock / g, sh->full = true;
    return true;
  }
  return false;
}

template <typename XT, typename YT, bool ADD>
cudaError_t LaunchNormT(const NormArgs& a, cudaStream_t s) {
  if (!a.vec) {
    LaunchKernel(norm_rows_scalar_kernel<XT, YT, ADD>, a.rows, kBlock, 0, s, a);
    return cudaGetLastError();
  }
  // rows of one head keep the layout they share with the fused norm + RoPE kernel unless they are an L2 norm
  const Shape sh = PickShape(a.d / 8, a.rows, a.threads_per_row, (a.q8_0 || a.xq) ? 4u : 1u, a.short_rows_k1,
                             a.d / 8 > 32 || a.l2);
  const unsigned grid = (a.rows + sh.rows_per_cta - 1) / sh.rows_per_cta;
  // (in, out) pairs the lean kernels are built for; the rest go through the general kernel
  constexpr bool kLeanTypes = (std::is_same_v<XT, float> && !std::is_same_v<YT, f16>) ||
                              (std::is_same_v<XT, bf16> && !std::is_same_v<YT, f16>) ||
                              (std::is_same_v<XT, f16> && std::is_same_v<YT, f16>);
  const bool lean = sh.full && (sh.k <= 2 || (sh.k == 4 && sh.lg == 3)) && a.rows_per_entry == 0 && a.w_period <= 1 && a.y16 == nullptr &&
                    a.rscale == nullptr && a.kb_tokens == 0 && !a.force_general;
  if constexpr (kLeanTypes) {
    if (lean) {
      if (sh.k == 4) return LaunchLean<XT, YT, 4, ADD>(a, sh, grid, s);
      return sh.k == 1 ? LaunchLean<XT, YT, 1, ADD>(a, sh, grid, s) : LaunchLean<XT, YT, 2, ADD>(a, sh, grid, s);
    }
    Shape odd;
    // (launches that cannot fill the GPU keep the general kernel's wide, short-chain layout: see PickShape)
    if (!sh.full && static_cast<uint64_t>(a.rows) * (a.d / 8) > 148u * 256u && a.threads_per_row == 0 && a.rows_per_entry == 0 && a.w_period <= 1 && a.y16 == nullptr && a.rscale == nullptr &&
        a.kb_tokens == 0 && !a.force_general && PickOddShape(a.d / 8, a.rows, sizeof(XT), &odd)) {
      // (those instantiations live in norm_odd.cu, which compiles beside this file)
      return LaunchNormLeanOdd(a, odd.lg, odd.k, odd.rows_per_cta, a.rows / odd.rows_per_cta, s);
    }
  }
  const float inv_d = 1.0f / static_cast<float>(a.d);
  switch (sh.k) {
    case 1: LaunchKernel(norm_rows_kernel<XT, YT, 1, 1, ADD>, grid, kBlock, 0, s, a, sh.lg, inv_d); break;
    case 2: LaunchKernel(norm_rows_kernel<XT, YT, 2, 1, ADD>, grid, kBlock, 0, s, a, sh.lg, inv_d); break;
    case 4: LaunchKernel(norm_rows_kernel<XT, YT, 4, 1, ADD>, grid, kBlock, 0, s, a, sh.lg, inv_d); break;
    case 8: LaunchKernel(norm_rows_kernel<XT, YT, 8, 1, ADD>, grid, kBlock, 0, s, a, sh.lg, inv_d); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <typename XT, typename YT>
cudaError_t LaunchNormA(const NormArgs& a, cudaStream_t s) {
  return a.delta ? LaunchNormT<XT, YT, true>(a, s) : LaunchNormT<XT, YT, false>(a, s);
}

template <typename XT>
cudaError_t LaunchNormY(const NormArgs& a, cudaStream_t s) {
  switch (a.y_dtype) {
    case kF32: return LaunchNormA<XT, float>(a, s);
    case kF16: return LaunchNormA<XT, f16>(a, s);
    case kBF16: return LaunchNormA<XT, bf16>(a, s);
  }
  return cudaErrorInvalidValue;
}

template <typename OT, typename ZT, typename YT>
cudaError_t LaunchGatedT(const GatedArgs& a, cudaStream_t s) {
  if (!a.vec) {
    LaunchKernel(gated_norm_scalar_kernel<OT, ZT, YT>, a.rows, kBlock, 0, s, a);
    return cudaGetLastError();
  }
  const float inv_d = 1.0f / static_cast<float>(a.d);
  const unsigned octs = a.d / 8;
  if (octs <= 32 && (octs & (octs - 1)) == 0 && a.rows % (kBlock / octs) == 0 && !a.force_general) {
    GatedLeanArgs l;
    l.o = a.o;
    l.z = a.z;
    l.w = a.w;
    l.y = a.y;
    l.d = a.d;
    l.lg = 0;
    while ((1u << l.lg) < octs) ++l.lg;
    l.mode = a.mode;
    l.eps = a.eps;
    l.inv_d = inv_d;
    LaunchKernel(gated_norm_lean_kernel<OT, ZT, YT>, a.rows / (kBlock / octs), kBlock, 0, s, l);
    return cudaGetLastError();
  }
  // One octet per thread on short rows: the layout of the lean kernel, so the two agree bit for bit.
  const Shape sh = PickShape(octs, a.rows, a.threads_per_row, 1u, 1);
  const unsigned grid = (a.rows + sh.rows_per_cta - 1) / sh.rows_per_cta;
  switch (sh.k) {
    case 1:
      if (sh.full) LaunchKernel(gated_norm_kernel<OT, ZT, YT, 1, 1, true>, grid, kBlock, 0, s, a, sh.lg, inv_d);
      else LaunchKernel(gated_norm_kernel<OT, ZT, YT, 1, 1, false>, grid, kBlock, 0, s, a, sh.lg, inv_d);
      break;
    case 2:
      if (sh.lg <= 5 && a.rows_per_group == 2) {  // short rows, two rows per thread group in flight
        const unsigned rpc2 = sh.rows_per_cta * 2;
        const unsigned grid2 = (a.rows + rpc2 - 1) / rpc2;
        if (sh.full && a.rows % rpc2 == 0) LaunchKernel(gated_norm_kernel<OT, ZT, YT, 2, 2, true>, grid2, kBlock, 0, s, a, sh.lg, inv_d);
        else LaunchKernel(gated_norm_kernel<OT, ZT, YT, 2, 2, false>, grid2, kBlock, 0, s, a, sh.lg, inv_d);
        break;
      }
      if (sh.full) LaunchKernel(gated_norm_kernel<OT, ZT, YT, 2, 1, true>, grid, kBlock, 0, s, a, sh.lg, inv_d);
      else LaunchKernel(gated_norm_kernel<OT, ZT, YT, 2, 1, false>, grid, kBlock, 0, s, a, sh.lg, inv_d);
      break;
    case 4: LaunchKernel(gated_norm_kernel<OT, ZT, YT, 4, 1, false>, grid, kBlock, 0, s, a, sh.lg, inv_d); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

// Largest d the vector path accepts: 256 threads x 8 octets x 8 elements.
cudaError_t LaunchNorm(const NormArgs& a, cudaStream_t s) {
  if (a.rows == 0) return cudaSuccess;
  switch (a.x_dtype) {
    case kF32: return LaunchNormY<float>(a, s);
    case kF16: return LaunchNormY<f16>(a, s);
    case kBF16: return LaunchNormY<bf16>(a, s);
  }
  return cudaErrorInvalidValue;
}

cudaError_t LaunchGatedNorm(const GatedArgs& a, cudaStream_t s) {
  if (a.rows == 0) return cudaSuccess;
  const int key = a.o_dtype * 9 + a.z_dtype * 3 + a.y_dtype;
  switch (key) {
    case kF32 * 9 + kF32 * 3 + kF32: return LaunchGatedT<float, float, float>(a, s);
    case kF32 * 9 + kF32 * 3 + kF16: return LaunchGatedT<float, float, f16>(a, s);
    case kF32 * 9 + kF32 * 3 + kBF16: return LaunchGatedT<float, float, bf16>(a, s);
    case kF32 * 9 + kF16 * 3 + kF16: return LaunchGatedT<float, f16, f16>(a, s);
    case kF16 * 9 + kF16 * 3 + kF16: return LaunchGatedT<f16, f16, f16>(a, s);
    case kBF16 * 9 + kBF16 * 3 + kBF16: return LaunchGatedT<bf16, bf16, bf16>(a, s);
    case kBF16 * 9 + kBF16 * 3 + kF32: return LaunchGatedT<bf16, bf16, float>(a, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace halo_b200
