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
#include "common.cuh"
#include "kernels.h"

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

// RMSNorm (shared gamma) + RoPE on rows of d <= 256 (one row = one head of one token).
// A CTA owns `tpc` whole tokens: it first fills shared (cos, -sin) / (cos, +sin) tables for
// those tokens - one sincosf per token and frequency instead of one per head and lane - then
// its thread groups walk the tokens' head rows, kRows rows per group per pass with all loads
// issued up front. A group of g lanes (g <= 32, shuffles only) owns a row; lane `lir` holds
// octets lir and (K == 2) lir + g. The sum of squares is formed exactly as the standalone
// norm kernel forms it for the same row length, so fused equals norm-then-rope bit for bit.
// Rotation: lane lir < half/8 holds the first halves of 8 pairs, lane lir + half/8 their
// partners, both in the k = 0 octet (the launcher picks K == 2 only when rot <= d / 2); the
// two exchange their normalized values with one shuffle per element and each computes
// own * cos + other * (-/+ sin): the CPU operator's a*c - b*s and a*s + b*c, term for term.
constexpr int kRows = 2;

template <typename IT, typename OT, int K>
__global__ void __launch_bounds__(kBlock, K == 2 ? 3 : 4) norm_rope_kernel(const NormRopeArgs a, const __grid_constant__ InvFreq f,
                                                             const unsigned lg, const unsigned tpc,
                                                             const float inv_d, const uint32_t heads_magic) {
  extern __shared__ float2 cs[];  // [2][tpc][half]: (cos, -sin) then (cos, +sin)
  const uint32_t half = a.rot / 2;
  const uint32_t tokens = (a.rows + a.heads - 1) / a.heads;
  const uint32_t t0 = blockIdx.x * tpc;
  for (uint32_t idx = threadIdx.x; idx < tpc * half; idx += kBlock) {
    const uint32_t t = t0 + idx / half, i = idx % half;
    if (t < tokens) {
      const uint32_t pos = token_pos(a.pos, t);
      const float angle = __fmul_rn(static_cast<float>(pos), f.f[i]);
      float sn, c;
      sincosf(angle, &sn, &c);
      cs[idx] = make_float2(c, -sn);
      cs[tpc * half + idx] = make_float2(c, sn);
      if (i == 0 && a.pos_out) a.pos_out[t] = pos;
    }
  }
  __syncthreads();

  const unsigned g = 1u << lg;
  const unsigned lane = threadIdx.x & 31u;
  const unsigned lir = threadIdx.x & (g - 1);
  const unsigned slots = kBlock >> lg, slot = threadIdx.x >> lg;
  const unsigned octs = a.d >> 3;
  const unsigned hp = a.rot / 16;  // lanes per half of the rotated span
  const bool rotates = lir < 2 * hp;
  const bool low = lir < hp;
  const unsigned src_lane = lane - lir + (rotates ? (low ? lir + hp : lir - hp) : lir);
  const float2* lane_tab = cs + (low ? 0u : tpc * half) + (low ? lir : lir - hp) * 8;
  const uint32_t row_begin = t0 * a.heads;
  uint32_t row_end = (t0 + tpc) * a.heads;
  if (row_end > a.rows) row_end = a.rows;

  Oct gm[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned j = (k << lg) + lir;
    gm[k] = oct_zero();
    if (a.w && j < octs) {
      gm[k] = oct_load_cached(a.w + j * 8);
      if (a.one_plus) {
        const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) gm[k].p[i] = __fadd2_rn(one, gm[k].p[i]);
      }
    }
  }

  for (uint32_t base = row_begin; base < row_end; base += slots * kRows) {
    Raw<IT> raw[kRows][K];
    bool ok[kRows][K];
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const uint32_t row = base + u * slots + slot;
      const IT* src = static_cast<const IT*>(a.in) + static_cast<size_t>(row) * a.in_row_stride;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        ok[u][k] = row < row_end && j < octs;
        if (ok[u][k]) raw[u][k] = raw_load(src + j * 8);
        else raw[u][k] = Raw<IT>{};
      }
    }
    if (a.gate) {
#pragma unroll
      for (int u = 0; u < kRows; ++u) {
        const uint32_t row = base + u * slots + slot;
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const unsigned j = (k << lg) + lir;
          if (ok[u][k]) {
            const Oct gt = oct_load(static_cast<const IT*>(a.in) + static_cast<size_t>(row) * a.in_row_stride + a.d + j * 8);
            oct_store(static_cast<IT*>(a.gate) + static_cast<size_t>(row) * a.d + j * 8, gt);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const uint32_t row = base + u * slots + slot;
      Oct x[K];
#pragma unroll
      for (int k = 0; k < K; ++k) x[k] = raw_unpack(raw[u][k]);
      if (a.w) {  // the norm kernel's arithmetic for a row of this length, step for step
        float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int k = 0; k < K; ++k) acc = oct_sumsq(x[k], acc);
        const float ss = group_sum(acc.x + acc.y, g, nullptr);  // g <= 32: shuffles only
        const float scale = rsqrtf(__fmaf_rn(ss, inv_d, a.eps));
#pragma unroll
        for (int k = 0; k < K; ++k) x[k] = oct_mul(oct_scale(x[k], scale), gm[k]);
      }
      float v[8];
      oct_to_array(x[0], v);
      const uint32_t rl = row < row_end ? row - row_begin : 0;
      const uint32_t tl = heads_magic ? __umulhi(rl, heads_magic) : rl / a.heads;
      const float2* tab = lane_tab + tl * half;
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const float o0 = __shfl_sync(kFullMask, v[i], src_lane);
        const float o1 = __shfl_sync(kFullMask, v[i + 1], src_lane);
        if (rotates) {
          const float4 t4 = *reinterpret_cast<const float4*>(tab + i);  // (cos, sin) of two frequencies
          v[i] = v[i] * t4.x + o0 * t4.y;
          v[i + 1] = v[i + 1] * t4.z + o1 * t4.w;
        }
      }
      OT* dst = static_cast<OT*>(a.out) + static_cast<size_t>(row) * a.d;
      OT* cdst = a.cache ? static_cast<OT*>(a.cache) + static_cast<size_t>(row) * a.d : nullptr;
      if (ok[u][0]) {
        store8(dst + lir * 8, v);
        if (cdst) store8(cdst + lir * 8, v);
      }
#pragma unroll
      for (int k = 1; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        if (ok[u][k]) {
          oct_store(dst + j * 8, x[k]);
          if (cdst) oct_store(cdst + j * 8, x[k]);
        }
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kBlock) split_qgate_kernel(const SplitArgs a) {
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
  if (a.vec) rope_kernel<T, true><<<grid, kBlock, smem, s>>>(a, f, tpc);
  else rope_kernel<T, false><<<grid, kBlock, smem, s>>>(a, f, tpc);
  return cudaGetLastError();
}

unsigned Gcd(unsigned a, unsigned b) {
  while (b) {
    const unsigned t = a % b;
    a = b;
    b = t;
  }
  return a;
}

template <typename IT, typename OT>
cudaError_t LaunchNormRopeT(const NormRopeArgs& a, const InvFreq& f, cudaStream_t s) {
  const unsigned octs = a.d / 8;
  // Two octets per lane halve the instructions per row; the rotated span must then sit in
  // the first octet of the lanes (rot <= d / 2), which holds for 64-of-256 and 16-of-64.
  const int k = (octs >= 2 && a.rot * 2 <= a.d) ? 2 : 1;
  unsigned g = 1, lg = 0;
  while (g * k < octs) g <<= 1, ++lg;
  // whole tokens per CTA such that the CTA's rows fill its passes (groups x kRows rows each)
  const unsigned rows_per_pass = kBlock / g * kRows;
  unsigned tpc = rows_per_pass / Gcd(rows_per_pass, a.heads);
  if (tpc > 32) tpc = 32;
  const unsigned tokens = (a.rows + a.heads - 1) / a.heads;
  if (tpc > tokens) tpc = tokens;
  // ... but never so many that the grid falls under about three CTAs per SM
  while (tpc > 1 && (tokens + tpc - 1) / tpc < 148u * 3u) tpc = (tpc + 1) / 2;
  const unsigned grid = (tokens + tpc - 1) / tpc;
  const size_t smem = 2 * static_cast<size_t>(tpc) * (a.rot / 2) * sizeof(float2);
  const float inv_d = 1.0f / static_cast<float>(a.d);
  // floor(n / heads) == umulhi(n, ceil(2^32 / heads)) for the n < 2^16 a CTA can see
  const uint32_t magic = (a.heads > 1 && a.heads < 2048)
                             ? static_cast<uint32_t>(((1ull << 32) + a.heads - 1) / a.heads)
                             : 0u;
  if (k == 2) norm_rope_kernel<IT, OT, 2><<<grid, kBlock, smem, s>>>(a, f, lg, tpc, inv_d, magic);
  else norm_rope_kernel<IT, OT, 1><<<grid, kBlock, smem, s>>>(a, f, lg, tpc, inv_d, magic);
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

cudaError_t LaunchSplitQgate(const SplitArgs& a, cudaStream_t s) {
  const size_t total = static_cast<size_t>(a.rows) * a.hd;
  if (total == 0) return cudaSuccess;
  size_t grid = (total + kBlock - 1) / kBlock;
  if (grid > 148u * 16u) grid = 148u * 16u;
  switch (a.dtype) {
    case kF32: split_qgate_kernel<float><<<static_cast<unsigned>(grid), kBlock, 0, s>>>(a); break;
    case kF16: split_qgate_kernel<f16><<<static_cast<unsigned>(grid), kBlock, 0, s>>>(a); break;
    case kBF16: split_qgate_kernel<bf16><<<static_cast<unsigned>(grid), kBlock, 0, s>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace halo_b200
