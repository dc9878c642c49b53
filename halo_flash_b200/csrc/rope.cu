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

// RMSNorm (shared gamma) + RoPE on rows of d <= 256 (one row = one head of one token), for one
// tensor or for Q and K together. Rows are numbered token by token (token t: tensor 1's heads,
// then tensor 2's); a CTA owns one pass of consecutive rows - kBlock / g thread groups x kRows
// rows, 32 rows at d = 256 - so the grid has thousands of short-lived CTAs and no tail. It first
// fills shared (cos, -sin) / (cos, +sin) tables for the two or three tokens those rows belong
// to - one sincosf per token and frequency instead of one per head and lane - then every group
// loads its kRows rows up front. A group of g lanes (g <= 32, shuffles only) owns a row; lane
// `lir` holds octets lir and (K == 2) lir + g. The sum of squares is formed exactly as the
// standalone norm kernel forms it for the same row length, so fused equals norm-then-rope bit
// for bit. Rotation: lane lir < half/8 holds the first halves of 8 pairs, lane lir + half/8
// their partners, both in the k = 0 octet (the launcher picks K == 2 only when rot <= d / 2);
// the two exchange their normalized values with one shuffle per element and each computes
// own * cos + other * (-/+ sin): the CPU operator's a*c - b*s and a*s + b*c, term for term.
constexpr int kRows = 2;

__device__ __forceinline__ uint32_t div_magic(uint32_t n, uint32_t d, uint32_t magic) {
  return magic ? __umulhi(n, magic) : n / d;
}

template <typename IT, typename OT, int K>
__global__ void __launch_bounds__(kBlock, K == 2 ? 3 : 4) norm_rope_kernel(const NormRopeArgs a, const __grid_constant__ InvFreq f,
                                                             const unsigned lg, const uint32_t rows_total,
                                                             const float inv_d, const uint32_t heads_magic) {
  extern __shared__ float2 cs[];  // [2][ntok][half]: (cos, -sin) then (cos, +sin)
  const uint32_t half = a.rot / 2;
  const uint32_t hall = a.heads + a.heads2;
  const unsigned slots = kBlock >> lg;
  const uint32_t vr0 = blockIdx.x * (slots * kRows);
  uint32_t vr1 = vr0 + slots * kRows;
  if (vr1 > rows_total) vr1 = rows_total;
  const uint32_t tok0 = div_magic(vr0, hall, heads_magic);
  const uint32_t ntok = div_magic(vr1 - 1, hall, heads_magic) - tok0 + 1;
  for (uint32_t idx = threadIdx.x; idx < ntok * half; idx += kBlock) {
    const uint32_t t = tok0 + idx / half, i = idx % half;
    const uint32_t pos = token_pos(a.pos, t);
    const float angle = __fmul_rn(static_cast<float>(pos), f.f[i]);
    float sn, c;
    sincosf(angle, &sn, &c);
    cs[idx] = make_float2(c, -sn);
    cs[ntok * half + idx] = make_float2(c, sn);
    // the first row of a token writes its position (exactly one CTA holds that row)
    if (i == 0 && a.pos_out && t * hall >= vr0) a.pos_out[t] = pos;
  }
  __syncthreads();

  const unsigned g = 1u << lg;
  const unsigned lane = threadIdx.x & 31u;
  const unsigned lir = threadIdx.x & (g - 1);
  const unsigned slot = threadIdx.x >> lg;
  const unsigned octs = a.d >> 3;
  const unsigned hp = a.rot / 16;  // lanes per half of the rotated span
  const bool rotates = lir < 2 * hp;
  const bool low = lir < hp;
  const unsigned src_lane = lane - lir + (rotates ? (low ? lir + hp : lir - hp) : lir);
  const float2* lane_tab = cs + (low ? 0u : ntok * half) + (low ? lir : lir - hp) * 8;

  Raw<IT> raw[kRows][K];
  bool ok[kRows][K];
  size_t out_off[kRows];
  uint32_t tl[kRows];
  bool second[kRows];
#pragma unroll
  for (int u = 0; u < kRows; ++u) {
    const uint32_t vr = vr0 + u * slots + slot;
    const bool in_cta = vr < vr1;
    const uint32_t token = in_cta ? div_magic(vr, hall, heads_magic) : tok0;
    tl[u] = token - tok0;
    const uint32_t h = in_cta ? vr - token * hall : 0;
    second[u] = h >= a.heads;
    const size_t row = second[u] ? static_cast<size_t>(token) * a.heads2 + (h - a.heads)
                                 : static_cast<size_t>(token) * a.heads + h;
    const bool row_ok = in_cta && (second[u] || row < a.rows);
    const IT* src = second[u] ? static_cast<const IT*>(a.in2) + row * a.in_row_stride2
                              : static_cast<const IT*>(a.in) + row * a.in_row_stride;
    out_off[u] = row * a.d;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const unsigned j = (k << lg) + lir;
      ok[u][k] = row_ok && j < octs;
      raw[u][k] = Raw<IT>{};
      if (ok[u][k]) raw[u][k] = raw_load(src + j * 8);
    }
    if (a.gate && !second[u]) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        if (ok[u][k]) oct_store(static_cast<IT*>(a.gate) + out_off[u] + j * 8, oct_load(src + a.d + j * 8));
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kRows; ++u) {
    Oct x[K];
#pragma unroll
    for (int k = 0; k < K; ++k) x[k] = raw_unpack(raw[u][k]);
    if (a.w) {  // the norm kernel's arithmetic for a row of this length, step for step
      float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int k = 0; k < K; ++k) acc = oct_sumsq(x[k], acc);
      const float ss = group_sum(acc.x + acc.y, g, nullptr);  // g <= 32: shuffles only
      const float scale = rsqrtf(__fmaf_rn(ss, inv_d, a.eps));
      const float* w = second[u] ? a.w2 : a.w;  // 1 KiB, resident in L1 after the first rows
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned j = (k << lg) + lir;
        Oct gm = j < octs ? oct_load_cached(w + j * 8) : oct_zero();
        if (a.one_plus) {
          const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
          for (int i = 0; i < 4; ++i) gm.p[i] = __fadd2_rn(one, gm.p[i]);
        }
        x[k] = oct_mul(oct_scale(x[k], scale), gm);
      }
    }
    float v[8];
    oct_to_array(x[0], v);
    const float2* tab = lane_tab + tl[u] * half;
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
    OT* dst = static_cast<OT*>(second[u] ? a.out2 : a.out) + out_off[u];
    void* cache = second[u] ? a.cache2 : a.cache;
    OT* cdst = cache ? static_cast<OT*>(cache) + out_off[u] : nullptr;
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

template <typename IT, typename OT>
cudaError_t LaunchNormRopeT(const NormRopeArgs& a, const InvFreq& f, cudaStream_t s) {
  const unsigned octs = a.d / 8;
  // Two octets per lane halve the instructions per row; the rotated span must then sit in
  // the first octet of the lanes (rot <= d / 2), which holds for 64-of-256 and 16-of-64.
  const int k = (octs >= 2 && a.rot * 2 <= a.d) ? 2 : 1;
  unsigned g = 1, lg = 0;
  while (g * k < octs) g <<= 1, ++lg;
  const unsigned rows_per_cta = kBlock / g * kRows;
  const unsigned hall = a.heads + a.heads2;
  const unsigned tokens = (a.rows + a.heads - 1) / a.heads;
  const uint64_t rows_total = static_cast<uint64_t>(tokens) * hall;
  if (rows_total > 0xFFFFFFFFull) return cudaErrorInvalidValue;
  const unsigned grid = static_cast<unsigned>((rows_total + rows_per_cta - 1) / rows_per_cta);
  const unsigned max_tok = rows_per_cta / hall + 2;  // tokens a CTA's rows can touch
  const size_t smem = 2 * static_cast<size_t>(max_tok) * (a.rot / 2) * sizeof(float2);
  if (smem > 48u * 1024u) return cudaErrorInvalidValue;
  const float inv_d = 1.0f / static_cast<float>(a.d);
  // floor(n / hall) == umulhi(n, ceil(2^32 / hall)) whenever n * hall < 2^32
  const uint32_t magic = (hall > 1 && rows_total * hall < (1ull << 32))
                             ? static_cast<uint32_t>(((1ull << 32) + hall - 1) / hall)
                             : 0u;
  const uint32_t rt = static_cast<uint32_t>(rows_total);
  if (k == 2) norm_rope_kernel<IT, OT, 2><<<grid, kBlock, smem, s>>>(a, f, lg, rt, inv_d, magic);
  else norm_rope_kernel<IT, OT, 1><<<grid, kBlock, smem, s>>>(a, f, lg, rt, inv_d, magic);
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
