// Device helpers shared by the sm_100a layer-op kernels: element types, 8-element
// ("octet") vector loads and stores, group reductions, activations.
//
// Arithmetic rules for every kernel in this library (they make the results
// comparable with halo-flash's scalar CPU operators, src/model/cpu_ops.cpp):
//   * fp32 arithmetic, IEEE division / sqrt / expf / sincosf (no fast-math),
//     compiled with -fmad=false so multiplies and adds round separately;
//   * 16-bit outputs are rounded once, to nearest even, from the fp32 value
//     (bf16 as src/kernels/core.hip:70-73, fp16 as a _Float16 cast).
#ifndef HALO_B200_COMMON_CUH_
#define HALO_B200_COMMON_CUH_

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace halo_b200 {

constexpr unsigned kFullMask = 0xFFFFFFFFu;
constexpr int kBlock = 256;  // threads per CTA of every row kernel

using bf16 = __nv_bfloat16;
using f16 = __half;

// ---- scalar conversions -----------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(f16 v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ f16 from_f32<f16>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// The value a T-typed buffer holds after storing v (what a later reader sees).
template <typename T>
__device__ __forceinline__ float round_through(float v) { return to_f32(from_f32<T>(v)); }

// ---- octet (8 consecutive elements) loads and stores ------------------------
// p must be 16-byte aligned. Loads are streaming (each input byte is read once).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load8(const f16* p, float (&v)[8]) {
  const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
// Cached (non-streaming) variant for small tables reused by every row (gammas).
__device__ __forceinline__ void load8_cached(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void store8(f16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
__device__ __forceinline__ void round_through8(float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = round_through<T>(v[i]);
}
template <>
__device__ __forceinline__ void round_through8<float>(float (&)[8]) {}

// ---- reductions ---------------------------------------------------------------
// Sum over the `g` threads of a row group (g a power of two, g <= kBlock, groups
// aligned to g within the CTA). g <= 32: shuffles only. g > 32: one shared-memory
// stage; `scratch` holds kBlock / 32 floats and every thread of the CTA must call.
__device__ __forceinline__ float group_sum(float v, unsigned g, float* scratch) {
  const unsigned gl = g < 32u ? g : 32u;
  for (unsigned o = gl >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  if (g > 32u) {
    const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const unsigned wpg = g >> 5, first = (warp / wpg) * wpg;
    float t = 0.0f;
    for (unsigned i = 0; i < wpg; ++i) t += scratch[first + i];
    v = t;
  }
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}

// ---- activations: src/model/cpu_ops.cpp:158-163 -------------------------------
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }

// ---- Q8 block epilogues (32 values = the 4 lanes of a quad, 8 values each) ----
// Maximum |v| over the quad this lane belongs to; all 32 lanes must call.
__device__ __forceinline__ float quad_amax(const float (&v)[8]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 1));
  m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 2));
  return m;
}

// True Q8_0 (src/core/lowbit.cpp:285-298): d = half(amax / 127); q = clamp(rint(x / float(d)), +-127),
// 0 when d == 0. Returns the 8 codes packed little-endian and the scale bits.
__device__ __forceinline__ uint2 q8_0_codes(const float (&v)[8], float amax, uint16_t* dbits) {
  const f16 dh = __float2half_rn(amax / 127.0f);
  const float d = __half2float(dh);
  *dbits = __half_as_ushort(dh);
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float q = 0.0f;
    if (d > 0.0f) q = fminf(fmaxf(rintf(v[i] / d), -127.0f), 127.0f);
    const int qi = static_cast<int>(q);
    w[i >> 2] |= (static_cast<uint32_t>(qi) & 0xFFu) << (8 * (i & 3));
  }
  return make_uint2(w[0], w[1]);
}

// int8 activation form (src/kernels/core.hip:3086-3101): scale = amax / 127 in fp32,
// q = rint(v / scale), 0 when scale == 0.
__device__ __forceinline__ uint2 i8_codes(const float (&v)[8], float scale) {
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int qi = scale > 0.0f ? static_cast<int>(rintf(v[i] / scale)) : 0;
    w[i >> 2] |= (static_cast<uint32_t>(qi) & 0xFFu) << (8 * (i & 3));
  }
  return make_uint2(w[0], w[1]);
}

// 8 code bytes to an address that is only 2-byte aligned (inside a 34-byte block).
__device__ __forceinline__ void store_codes_u16(uint8_t* p, uint2 c) {
  uint16_t* q = reinterpret_cast<uint16_t*>(p);
  q[0] = static_cast<uint16_t>(c.x);
  q[1] = static_cast<uint16_t>(c.x >> 16);
  q[2] = static_cast<uint16_t>(c.y);
  q[3] = static_cast<uint16_t>(c.y >> 16);
}

}  // namespace halo_b200

#endif  // HALO_B200_COMMON_CUH_
