// Device helpers shared by the sm_100a layer-op kernels: element types, 8-element
// ("octet") vector loads and stores, group reductions, activations.
//
// Arithmetic rules for every kernel in this library (they make the results
// comparable with halo-flash's scalar CPU operators, src/model/cpu_ops.cpp):
//   * fp32 arithmetic compiled with -fmad=false, so scalar multiplies and adds round
//     separately as on the CPU. The deliberate departures, all far inside the 1e-5 the
//     path allows: the sum of squares (fused multiply-adds in fp32; the CPU sums in
//     double), the norm scale (hardware rsqrt, 2 ulp), the gate functions (hardware
//     exp2 / reciprocal, .ftz forms) and the conv taps (an FMA chain in tap order);
//   * packed fp32x2 instructions (FMUL2 / FADD2 / FFMA2) are used only where no product
//     feeds a sum whose two roundings matter: ptxas contracts a packed multiply into the
//     packed add that consumes it - measured on sm_100a, also for inline PTX that names
//     .rn on both - so every "a * b + c * d as the CPU rounds it" (the rotation, the
//     experts' sum, the combine into an fp32 residual) is written with scalar
//     multiplies and adds;
//   * the Q8 encoders produce the scales and codes of the CPU's IEEE divisions bit for
//     bit without dividing (div127, round_div_codes below);
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

// Programmatic dependent launch. Every kernel of the library starts with pdl_begin() (some after issuing L2 hints,
// below): it waits until the kernel before this one in the stream has completed and its writes are visible, and
// then lets the kernel after this one be scheduled, whose CTAs sit in their own pdl_begin() until this grid has
// completed. Nothing is read or written before the wait. The launch gap between two 12-microsecond kernels (CTA
// scheduling, parameter fetch, index arithmetic) thereby overlaps the tail of the earlier kernel. Both instructions
// are no-ops in a kernel launched without the attribute LaunchKernel() sets.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// When to let the kernel behind be scheduled. Triggering at the top of the kernel lets every later launch of a stream
// or graph become resident at once, each parked in its own wait: behind launches of a few dozen to a few hundred CTAs
// that pile-up made the latency-bound kernels up to 40 % slower than plain launches (add + norm of 256 rows 3.4 us
// against 2.8 plain, 2.0 us with the trigger after the wait; the 230-launch chain 0.450 -> 0.381 ms at 128 tokens,
// 0.512 -> 0.481 at 256; the decode step 317 -> 292 us). A launch that fills the GPU leaves no room for a pile-up and
// gains a little from the early trigger (its successor's first CTAs get their hints out sooner). So: at the top
// for grids of kEarlyTriggerCtas and more, after the wait otherwise (256, 512 and 1024 measured within 1 % of each
// other on the chain at 128 .. 1024 tokens; at 512 tokens alone the early trigger everywhere was 3 % faster).
#ifndef HALO_EARLY_CTAS
#define HALO_EARLY_CTAS 512
#endif
constexpr unsigned kEarlyTriggerCtas = HALO_EARLY_CTAS;
__device__ __forceinline__ void pdl_trigger_early() {
  if (gridDim.x >= kEarlyTriggerCtas) pdl_launch_dependents();
}
__device__ __forceinline__ void pdl_wait_and_trigger() {
  pdl_wait();
  pdl_launch_dependents();  // a second trigger of a grid that triggered early is a no-op
}
// A kernel without anything to do ahead of its wait starts with this.
__device__ __forceinline__ void pdl_begin() {
  pdl_trigger_early();
  pdl_wait_and_trigger();
}

// Ahead of pdl_begin() a CTA may ask L2 for the span of global memory it is about to read
// (`bytes` a multiple of 16, p 16-byte aligned; one thread, one instruction). A prefetch is only a hint and L2 is
// the point of coherence, so this is safe even when the kernel ahead still has to WRITE those bytes (its stores
// update the line in L2). What it buys: the CTAs that sit in griddepcontrol.wait while the kernel ahead drains
// do not all leave it into an empty memory pipeline - their first loads find L2. Measured on 4096-token launches:
// SwiGLU 22.4 -> 21.5 us, gated norm 16.5 -> 15.7, add + norm 11.7 -> 11.4, hyper-connection combine 37.8 -> 34.4.
// Which kernels do it is decided per kernel at compile time, because the preamble is not free: the general form of the
// Q8-epilogue norm kernel (all outputs tested at run time, 44 - 48 registers x 5 CTAs) lost 7 - 12 % from its mere
// presence, and launches of a few rows (decode) gain nothing from a hint. The epilogue kernel's fixed modes (40 - 45
// registers) do gain - 12.3 -> 11.0 us at 4096 tokens with both hints - and are compiled with and without them.
#ifndef HALO_PF_NORM
#define HALO_PF_NORM 1
#endif
#ifndef HALO_PF_NORM_EPI
#define HALO_PF_NORM_EPI 1
#endif
#ifndef HALO_PF_GATED
#define HALO_PF_GATED 1
#endif
#ifndef HALO_PF_ELT
#define HALO_PF_ELT 1
#endif
#ifndef HALO_PF_ROPE_STAGED
#define HALO_PF_ROPE_STAGED 1
#endif
#ifndef HALO_PF_HC
#define HALO_PF_HC 1
#endif
#ifndef HALO_PF_CONV
#define HALO_PF_CONV 1
#endif
#ifndef HALO_PF_ROPE_GENERAL
#define HALO_PF_ROPE_GENERAL 1
#endif
#ifndef HALO_PF_HC_ELT
#define HALO_PF_HC_ELT 1
#endif
#ifndef HALO_PF_QUANT
#define HALO_PF_QUANT 1
#endif
#ifndef HALO_PF_MOE
#define HALO_PF_MOE 1
#endif
// One-shot CTAs run in waves that load, then compute, in step with each other, so HBM idles while a wave computes.
// With "prefetch ahead" a CTA, once its own loads are issued, hints to L2 the inputs of the CTA one wave of resident
// CTAs later (148 SMs x resident CTAs per SM), which keeps HBM busy through the compute phase. Measured at 4096 /
// 65 536 tokens: add + norm 11.4 -> 10.4 us / 158 -> 158; L2 norm 10.6 -> 9.9 / 156 -> 169 (worse: after a few
// dozen waves the CTAs are out of step anyway and the hint only adds L2 traffic); gated norm 15.8 -> 14.8 /
// 240 -> 235; SwiGLU 21.5 -> 21.8 / 314 -> 371; the Q8-epilogue norm in its fixed modes 12.4 -> 11.0 (with the hint
// before the wait; 13.6 without it) / no change. Hence: the norm kernels do it for launches of up to kAheadMaxWaves
// waves, the gated norm always, the others never.
#ifndef HALO_PF_AHEAD_NORM
#define HALO_PF_AHEAD_NORM 1
#endif
#ifndef HALO_PF_AHEAD_GATED
#define HALO_PF_AHEAD_GATED 1
#endif
constexpr unsigned kSms = 148;
constexpr unsigned kAheadMaxWaves = 16;
__device__ __forceinline__ void prefetch_l2_span(const void* p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

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

// ---- octets as four float2 pairs (packed fp32x2 arithmetic on sm_100) --------------
// The row kernels are bound by instruction issue as much as by HBM, so their inner
// math runs on FADD2 / FMUL2 / FFMA2: one instruction per two elements, each lane
// rounded exactly as the scalar instruction would.
struct Oct {
  float2 p[4];
};
__device__ __forceinline__ Oct oct_zero() {
  Oct o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.p[i] = make_float2(0.0f, 0.0f);
  return o;
}
__device__ __forceinline__ Oct oct_unpack_bf16(uint4 u) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  Oct o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.p[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
  return o;
}
__device__ __forceinline__ uint4 oct_pack_bf16(const Oct& o) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(o.p[i].x, o.p[i].y);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ Oct oct_unpack_f16(uint4 u) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  Oct o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.p[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
  return o;
}
__device__ __forceinline__ uint4 oct_pack_f16(const Oct& o) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(o.p[i].x, o.p[i].y);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ Oct oct_load(const float* p) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  Oct o;
  o.p[0] = make_float2(a.x, a.y); o.p[1] = make_float2(a.z, a.w);
  o.p[2] = make_float2(b.x, b.y); o.p[3] = make_float2(b.z, b.w);
  return o;
}
__device__ __forceinline__ Oct oct_load(const bf16* p) { return oct_unpack_bf16(__ldcs(reinterpret_cast<const uint4*>(p))); }
__device__ __forceinline__ Oct oct_load(const f16* p) { return oct_unpack_f16(__ldcs(reinterpret_cast<const uint4*>(p))); }
__device__ __forceinline__ Oct oct_load_cached(const float* p) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  Oct o;
  o.p[0] = make_float2(a.x, a.y); o.p[1] = make_float2(a.z, a.w);
  o.p[2] = make_float2(b.x, b.y); o.p[3] = make_float2(b.z, b.w);
  return o;
}
__device__ __forceinline__ void oct_store(float* p, const Oct& o) {
  reinterpret_cast<float4*>(p)[0] = make_float4(o.p[0].x, o.p[0].y, o.p[1].x, o.p[1].y);
  reinterpret_cast<float4*>(p)[1] = make_float4(o.p[2].x, o.p[2].y, o.p[3].x, o.p[3].y);
}
__device__ __forceinline__ void oct_store(bf16* p, const Oct& o) { *reinterpret_cast<uint4*>(p) = oct_pack_bf16(o); }
__device__ __forceinline__ void oct_store(f16* p, const Oct& o) { *reinterpret_cast<uint4*>(p) = oct_pack_f16(o); }
// Store, and leave in `o` the values a later reader of the buffer sees.
__device__ __forceinline__ void oct_store_round(float* p, Oct& o) { oct_store(p, o); }
__device__ __forceinline__ void oct_store_round(bf16* p, Oct& o) {
  const uint4 u = oct_pack_bf16(o);
  *reinterpret_cast<uint4*>(p) = u;
  o = oct_unpack_bf16(u);
}
__device__ __forceinline__ void oct_store_round(f16* p, Oct& o) {
  const uint4 u = oct_pack_f16(o);
  *reinterpret_cast<uint4*>(p) = u;
  o = oct_unpack_f16(u);
}
// Store, rounded, with an L2 "keep" hint: for a buffer that is read again a few kernels later (the residual
// stream: 16.8 MB at 4096 x 2048 bf16, re-read by the next add + norm after 100-250 MB of other traffic has
// passed through the 126 MB L2). `policy` comes from l2_keep_policy().
__device__ __forceinline__ uint64_t l2_keep_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// The keep policy, or the ordinary one when the buffer is too large to stay (selected without a branch).
__device__ __forceinline__ uint64_t l2_policy(bool keep) {
  uint64_t normal;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(normal));
  const uint64_t last = l2_keep_policy();
  return keep ? last : normal;
}
__device__ __forceinline__ void store16_keep(void* p, uint4 u, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(p), "r"(u.x), "r"(u.y), "r"(u.z),
               "r"(u.w), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void oct_store_round_keep(float* p, Oct& o, uint64_t policy) {
  store16_keep(p, make_uint4(__float_as_uint(o.p[0].x), __float_as_uint(o.p[0].y), __float_as_uint(o.p[1].x),
                             __float_as_uint(o.p[1].y)), policy);
  store16_keep(p + 4, make_uint4(__float_as_uint(o.p[2].x), __float_as_uint(o.p[2].y), __float_as_uint(o.p[3].x),
                                 __float_as_uint(o.p[3].y)), policy);
}
__device__ __forceinline__ void oct_store_round_keep(bf16* p, Oct& o, uint64_t policy) {
  const uint4 u = oct_pack_bf16(o);
  store16_keep(p, u, policy);
  o = oct_unpack_bf16(u);
}
__device__ __forceinline__ void oct_store_round_keep(f16* p, Oct& o, uint64_t policy) {
  const uint4 u = oct_pack_f16(o);
  store16_keep(p, u, policy);
  o = oct_unpack_f16(u);
}
__device__ __forceinline__ Oct oct_add(const Oct& a, const Oct& b) {
  Oct o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.p[i] = __fadd2_rn(a.p[i], b.p[i]);
  return o;
}
__device__ __forceinline__ Oct oct_mul(const Oct& a, const Oct& b) {
  Oct o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.p[i] = __fmul2_rn(a.p[i], b.p[i]);
  return o;
}
__device__ __forceinline__ Oct oct_scale(const Oct& a, float s) {
  const float2 s2 = make_float2(s, s);
  Oct o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.p[i] = __fmul2_rn(a.p[i], s2);
  return o;
}
// acc += a * a per lane (fused: the sum of squares is the one place an FMA is used)
__device__ __forceinline__ float2 oct_sumsq(const Oct& a, float2 acc) {
#pragma unroll
  for (int i = 0; i < 4; ++i) acc = __ffma2_rn(a.p[i], a.p[i], acc);
  return acc;
}
__device__ __forceinline__ void oct_to_array(const Oct& o, float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) v[2 * i] = o.p[i].x, v[2 * i + 1] = o.p[i].y;
}

// Raw octets: the loaded bits, converted only where they are consumed, so a thread that
// issues many loads up front holds 4 registers per 16-bit octet instead of 8.
template <typename T>
struct Raw;
template <>
struct Raw<float> {
  float4 a, b;
};
template <>
struct Raw<bf16> {
  uint4 u;
};
template <>
struct Raw<f16> {
  uint4 u;
};
__device__ __forceinline__ Raw<float> raw_load(const float* p) {
  Raw<float> r;
  r.a = __ldcs(reinterpret_cast<const float4*>(p));
  r.b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  return r;
}
__device__ __forceinline__ Raw<bf16> raw_load(const bf16* p) {
  Raw<bf16> r;
  r.u = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}
__device__ __forceinline__ Raw<f16> raw_load(const f16* p) {
  Raw<f16> r;
  r.u = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}
__device__ __forceinline__ Oct raw_unpack(const Raw<float>& r) {
  Oct o;
  o.p[0] = make_float2(r.a.x, r.a.y); o.p[1] = make_float2(r.a.z, r.a.w);
  o.p[2] = make_float2(r.b.x, r.b.y); o.p[3] = make_float2(r.b.z, r.b.w);
  return o;
}
__device__ __forceinline__ Oct raw_unpack(const Raw<bf16>& r) { return oct_unpack_bf16(r.u); }
__device__ __forceinline__ Oct raw_unpack(const Raw<f16>& r) { return oct_unpack_f16(r.u); }

// Sum of two 16-bit octets IN their storage type: four packed add.rn instructions instead of two unpacks, four
// packed fp32 adds and a pack (24 instructions). The result is the residual the fp32 path stores, bit for bit:
// for two bf16 (fp16) operands the fp32 sum is exact whenever their exponents are at most 16 (13) apart, and
// beyond that the smaller operand is below half a unit in the last place of the larger one either way, so
// "add in fp32, round once to 16 bits" and the correctly rounded 16-bit add agree for all finite inputs.
__device__ __forceinline__ uint32_t add2_bf16(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t add2_f16(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ Raw<bf16> raw_add(const Raw<bf16>& a, const Raw<bf16>& b) {
  Raw<bf16> r;
  r.u = make_uint4(add2_bf16(a.u.x, b.u.x), add2_bf16(a.u.y, b.u.y), add2_bf16(a.u.z, b.u.z), add2_bf16(a.u.w, b.u.w));
  return r;
}
__device__ __forceinline__ Raw<f16> raw_add(const Raw<f16>& a, const Raw<f16>& b) {
  Raw<f16> r;
  r.u = make_uint4(add2_f16(a.u.x, b.u.x), add2_f16(a.u.y, b.u.y), add2_f16(a.u.z, b.u.z), add2_f16(a.u.w, b.u.w));
  return r;
}

// ---- reductions ---------------------------------------------------------------
// Sum over the `g` threads of a row group (g a power of two, g <= kBlock, groups
// aligned to g within the CTA). g <= 32: shuffles only. g > 32: one shared-memory
// stage; `scratch` holds kBlock / 32 floats and every thread of the CTA must call.
__device__ __forceinline__ float group_sum(float v, unsigned g, float* scratch) {
  // Butterfly over min(g, 32) lanes, widest stride first. Fully unrolled with warp-uniform
  // guards: the same additions in the same order as a loop from g/2 down to 1, without its
  // loop-carried compare and branch.
#pragma unroll
  for (unsigned o = 16; o > 0; o >>= 1)
    if (o < g) v += __shfl_xor_sync(kFullMask, v, o);
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

// The same for g <= 32 with no shared-memory stage in the code at all. Kernels that can only see
// short rows use this form: the mere presence of the (never executed) barrier path of
// group_sum cost the one-octet-per-thread kernels about 9 % (18.1 vs 16.6 us on the gated norm).
__device__ __forceinline__ float group_sum_narrow(float v, unsigned g) {
#pragma unroll
  for (unsigned o = 16; o > 0; o >>= 1)
    if (o < g) v += __shfl_xor_sync(kFullMask, v, o);
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
// sigmoid(x) = 1 / (1 + exp(-x)) on the hardware exp2 and reciprocal units: one multiply
// (-x * log2 e), ex2.approx, one add, rcp.approx - 4 instructions instead of ~30 for the IEEE
// expf + division, which made the gate math, not HBM, the bound of SwiGLU and the gated norm.
// The .ftz forms are spelled out: the default (denormal-preserving) forms wrap each unit in a
// range test and two rescaling multiplies, which the instruction histogram showed as six
// multiplies per element. Flushing is harmless here: a denormal exponent argument gives 2^0 = 1
// either way, exp underflows only where 1 + e == 1, and 1 + e >= 1 is never denormal.
// Relative error <= ~1e-6 for |x| <= 30 and <= ~6e-8 * |x| beyond (the product rounds once),
// against the 1e-5 the path allows; x -> -inf gives e = +inf and a gate of exactly 0, as the
// CPU operator does.
__device__ __forceinline__ float ex2_approx(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
__device__ __forceinline__ float rcp_approx(float t) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
__device__ __forceinline__ float sigmoid_f(float x) { return rcp_approx(1.0f + ex2_approx(x * -1.4426950408889634f)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
// Two gates at once: the multiply, the add and the final product are packed fp32x2 instructions
// (the exp2 and the reciprocal stay one per value), 3.5 issue slots per value instead of 5.
// Each lane computes exactly what sigmoid_f / silu_f compute.
__device__ __forceinline__ float2 sigmoid2_f(float2 x) {
  const float2 t = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  const float2 d = __fadd2_rn(make_float2(1.0f, 1.0f), make_float2(ex2_approx(t.x), ex2_approx(t.y)));
  return make_float2(rcp_approx(d.x), rcp_approx(d.y));
}
__device__ __forceinline__ float2 silu2_f(float2 x) { return __fmul2_rn(x, sigmoid2_f(x)); }

// ---- Q8 block epilogues (32 values = the 4 lanes of a quad, 8 values each) ----
// Three-input maximum (one FMNMX3 on sm_100): max3f ignores NaN operands as fmaxf does, max3f_nan
// returns NaN when any operand is NaN.
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float max3f_nan(float a, float b, float c) {
  float r;
  asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// max |v[i]| over 8 values in four instructions.
__device__ __forceinline__ float amax8(const float (&v)[8]) {
  const float a = max3f(fabsf(v[0]), fabsf(v[1]), fabsf(v[2]));
  const float b = max3f(fabsf(v[3]), fabsf(v[4]), fabsf(v[5]));
  return fmaxf(max3f(fabsf(v[6]), fabsf(v[7]), a), b);
}
// Maximum |v| over the quad this lane belongs to; all 32 lanes must call.
__device__ __forceinline__ float quad_amax(const float (&v)[8]) {
  float m = amax8(v);
  m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 1));
  m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 2));
  return m;
}

// x / 127.0f, correctly rounded, without the division: q0 = x * z with z = RN(1 / 127), the exact
// remainder r = x - 127 q0 from one FMA, and the correction q0 + r z from a second. Equal to the IEEE
// quotient for EVERY non-negative finite float, subnormals included (checked exhaustively over all 2^31 - 2^23
// bit patterns against the host's division); infinity and NaN pass through q0, as x / 127 gives them.
__device__ __forceinline__ float div127(float x) {
  constexpr float z = 1.0f / 127.0f;
  const float q0 = __fmul_rn(x, z);
  const float r = __fmaf_rn(-q0, 127.0f, x);
  const float q = __fmaf_rn(r, z, q0);
  return fabsf(x) < __int_as_float(0x7F800000) ? q : q0;
}

// q[i] = clamp(rint(v[i] / d), +-127) for 8 values as 8 packed two's-complement bytes, with the
// results of the IEEE division but (almost always) without dividing. t = v * rcp(d) is within
// 2.3e-5 of the real quotient for |t| <= 127.5 and the correctly rounded quotient within 8e-6,
// so whenever t is farther than 1e-4 from a rounding boundary (n + 0.5) both round to the same
// integer. Rounding to nearest-even is the add of 1.5 * 2^23 (fused with the product: away from a boundary
// the singly and the doubly rounded sums are the same integer), whose low mantissa byte is the
// code. The fast path also skips the clamp: with |v| <= amax and d a normal half within 2^-11
// of amax / 127 the quotient stays below 127.1. A thread redoes its 8 values with the division
// and the clamp when one of them is within 1e-4 of a boundary (about 1 in 600) or is NaN (the
// distance is then NaN and the NaN-propagating maximum fails the test), or when d is a subnormal
// half, infinite or NaN. Clamping before the rounding equals clamping after it (the bounds are
// integers), and NaN clamps to -127 either way. The fast path runs on packed fp32x2 instructions.
__device__ __forceinline__ uint2 round_div_codes(const float (&v)[8], float d) {
  constexpr float kMagic = 12582912.0f;
  const float r = rcp_approx(d);
  const float2 r2 = make_float2(r, r), magic2 = make_float2(kMagic, kMagic), minus2 = make_float2(-1.0f, -1.0f);
  uint32_t bits[8];
  float2 f[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // three packed FMAs per pair: s = v r + magic (the rounding), -n = magic - s (exact), f = v r - n (the distance
    // of the unrounded quotient from the integer it was rounded to, with a single rounding)
    const float2 vv = make_float2(v[2 * i], v[2 * i + 1]);
    const float2 s = __ffma2_rn(vv, r2, magic2);
    const float2 nn = __ffma2_rn(s, minus2, magic2);
    f[i] = __ffma2_rn(vv, r2, nn);
    bits[2 * i] = __float_as_uint(s.x);
    bits[2 * i + 1] = __float_as_uint(s.y);
  }
  const float far = max3f_nan(max3f_nan(fabsf(f[0].x), fabsf(f[0].y), fabsf(f[1].x)),
                              max3f_nan(fabsf(f[1].y), fabsf(f[2].x), fabsf(f[2].y)),
                              max3f_nan(fabsf(f[3].x), fabsf(f[3].y), 0.0f));
  const bool ok = d >= 6.2e-5f && d < 1e30f && far <= 0.4999f;
  if (!ok) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float t = fminf(fmaxf(__fdiv_rn(v[i], d), -127.0f), 127.0f);
      bits[i] = __float_as_uint(__fadd_rn(t, kMagic));
    }
  }
  return make_uint2(__byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410),
                    __byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410));
}

// True Q8_0 (src/core/lowbit.cpp:285-298): d = half(amax / 127); q = clamp(rint(x / float(d)), +-127),
// 0 when d == 0. Returns the 8 codes packed little-endian and the scale bits.
__device__ __forceinline__ uint2 q8_0_codes(const float (&v)[8], float amax, uint16_t* dbits) {
  const f16 dh = __float2half_rn(div127(amax));
  const float d = __half2float(dh);
  *dbits = __half_as_ushort(dh);
  return d > 0.0f ? round_div_codes(v, d) : make_uint2(0u, 0u);
}

// int8 activation form (src/kernels/core.hip:3086-3101): scale = amax / 127 in fp32,
// q = rint(v / scale), 0 when scale == 0. (|v| <= amax keeps the quotient within +-127.)
__device__ __forceinline__ uint2 i8_codes(const float (&v)[8], float scale) {
  return scale > 0.0f ? round_div_codes(v, scale) : make_uint2(0u, 0u);
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
