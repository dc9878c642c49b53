// Streaming elementwise ops for sm_100a: SwiGLU (SiLU(gate) * up), residual add,
// axpy and the sigmoid output gate. Replaces halo_silu_mul, halo_silu_mul_h,
// halo_add, halo_axpy and halo_sigmoid_gate (src/kernels/core.hip:313-339);
// arithmetic follows src/model/qwen35.cpp:322-329 and src/model/cpu_ops.cpp:158-163.
//
// Each thread owns kUnroll octets spaced one CTA-width apart, issues all of its
// 16-byte loads first and only then computes, so a CTA keeps
// kUnroll * 2 * 4 KiB of reads in flight with fully coalesced warp accesses.
#include "common.cuh"
#include "kernels.h"

namespace halo_b200 {
namespace {

// Two octets per thread: with the L2 hint ahead of the dependent-launch wait (below) the SwiGLU of 4096 tokens takes
// 20.4 us, against 21.5 us with four (more, shorter CTAs leave a shorter tail; four was faster before the hint).
#ifndef HALO_ELT_UNROLL
#define HALO_ELT_UNROLL 2
#endif
constexpr int kUnroll = HALO_ELT_UNROLL;

__device__ __forceinline__ float apply(int op, float a, float b, float alpha) {
  switch (op) {
    case kOpSiluMul: return silu_f(a) * b;
    case kOpAdd: return a + b;
    case kOpAxpy: return a + alpha * b;
    default: return a * sigmoid_f(b);
  }
}

template <int OP>
__device__ __forceinline__ Oct apply8(const Oct& a, const Oct& b, float alpha) {
  Oct o;
  if constexpr (OP == kOpAdd) {
    o = oct_add(a, b);
  } else if constexpr (OP == kOpAxpy) {
    // scalar on purpose: a packed multiply feeding a packed add was seen to contract into an FMA
#pragma unroll
    for (int i = 0; i < 4; ++i) o.p[i] = make_float2(a.p[i].x + alpha * b.p[i].x, a.p[i].y + alpha * b.p[i].y);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (OP == kOpSiluMul) o.p[i] = __fmul2_rn(silu2_f(a.p[i]), b.p[i]);
      else o.p[i] = __fmul2_rn(a.p[i], sigmoid2_f(b.p[i]));
    }
  }
  return o;
}

// Kernel-side view of the segments: CTA b belongs to the segment s with
// first_cta[s] <= b < first_cta[s + 1]; a CTA never straddles two tensors.
struct VecSegments {
  const void* a[kMaxSegments];
  const void* b[kMaxSegments];
  void* y[kMaxSegments];
  uint64_t octs[kMaxSegments];
  uint32_t first_cta[kMaxSegments + 1];
  float alpha;
};

// The raw loads of all kUnroll octets are issued first (kUnroll * 2 * 16 bytes in flight per
// thread); each octet is then converted, computed and stored in turn, which keeps the
// register count low enough for 5 resident CTAs per SM.
// U octets per thread: kUnroll for streaming sizes; 1 when the whole launch cannot fill the GPU (decode),
// where its duration is one warp's chain of dependent instructions and the shortest chain wins.
template <typename IT, typename OT, int OP, int U>
__global__ void __launch_bounds__(kBlock, sizeof(IT) == 4 ? 3 : 5) elementwise_vec_kernel(const VecSegments v) {
  constexpr int kUnroll = U;  // shadows the file-scope constant inside this kernel
  pdl_trigger_early();
  // Segment lookup by compare-and-select over constant indices: indexing the parameter arrays
  // with a run-time value would make the compiler copy them to local memory.
  const void* sa = v.a[0];
  const void* sb = v.b[0];
  void* sy = v.y[0];
  uint64_t octs = v.octs[0];
  uint32_t first = 0;
#pragma unroll
  for (int i = 1; i < kMaxSegments; ++i) {
    if (blockIdx.x >= v.first_cta[i]) {
      sa = v.a[i], sb = v.b[i], sy = v.y[i], octs = v.octs[i], first = v.first_cta[i];
    }
  }
  const IT* pa = static_cast<const IT*>(sa);
  const IT* pb = static_cast<const IT*>(sb);
  OT* py = static_cast<OT*>(sy);
  if (HALO_PF_ELT != 0 && threadIdx.x == 0) {  // the CTA's kBlock * kUnroll octets are one contiguous span of each input
    const uint64_t o0 = static_cast<uint64_t>(blockIdx.x - first) * (kBlock * kUnroll);
    const uint64_t n = octs - o0 < static_cast<uint64_t>(kBlock * kUnroll) ? octs - o0 : static_cast<uint64_t>(kBlock * kUnroll);
    prefetch_l2_span(pa + o0 * 8, static_cast<unsigned>(n * 8 * sizeof(IT)));
    prefetch_l2_span(pb + o0 * 8, static_cast<unsigned>(n * 8 * sizeof(IT)));
  }
  pdl_wait_and_trigger();
  const uint64_t base = static_cast<uint64_t>(blockIdx.x - first) * (kBlock * kUnroll) + threadIdx.x;
  if (base + static_cast<uint64_t>(kUnroll - 1) * kBlock < octs) {  // the whole tile is inside: no predicates
    Raw<IT> ra[kUnroll], rb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t j = base + static_cast<uint64_t>(u) * kBlock;
      ra[u] = raw_load(pa + j * 8);
      rb[u] = raw_load(pb + j * 8);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t j = base + static_cast<uint64_t>(u) * kBlock;
      oct_store(py + j * 8, apply8<OP>(raw_unpack(ra[u]), raw_unpack(rb[u]), v.alpha));
    }
  } else {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t j = base + static_cast<uint64_t>(u) * kBlock;
      if (j < octs) oct_store(py + j * 8, apply8<OP>(oct_load(pa + j * 8), oct_load(pb + j * 8), v.alpha));
    }
  }
}

// Scalar path: unaligned buffers and the < 8 element tail of the vector path.
template <typename IT, typename OT, int OP>
__global__ void __launch_bounds__(kBlock) elementwise_scalar_kernel(const IT* pa, const IT* pb, OT* py,
                                                                   const uint64_t begin, const uint64_t n,
                                                                   const float alpha) {
  pdl_begin();
  for (uint64_t i = begin + static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += static_cast<uint64_t>(gridDim.x) * kBlock)
    py[i] = from_f32<OT>(apply(OP, to_f32(pa[i]), to_f32(pb[i]), alpha));
}

template <typename IT, typename OT, int OP>
cudaError_t LaunchOp(const EltArgs& a, cudaStream_t s) {
  uint64_t done[kMaxSegments] = {};
  if (a.vec) {
    VecSegments v = {};
    v.alpha = a.alpha;
    uint64_t total_octs = 0;
    for (int i = 0; i < a.nseg; ++i) total_octs += a.seg[i].n / 8;
    const bool tiny = total_octs <= 148u * 256u;
    const uint64_t per_cta = static_cast<uint64_t>(kBlock) * (tiny ? 1 : kUnroll);
    uint64_t ctas = 0;
    for (int i = 0; i < kMaxSegments; ++i) {
      v.first_cta[i] = static_cast<uint32_t>(ctas);
      if (i < a.nseg) {
        v.a[i] = a.seg[i].a;
        v.b[i] = a.seg[i].b;
        v.y[i] = a.seg[i].y;
        v.octs[i] = a.seg[i].n / 8;
        done[i] = v.octs[i] * 8;
        ctas += (v.octs[i] + per_cta - 1) / per_cta;
        if (ctas > 0x7FFFFFFFull) return cudaErrorInvalidValue;
      }
    }
    v.first_cta[kMaxSegments] = static_cast<uint32_t>(ctas);
    for (int i = a.nseg; i < kMaxSegments; ++i) v.first_cta[i] = 0xFFFFFFFFu;  // never selected
    if (ctas) {
      if (tiny) LaunchKernel(elementwise_vec_kernel<IT, OT, OP, 1>, static_cast<unsigned>(ctas), kBlock, 0, s, v);
      else LaunchKernel(elementwise_vec_kernel<IT, OT, OP, kUnroll>, static_cast<unsigned>(ctas), kBlock, 0, s, v);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
    }
  }
  for (int i = 0; i < a.nseg; ++i) {
    if (done[i] < a.seg[i].n) {
      uint64_t grid = (a.seg[i].n - done[i] + kBlock - 1) / kBlock;
      if (grid > 148u * 32u) grid = 148u * 32u;
      LaunchKernel(elementwise_scalar_kernel<IT, OT, OP>, static_cast<unsigned>(grid), kBlock, 0, s, 
          static_cast<const IT*>(a.seg[i].a), static_cast<const IT*>(a.seg[i].b), static_cast<OT*>(a.seg[i].y), done[i],
          a.seg[i].n, a.alpha);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
    }
  }
  return cudaSuccess;
}

template <typename IT, typename OT>
cudaError_t LaunchIO(const EltArgs& a, cudaStream_t s) {
  switch (a.op) {
    case kOpSiluMul: return LaunchOp<IT, OT, kOpSiluMul>(a, s);
    case kOpAdd: return LaunchOp<IT, OT, kOpAdd>(a, s);
    case kOpAxpy: return LaunchOp<IT, OT, kOpAxpy>(a, s);
    case kOpSigmoidGate: return LaunchOp<IT, OT, kOpSigmoidGate>(a, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t LaunchElementwise(const EltArgs& a, cudaStream_t s) {
  if (a.nseg < 1 || a.nseg > kMaxSegments) return cudaErrorInvalidValue;
  const int key = a.in_dtype * 3 + a.y_dtype;
  switch (key) {
    case kF32 * 3 + kF32: return LaunchIO<float, float>(a, s);
    case kF32 * 3 + kF16: return LaunchIO<float, f16>(a, s);
    case kF32 * 3 + kBF16: return LaunchIO<float, bf16>(a, s);
    case kF16 * 3 + kF16: return LaunchIO<f16, f16>(a, s);
    case kBF16 * 3 + kBF16: return LaunchIO<bf16, bf16>(a, s);
    case kBF16 * 3 + kF32: return LaunchIO<bf16, float>(a, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace halo_b200
