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

constexpr int kUnroll = 4;

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
    o = oct_add(a, oct_scale(b, alpha));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (OP == kOpSiluMul) {
        const float2 s = make_float2(silu_f(a.p[i].x), silu_f(a.p[i].y));
        o.p[i] = __fmul2_rn(s, b.p[i]);
      } else {
        const float2 s = make_float2(sigmoid_f(b.p[i].x), sigmoid_f(b.p[i].y));
        o.p[i] = __fmul2_rn(a.p[i], s);
      }
    }
  }
  return o;
}

// The raw loads of all kUnroll octets are issued first (kUnroll * 2 * 16 bytes in flight per
// thread); each octet is then converted, computed and stored in turn, which keeps the
// register count low enough for 5 resident CTAs per SM.
template <typename IT, typename OT, int OP>
__global__ void __launch_bounds__(kBlock, sizeof(IT) == 4 ? 3 : 5) elementwise_vec_kernel(const EltArgs a, const uint64_t octs) {
  const IT* pa = static_cast<const IT*>(a.a);
  const IT* pb = static_cast<const IT*>(a.b);
  OT* py = static_cast<OT*>(a.y);
  const uint64_t base = static_cast<uint64_t>(blockIdx.x) * (kBlock * kUnroll) + threadIdx.x;
  if (base + static_cast<uint64_t>(kUnroll - 1) * kBlock < octs) {  // the whole CTA tile is inside: no predicates
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
      oct_store(py + j * 8, apply8<OP>(raw_unpack(ra[u]), raw_unpack(rb[u]), a.alpha));
    }
  } else {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t j = base + static_cast<uint64_t>(u) * kBlock;
      if (j < octs) oct_store(py + j * 8, apply8<OP>(oct_load(pa + j * 8), oct_load(pb + j * 8), a.alpha));
    }
  }
}

// Scalar path: unaligned buffers and the < 8 element tail of the vector path.
template <typename IT, typename OT, int OP>
__global__ void __launch_bounds__(kBlock) elementwise_scalar_kernel(const EltArgs a, const uint64_t begin) {
  const IT* pa = static_cast<const IT*>(a.a);
  const IT* pb = static_cast<const IT*>(a.b);
  OT* py = static_cast<OT*>(a.y);
  for (uint64_t i = begin + static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < a.n;
       i += static_cast<uint64_t>(gridDim.x) * kBlock)
    py[i] = from_f32<OT>(apply(OP, to_f32(pa[i]), to_f32(pb[i]), a.alpha));
}

template <typename IT, typename OT, int OP>
cudaError_t LaunchOp(const EltArgs& a, cudaStream_t s) {
  uint64_t done = 0;
  if (a.vec) {
    const uint64_t octs = a.n / 8;
    if (octs) {
      const uint64_t per_cta = static_cast<uint64_t>(kBlock) * kUnroll;
      const uint64_t grid = (octs + per_cta - 1) / per_cta;
      if (grid > 0x7FFFFFFFull) return cudaErrorInvalidValue;
      elementwise_vec_kernel<IT, OT, OP><<<static_cast<unsigned>(grid), kBlock, 0, s>>>(a, octs);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
    }
    done = octs * 8;
  }
  if (done < a.n) {
    uint64_t grid = (a.n - done + kBlock - 1) / kBlock;
    if (grid > 148u * 32u) grid = 148u * 32u;
    elementwise_scalar_kernel<IT, OT, OP><<<static_cast<unsigned>(grid), kBlock, 0, s>>>(a, done);
    return cudaGetLastError();
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
  if (a.n == 0) return cudaSuccess;
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
