// Standalone Q8 activation quantizers for sm_100a. Replaces halo_quantize_q8_rows,
// halo_quantize_q8_kblocked (src/kernels/core.hip:3086-3101, 3313-3331) and
// halo_q8x_cols and halo_hc_norm_q8x (src/kernels/batch_decode.hip:197-222, 977-999: the
// same two-level quantizer behind xn = (res x scale) x norm_w), and adds the true Q8_0
// row encoder of src/core/lowbit.cpp:285-298 as a device op. The same block
// routines run as the epilogue of the fused add + RMSNorm kernel (norm.cu).
//
// One thread per octet; the four lanes of a quad hold one 32-value block and
// find its maximum with two shuffles.
#include "common.cuh"
#include "kernels.h"

namespace halo_b200 {
namespace {

template <typename XT>
__global__ void __launch_bounds__(kBlock) quantize_vec_kernel(const QuantArgs a) {
  pdl_trigger_early();
  const uint32_t opr = a.cols / 8;
  if (HALO_PF_QUANT != 0 && threadIdx.x == 0 && a.x_stride == a.cols) {  // dense rows: the CTA's octets are one span of x
    const uint64_t o0 = static_cast<uint64_t>(blockIdx.x) * kBlock, total = static_cast<uint64_t>(a.rows) * opr;
    const uint64_t n = total - o0 < kBlock ? total - o0 : kBlock;
    prefetch_l2_span(static_cast<const XT*>(a.x) + o0 * 8, static_cast<unsigned>(n * 8 * sizeof(XT)));
  }
  pdl_wait_and_trigger();
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x;
  const uint32_t row = static_cast<uint32_t>(idx / opr), j = static_cast<uint32_t>(idx % opr);
  const bool ok = row < a.rows;
  const uint32_t c0 = j * 8;
  float v[8];
  if (ok) {
    load8(static_cast<const XT*>(a.x) + static_cast<size_t>(row) * a.x_stride + c0, v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
  }
  if (a.pre_w && ok) {  // xn = (x * scale of the row's group) * w, kept as well as quantized
    const float sc = a.pre_scale[static_cast<size_t>(row) * (a.cols / a.pre_h) + c0 / a.pre_h];
    float w[8];
    load8_cached(a.pre_w + c0, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], sc), w[i]);
    store8(a.xn + static_cast<size_t>(row) * a.cols + c0, v);
  }
  const float amax = quad_amax(v);
  if (a.q8_0) {
    uint16_t dbits;
    const uint2 codes = q8_0_codes(v, amax, &dbits);
    if (ok) {
      uint8_t* blk = a.q8_0 + static_cast<size_t>(row) * (a.cols / 32) * 34 + static_cast<size_t>(c0 / 32) * 34;
      if ((c0 & 31u) == 0) *reinterpret_cast<uint16_t*>(blk) = dbits;
      store_codes_u16(blk + 2 + (c0 & 31u), codes);
    }
  }
  if (a.xq) {
    const float scale = div127(amax);
    const uint2 codes = i8_codes(v, scale);
    if (ok) {
      if (a.kb_tokens) {
        *reinterpret_cast<uint2*>(a.xq + (static_cast<size_t>(c0 / 64) * a.kb_tokens + row) * 64 + c0 % 64) = codes;
        if ((c0 & 31u) == 0) a.xd[static_cast<size_t>(c0 / 32) * a.kb_tokens + row] = scale;
      } else {
        *reinterpret_cast<uint2*>(a.xq + static_cast<size_t>(row) * a.cols + c0) = codes;
        if ((c0 & 31u) == 0) a.xd[static_cast<size_t>(row) * (a.cols / 32) + c0 / 32] = scale;
      }
    }
    if (a.xq2) {  // the residual v - q * scale, quantized again (two int8 levels)
      float r[8];
      const uint32_t w[2] = {codes.x, codes.y};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int q = static_cast<int8_t>((w[i >> 2] >> (8 * (i & 3))) & 0xFFu);
        r[i] = v[i] - static_cast<float>(q) * scale;
      }
      const float rmax = quad_amax(r);
      const float s2 = div127(rmax);
      const uint2 c2 = i8_codes(r, s2);
      if (ok) {
        *reinterpret_cast<uint2*>(a.xq2 + static_cast<size_t>(row) * a.cols + c0) = c2;
        if ((c0 & 31u) == 0) a.xd2[static_cast<size_t>(row) * (a.cols / 32) + c0 / 32] = s2;
      }
    }
  }
}

// One warp per 32-value block, one element per lane: any alignment.
template <typename XT>
__global__ void __launch_bounds__(kBlock) quantize_scalar_kernel(const QuantArgs a) {
  pdl_begin();
  const uint32_t bpr = a.cols / 32;
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t nblk = static_cast<uint64_t>(a.rows) * bpr;
  for (uint64_t b = static_cast<uint64_t>(blockIdx.x) * (kBlock / 32) + (threadIdx.x >> 5); b < nblk;
       b += static_cast<uint64_t>(gridDim.x) * (kBlock / 32)) {
    const uint32_t row = static_cast<uint32_t>(b / bpr), blk = static_cast<uint32_t>(b % bpr);
    const uint32_t c = blk * 32 + lane;
    float v = to_f32(static_cast<const XT*>(a.x)[static_cast<size_t>(row) * a.x_stride + c]);
    if (a.pre_w) {
      v = __fmul_rn(__fmul_rn(v, a.pre_scale[static_cast<size_t>(row) * (a.cols / a.pre_h) + c / a.pre_h]), a.pre_w[c]);
      a.xn[static_cast<size_t>(row) * a.cols + c] = v;
    }
    const float amax = warp_max(fabsf(v));
    if (a.q8_0) {
      const f16 dh = __float2half_rn(amax / 127.0f);
      const float d = __half2float(dh);
      float q = 0.0f;
      if (d > 0.0f) q = fminf(fmaxf(rintf(v / d), -127.0f), 127.0f);
      uint8_t* out = a.q8_0 + static_cast<size_t>(row) * bpr * 34 + static_cast<size_t>(blk) * 34;
      if (lane == 0) {
        out[0] = static_cast<uint8_t>(__half_as_ushort(dh) & 0xFFu);
        out[1] = static_cast<uint8_t>(__half_as_ushort(dh) >> 8);
      }
      out[2 + lane] = static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(q)));
    }
    if (a.xq) {
      const float scale = amax / 127.0f;
      const int q = scale > 0.0f ? static_cast<int>(rintf(v / scale)) : 0;
      if (a.kb_tokens) {
        a.xq[(static_cast<size_t>(c / 64) * a.kb_tokens + row) * 64 + c % 64] = static_cast<int8_t>(q);
        if (lane == 0) a.xd[static_cast<size_t>(blk) * a.kb_tokens + row] = scale;
      } else {
        a.xq[static_cast<size_t>(row) * a.cols + c] = static_cast<int8_t>(q);
        if (lane == 0) a.xd[static_cast<size_t>(row) * bpr + blk] = scale;
      }
      if (a.xq2) {
        const float r = v - static_cast<float>(q) * scale;
        const float s2 = warp_max(fabsf(r)) / 127.0f;
        const int q2 = s2 > 0.0f ? static_cast<int>(rintf(r / s2)) : 0;
        a.xq2[static_cast<size_t>(row) * a.cols + c] = static_cast<int8_t>(q2);
        if (lane == 0) a.xd2[static_cast<size_t>(row) * bpr + blk] = s2;
      }
    }
  }
}

template <typename XT>
cudaError_t LaunchQuantT(const QuantArgs& a, cudaStream_t s) {
  if (a.vec) {
    const uint64_t octs = static_cast<uint64_t>(a.rows) * (a.cols / 8);
    const uint64_t grid = (octs + kBlock - 1) / kBlock;
    if (grid > 0x7FFFFFFFull) return cudaErrorInvalidValue;
    LaunchKernel(quantize_vec_kernel<XT>, static_cast<unsigned>(grid), kBlock, 0, s, a);
  } else {
    const uint64_t nblk = static_cast<uint64_t>(a.rows) * (a.cols / 32);
    uint64_t grid = (nblk + kBlock / 32 - 1) / (kBlock / 32);
    if (grid > 148u * 32u) grid = 148u * 32u;
    LaunchKernel(quantize_scalar_kernel<XT>, static_cast<unsigned>(grid), kBlock, 0, s, a);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t LaunchQuantize(const QuantArgs& a, cudaStream_t s) {
  if (a.rows == 0 || a.cols == 0) return cudaSuccess;
  switch (a.x_dtype) {
    case kF32: return LaunchQuantT<float>(a, s);
    case kF16: return LaunchQuantT<f16>(a, s);
    case kBF16: return LaunchQuantT<bf16>(a, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace halo_b200
