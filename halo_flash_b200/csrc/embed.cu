// Token-embedding row gather with Q8_0 dequant for sm_100a. Replaces
// halo_matvec_q8_0_embed, _embed_p and _embed_rows (src/kernels/core.hip:91-97,
// 200-232); values follow src/core/quant.cpp:411-421 (fp16 scale x int8, exact in
// fp32) through src/model/cpu_ops.cpp:47-72.
//
// A Q8_0 row is cols / 32 blocks of 34 bytes (2-byte fp16 scale, 32 int8), so a
// block is only 2-byte aligned and cannot be read with vector loads directly.
// Each warp stages a whole row into shared memory with 16-byte cp.async copies
// (the row start is 16-byte aligned whenever row_bytes is a multiple of 16: 2176
// bytes at 2048 columns), then every lane picks one octet out of shared memory
// with 2-byte reads and writes one 16-byte (bf16 / fp16) or 32-byte (fp32) store.
#include "common.cuh"
#include "kernels.h"

namespace halo_b200 {
namespace {

constexpr int kWarps = kBlock / 32;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned sa = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

template <typename OT>
__global__ void __launch_bounds__(kBlock) embed_q8_0_kernel(const EmbedArgs a, const unsigned warps,
                                                           const unsigned row_smem) {
  pdl_begin();
  extern __shared__ __align__(16) uint8_t stage[];
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  if (warp >= warps) return;
  uint8_t* buf = stage + static_cast<size_t>(warp) * row_smem;
  const unsigned chunks = static_cast<unsigned>(a.row_bytes / 16);
  const unsigned octs = a.cols / 8;
  OT* out = static_cast<OT*>(a.out);
  for (uint32_t t = blockIdx.x * warps + warp; t < a.tokens; t += gridDim.x * warps) {
    const uint32_t id = a.ids ? a.ids[static_cast<size_t>(t) * a.id_stride + a.id_slot] : a.token;
    const bool in_range = a.vocab == 0 || id < a.vocab;
    if (in_range) {
      const uint8_t* src = a.table + static_cast<size_t>(id) * a.row_bytes;
      for (unsigned c = lane; c < chunks; c += 32) cp_async16(buf + c * 16, src + c * 16);
      cp_async_wait_all();
    }
    __syncwarp();
    for (unsigned j = lane; j < octs; j += 32) {
      float v[8];
      if (in_range) {
        const uint8_t* blk = buf + (j >> 2) * 34;
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(blk)));
        const uint16_t* q = reinterpret_cast<const uint16_t*>(blk + 2 + 8 * (j & 3u));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint16_t pair = q[i];
          v[2 * i] = d * static_cast<float>(static_cast<int8_t>(pair & 0xFFu));
          v[2 * i + 1] = d * static_cast<float>(static_cast<int8_t>(pair >> 8));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
      }
      store8(out + static_cast<size_t>(t) * a.cols + j * 8, v);
    }
    __syncwarp();  // the row buffer is reused by the next token
  }
}

// One thread per element, byte loads: any alignment, any row_bytes.
template <typename OT>
__global__ void __launch_bounds__(kBlock) embed_q8_0_scalar_kernel(const EmbedArgs a) {
  pdl_begin();
  OT* out = static_cast<OT*>(a.out);
  const size_t total = static_cast<size_t>(a.tokens) * a.cols;
  for (size_t idx = static_cast<size_t>(blockIdx.x) * kBlock + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * kBlock) {
    const uint32_t t = static_cast<uint32_t>(idx / a.cols), c = static_cast<uint32_t>(idx % a.cols);
    const uint32_t id = a.ids ? a.ids[static_cast<size_t>(t) * a.id_stride + a.id_slot] : a.token;
    float v = 0.0f;
    if (a.vocab == 0 || id < a.vocab) {
      const uint8_t* b = a.table + static_cast<size_t>(id) * a.row_bytes + static_cast<size_t>(c / 32) * 34;
      const uint16_t dbits = static_cast<uint16_t>(b[0] | (b[1] << 8));
      v = __half2float(__ushort_as_half(dbits)) * static_cast<float>(static_cast<int8_t>(b[2 + c % 32]));
    }
    out[idx] = from_f32<OT>(v);
  }
}

template <typename OT>
cudaError_t LaunchEmbedT(const EmbedArgs& a, cudaStream_t s) {
  const unsigned row_smem = static_cast<unsigned>((a.row_bytes + 15) / 16 * 16);
  unsigned warps = kWarps;
  while (warps > 1 && static_cast<size_t>(warps) * row_smem > 48u * 1024u) warps >>= 1;
  if (a.vec && static_cast<size_t>(warps) * row_smem <= 48u * 1024u) {
    unsigned grid = (a.tokens + warps - 1) / warps;
    if (grid > 148u * 8u) grid = 148u * 8u;
    LaunchKernel(embed_q8_0_kernel<OT>, grid, kBlock, static_cast<size_t>(warps) * row_smem, s, a, warps, row_smem);
    return cudaGetLastError();
  }
  const size_t total = static_cast<size_t>(a.tokens) * a.cols;
  size_t grid = (total + kBlock - 1) / kBlock;
  if (grid > 148u * 32u) grid = 148u * 32u;
  LaunchKernel(embed_q8_0_scalar_kernel<OT>, static_cast<unsigned>(grid), kBlock, 0, s, a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t LaunchEmbedQ8_0(const EmbedArgs& a, cudaStream_t s) {
  if (a.tokens == 0 || a.cols == 0) return cudaSuccess;
  switch (a.out_dtype) {
    case kF32: return LaunchEmbedT<float>(a, s);
    case kF16: return LaunchEmbedT<f16>(a, s);
    case kBF16: return LaunchEmbedT<bf16>(a, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace halo_b200
