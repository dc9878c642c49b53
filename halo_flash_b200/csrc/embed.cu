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

// A warp works on one SEGMENT of one row: 1 / segs of its blocks (a multiple of 8 blocks, so a multiple of
// 272 = 17 x 16 bytes: the segment starts 16-byte aligned in the table). segs is 1 for streaming sizes; when
// the launch cannot fill the GPU anyway it is raised (up to 8) so that a lane converts as few octets as
// possible: a lane's chain of dependent instructions is what such a launch lasts (8 octets per lane at
// 2048 columns and segs = 1, one at segs = 8).
template <typename OT>
__global__ void __launch_bounds__(kBlock) embed_q8_0_kernel(const EmbedArgs a, const unsigned warps,
                                                           const unsigned seg_smem, const unsigned segs) {
  pdl_begin();
  extern __shared__ __align__(16) uint8_t stage[];
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  if (warp >= warps) return;
  uint8_t* buf = stage + static_cast<size_t>(warp) * seg_smem;
  const unsigned seg_blocks = (a.cols / 32) / segs;
  const unsigned seg_bytes = seg_blocks * 34;
  const unsigned chunks = segs > 1 ? seg_bytes / 16 : static_cast<unsigned>(a.row_bytes / 16);
  const unsigned octs = seg_blocks * 4;
  OT* out = static_cast<OT*>(a.out);
  const uint32_t items = a.tokens * segs;
  for (uint32_t item = blockIdx.x * warps + warp; item < items; item += gridDim.x * warps) {
    const uint32_t t = item / segs, sg = item - t * segs;
    const uint32_t id = a.ids ? a.ids[static_cast<size_t>(t) * a.id_stride + a.id_slot] : a.token;
    const bool in_range = a.vocab == 0 || id < a.vocab;
    if (in_range) {
      const uint8_t* src = a.table + static_cast<size_t>(id) * a.row_bytes + static_cast<size_t>(sg) * seg_bytes;
      for (unsigned c = lane; c < chunks; c += 32) cp_async16(buf + c * 16, src + c * 16);
      cp_async_wait_all();
    }
    __syncwarp();
    OT* dst = out + static_cast<size_t>(t) * a.cols + static_cast<size_t>(sg) * seg_blocks * 32;
    if (!in_range) {
      const float z[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      for (unsigned j = lane; j < octs; j += 32) store8(dst + j * 8, z);
    } else {
      // A lane's octets j = lane, lane + 32, ... are eight blocks = 272 bytes apart, so its quarter of a block, the
      // alignment of its eight code bytes and therefore the funnel shift are the same for every one of them: they
      // are computed once and the loop only steps two pointers (the per-octet index arithmetic used to cost
      // more instructions than the conversion).
      const unsigned at0 = (lane >> 2) * 34u + 2u + 8u * (lane & 3u);
      const unsigned sh = (at0 & 2u) * 8u;
      const uint8_t* wp = buf + (at0 & ~3u);
      const uint8_t* dp = buf + (lane >> 2) * 34u;
      const float2 bias = make_float2(-8388736.0f, -8388736.0f);
      OT* o = dst + lane * 8;
      for (unsigned j = lane; j < octs; j += 32, wp += 272, dp += 272, o += 256) {
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(dp)));
        const float2 d2 = make_float2(d, d);
        // the 8 code bytes start 2 bytes into a block, so on a 4-byte boundary in odd blocks only: three
        // aligned words and a funnel shift by 0 or 16 bits give them as two words either way. The third word is
        // needed only for the shifted case, which never is the buffer's last block (a segment has a multiple of 8
        // blocks and odd blocks are aligned; a whole row of any other block count ends at least 2 bytes before
        // its 16-byte padded buffer does): reading it unconditionally ran 4 bytes past the last warp's buffer
        const uint32_t* w32 = reinterpret_cast<const uint32_t*>(wp);
        const uint32_t w0 = w32[0], w1 = w32[1], w2 = sh ? w32[2] : 0u;
        const uint32_t code[2] = {__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh)};
        // int8 -> float without a conversion instruction: the byte, biased by 128, becomes the low mantissa
        // byte of 2^23 (0x4B0000xx = 2^23 + xx); subtracting 2^23 + 128 leaves the code, exactly; then x scale
        float v[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t x = code[h] ^ 0x80808080u;
          const float2 lo = make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)),
                                        __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541)));
          const float2 hi = make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)),
                                        __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543)));
          const float2 a0 = __fmul2_rn(__fadd2_rn(lo, bias), d2), a1 = __fmul2_rn(__fadd2_rn(hi, bias), d2);
          v[4 * h] = a0.x, v[4 * h + 1] = a0.y, v[4 * h + 2] = a1.x, v[4 * h + 3] = a1.y;
        }
        store8(o, v);
      }
    }
    __syncwarp();  // the segment buffer is reused by the warp's next item
  }
}

// Rows whose byte length is a multiple of 8 (a multiple of four blocks) and whose octets divide evenly over a warp:
// straight from global memory into registers, no staging. A lane's octet j = lane + 32 i lies 34 (j / 4) + 2 +
// 8 (j % 4) bytes into the row; since 32 octets are eight blocks = 272 bytes, that offset is the lane's own constant
// plus 272 i, and so is its misalignment s in {0, 2, 4, 6} against 8 bytes. The lane reads the two aligned 8-byte words
// around its codes (the second only when s != 0; it then still lies inside the row, because a row's last block is
// 8-byte aligned when its length is), picks three of their four halves and funnel-shifts by 0 or 16 bits. Every load of
// the row - NPL x (two words + the 2-byte scale) per lane - is issued before the first conversion.
template <typename OT, int NPL>
__global__ void __launch_bounds__(kBlock) embed_q8_0_direct_kernel(const EmbedArgs a) {
  pdl_begin();
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const unsigned at0 = (lane >> 2) * 34u + 2u + 8u * (lane & 3u);  // the lane's first octet in the row
  const unsigned s = at0 & 7u;
  const unsigned sh = (s & 2u) * 8u;
  const bool high = s >= 4u;  // the codes start in the second half of the first word
  OT* out = static_cast<OT*>(a.out);
  const float2 bias = make_float2(-8388736.0f, -8388736.0f);
  for (uint32_t t = blockIdx.x * kWarps + warp; t < a.tokens; t += gridDim.x * kWarps) {
    const uint32_t id = a.ids ? a.ids[static_cast<size_t>(t) * a.id_stride + a.id_slot] : a.token;
    OT* o = out + static_cast<size_t>(t) * a.cols + lane * 8;
    if (a.vocab != 0 && id >= a.vocab) {
      const float z[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < NPL; ++i) store8(o + i * 256, z);
      continue;
    }
    const uint8_t* row = a.table + static_cast<size_t>(id) * a.row_bytes;
    const uint2* wp = reinterpret_cast<const uint2*>(row + (at0 & ~7u));
    const uint16_t* dp = reinterpret_cast<const uint16_t*>(row + (lane >> 2) * 34u);
    uint2 wa[NPL], wb[NPL];
    uint16_t db[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      wa[i] = wp[i * 34];  // 272 bytes on
      wb[i] = s ? wp[i * 34 + 1] : make_uint2(0u, 0u);
      db[i] = dp[i * 136];
    }
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const float d = __half2float(__ushort_as_half(db[i]));
      const float2 d2 = make_float2(d, d);
      const uint32_t w0 = high ? wa[i].y : wa[i].x, w1 = high ? wb[i].x : wa[i].y, w2 = high ? wb[i].y : wb[i].x;
      const uint32_t code[2] = {__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh)};
      // int8 -> float by the 2^23 mantissa trick (see the staged kernel), then x scale
      float v[8];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t x = code[h] ^ 0x80808080u;
        const float2 lo = make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)),
                                      __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541)));
        const float2 hi = make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)),
                                      __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543)));
        const float2 a0 = __fmul2_rn(__fadd2_rn(lo, bias), d2), a1 = __fmul2_rn(__fadd2_rn(hi, bias), d2);
        v[4 * h] = a0.x, v[4 * h + 1] = a0.y, v[4 * h + 2] = a1.x, v[4 * h + 3] = a1.y;
      }
      store8(o + i * 256, v);
    }
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
    // segments per row: as many (<= 8) as keep every warp busy once, whole groups of 8 blocks each
    const unsigned blocks = a.cols / 32;
    unsigned segs = 1;
    while (segs < 8 && blocks % (16 * segs) == 0 && static_cast<uint64_t>(a.tokens) * segs * 2 <= 148u * 64u) segs <<= 1;
    // whole rows of 8 NPL blocks, 8-byte aligned (the table is 16-byte aligned on this path), a row per warp and more
    // rows than resident warps: the direct kernel
    if (a.direct && segs == 1 && a.row_bytes == static_cast<uint64_t>(blocks) * 34 && blocks % 8 == 0) {
      unsigned dgrid = (a.tokens + kWarps - 1) / kWarps;
      if (dgrid > 148u * 8u) dgrid = 148u * 8u;
      switch (blocks / 8) {
        case 4: LaunchKernel(embed_q8_0_direct_kernel<OT, 4>, dgrid, kBlock, 0, s, a); return cudaGetLastError();
        case 8: LaunchKernel(embed_q8_0_direct_kernel<OT, 8>, dgrid, kBlock, 0, s, a); return cudaGetLastError();
        case 10: LaunchKernel(embed_q8_0_direct_kernel<OT, 10>, dgrid, kBlock, 0, s, a); return cudaGetLastError();
        default: break;
      }
    }
    unsigned grid = (a.tokens * segs + warps - 1) / warps;
    if (grid > 148u * 8u) grid = 148u * 8u;
    const unsigned seg_smem = segs > 1 ? (blocks / segs) * 34 : row_smem;
    LaunchKernel(embed_q8_0_kernel<OT>, grid, kBlock, static_cast<size_t>(warps) * seg_smem, s, a, warps, seg_smem, segs);
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
