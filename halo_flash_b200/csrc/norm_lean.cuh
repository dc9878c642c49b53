// The lean row-norm kernels (dense rows, whole CTAs, nothing predicated) and their launchers, shared by norm.cu (one,
// two and four octets per thread) and norm_odd.cu (three and five): a header, so that the two sets of instantiations
// compile in parallel. See norm.cu for the layout.
#ifndef HALO_B200_NORM_LEAN_CUH_
#define HALO_B200_NORM_LEAN_CUH_

#include <type_traits>

#include "common.cuh"
#include "kernels.h"

#ifndef HALO_EPI_CTAS
#define HALO_EPI_CTAS 5
#endif

namespace halo_b200 {
namespace {

// Threads per row (g = 1 << lg), octets per thread (k) and rows per thread group (r).
struct Shape {
  unsigned lg;
  int k, r;
  unsigned rows_per_cta;
  bool full;
};

// The lean kernel for the common case: dense rows that fill the grid exactly (no predicates),
// one shared gamma row or none, output y and / or the Q8 epilogues, nothing else. It takes its
// few operands as plain arguments and carries no code for the rare features: the row kernels
// run CTAs that live for a microsecond, and both instruction count and code size showed up in
// their time (the general kernel above measured 13 % slower on the same rows).
struct LeanArgs {
  const void* x;
  const void* delta;
  void* res;
  const float* w;
  void* y;
  uint8_t* q8_0;
  int8_t* xq;
  float* xd;
  uint32_t d;
  float eps, inv_d;
  uint32_t lg;
  int one_plus, l2;
  int stage_q8;  // Q8_0 blocks leave through shared memory as 16-byte stores (see the kernel)
  int keep_res;  // store the residual with the L2 keep policy (it is small enough to stay there)
  uint32_t ahead;  // kernels without an epilogue: hint to L2 the rows of the CTA this many CTAs later (0 = none)
};

// WIDE: more than one warp per row (g > 32), the reduction crosses shared memory and a barrier.
// MODE: 0 = w, y, one_plus and l2 are tested at run time; 1 = RMSNorm with gamma w into y;
// 2 = the same with gamma 1 + w; 3 = L2 norm without gamma into y; with EPI, 4 = RMSNorm with gamma 1 + w into y and
// into staged Q8_0 blocks, 5 = the same without y, 6 / 7 = the same two with int8 codes + fp32 block scales instead of the
// Q8_0 blocks. The fixed modes exist because even warp-uniform tests
// cost these microsecond CTAs 3-4 % (12.6 vs 12.1 us on the add + norm of 4096 x 2048).
// Everything after the loads of one row per thread group: (add, store the sum,) sum of squares, scale, gamma,
// stores and Q8 epilogues. rx / rd hold the thread's K octets of x (and delta) as loaded; `row` is the group's row.
template <typename XT, typename YT, int K, bool ADD, bool EPI, bool WIDE, int MODE>
__device__ __forceinline__ void norm_lean_row(const LeanArgs& a, const Raw<XT> (&rx)[K], const Raw<XT> (&rd)[ADD ? K : 1],
                                              const uint32_t row, float* scratch, uint8_t (*stage)[EPI ? K : 1][EPI ? 272 : 16]) {
  const unsigned lg = a.lg, g = 1u << lg;
  const unsigned lir = threadIdx.x & (g - 1);
  const size_t off = static_cast<size_t>(row) * a.d;
  Oct v[K];
  if constexpr (ADD) {
    XT* res = static_cast<XT*>(a.res) + off;
    const uint64_t keep = l2_policy(a.keep_res != 0);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      // the norm reads the residual as stored; the next add + norm reads it again: ask L2 to keep it
      if constexpr (sizeof(XT) == 2) {  // summed in the storage type (raw_add: the same bits, a third of the instructions)
        const Raw<XT> sum = raw_add(rx[k], rd[k]);
        store16_keep(res + (((k << lg) + lir) << 3), sum.u, keep);
        v[k] = raw_unpack(sum);
      } else {
        v[k] = oct_add(raw_unpack(rx[k]), raw_unpack(rd[k]));
        oct_store_round_keep(res + (((k << lg) + lir) << 3), v[k], keep);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = raw_unpack(rx[k]);
  }
  constexpr bool kEpiQ8 = EPI && (MODE == 4 || MODE == 5);  // gamma 1 + w, staged Q8_0 blocks, no int8 copy; y in mode 4 only
  constexpr bool kEpiI8 = EPI && (MODE == 6 || MODE == 7);  // gamma 1 + w, int8 codes + fp32 scales, no Q8_0 blocks; y in mode 6 only
  constexpr bool kEpiFixed = kEpiQ8 || kEpiI8;
  constexpr bool kLateGamma = MODE == 1 || MODE == 2 || EPI;  // gamma fetched per octet after the reduction: fewer live registers
  Oct gm[K];
  if (!kLateGamma && MODE != 3 && (MODE != 0 || a.w)) {  // fetched before the reduction: the L2 round trip overlaps the shuffles / barrier
#pragma unroll
    for (int k = 0; k < K; ++k) {
      gm[k] = oct_load_cached(a.w + (((k << lg) + lir) << 3));
      if (MODE == 2 || (MODE == 0 && a.one_plus)) {
        const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) gm[k].p[i] = __fadd2_rn(one, gm[k].p[i]);
      }
    }
  }
  float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int k = 0; k < K; ++k) acc = oct_sumsq(v[k], acc);
  const float ss = WIDE ? group_sum(acc.x + acc.y, g, scratch) : group_sum_narrow(acc.x + acc.y, g);
  const float scale = (MODE == 3 || (MODE == 0 && a.l2)) ? rsqrtf(ss + a.eps) : rsqrtf(__fmaf_rn(ss, a.inv_d, a.eps));
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned j = (k << lg) + lir;
    v[k] = oct_scale(v[k], scale);
    if constexpr (kLateGamma) {
      if (MODE != 0 || a.w) {
        gm[k] = oct_load_cached(a.w + (j << 3));
        if (MODE == 2 || kEpiFixed || (MODE == 0 && a.one_plus)) {
          const float2 one = make_float2(1.0f, 1.0f);
#pragma unroll
          for (int i = 0; i < 4; ++i) gm[k].p[i] = __fadd2_rn(one, gm[k].p[i]);
        }
      }
    }
    if (MODE == 1 || MODE == 2 || kEpiFixed || (MODE == 0 && a.w)) v[k] = oct_mul(v[k], gm[k]);
    if ((MODE == 5 || MODE == 7) ? false : (MODE != 0 || a.y)) oct_store(static_cast<YT*>(a.y) + off + (j << 3), v[k]);
  }
  if constexpr (EPI) {
    // The K octets go through the epilogue phase by phase, not one after the other: their block maxima,
    // scale divisions and code roundings are independent of each other and interleave (3 % at T = 4096).
    float arr[K][8], amax[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      oct_to_array(v[k], arr[k]);
      amax[k] = amax8(arr[k]);
    }
#pragma unroll
    for (int k = 0; k < K; ++k) amax[k] = fmaxf(amax[k], __shfl_xor_sync(kFullMask, amax[k], 1));
#pragma unroll
    for (int k = 0; k < K; ++k) amax[k] = fmaxf(amax[k], __shfl_xor_sync(kFullMask, amax[k], 2));
    const unsigned lane = threadIdx.x & 31u;
    if (kEpiQ8 || (!kEpiI8 && a.q8_0)) {
      uint16_t dbits[K];
      uint2 codes[K];
#pragma unroll
      for (int k = 0; k < K; ++k) codes[k] = q8_0_codes(arr[k], amax[k], &dbits[k]);
      if (kEpiQ8 || a.stage_q8) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
          uint8_t* sb = stage[threadIdx.x >> 5][k] + (lane >> 2) * 34;
          if ((lane & 3u) == 0) *reinterpret_cast<uint16_t*>(sb) = dbits[k];
          store_codes_u16(sb + 2 + ((lane & 3u) << 3), codes[k]);
        }
        __syncwarp();
        if (lane < 17) {
#pragma unroll
          for (int k = 0; k < K; ++k) {
            const uint32_t c0 = ((k << lg) + lir) << 3;
            const size_t blk_index = static_cast<size_t>(row) * (a.d >> 5) + (c0 >> 5);
            uint8_t* out = a.q8_0 + (blk_index - (lane >> 2)) * 34;  // the warp's first block
            reinterpret_cast<uint4*>(out)[lane] = reinterpret_cast<const uint4*>(stage[threadIdx.x >> 5][k])[lane];
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const uint32_t c0 = ((k << lg) + lir) << 3;
          uint8_t* blk = a.q8_0 + (static_cast<size_t>(row) * (a.d >> 5) + (c0 >> 5)) * 34;
          if ((c0 & 31u) == 0) *reinterpret_cast<uint16_t*>(blk) = dbits[k];
          store_codes_u16(blk + 2 + (c0 & 31u), codes[k]);
        }
      }
    }
    if (kEpiI8 || (!kEpiQ8 && a.xq)) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const uint32_t c0 = ((k << lg) + lir) << 3;
        const float qs = div127(amax[k]);
        *reinterpret_cast<uint2*>(a.xq + off + c0) = i8_codes(arr[k], qs);
        if ((c0 & 31u) == 0) a.xd[static_cast<size_t>(row) * (a.d >> 5) + (c0 >> 5)] = qs;
      }
    }
  }
}

// HINTS (epilogue kernels only; the others follow HALO_PF_NORM / HALO_PF_AHEAD_NORM): compile the L2 hints in. The
// epilogue kernels exist with and without them, because a launch of a few rows (decode) gains nothing from a hint and
// pays for the preamble (319.8 -> 333.0 us per 230-launch decode step when every Q8_0 add + norm carried it).
template <typename XT, typename YT, int K, bool ADD, bool EPI, bool WIDE, int MODE, bool HINTS = false>
__global__ void __launch_bounds__(kBlock, K > 2 ? (sizeof(XT) == 2 ? (K == 5 ? 3 : 4) : 1) : (!EPI && MODE != 0 && sizeof(XT) == 2) ? 6 : (EPI && sizeof(XT) == 2) ? HALO_EPI_CTAS : 1) norm_rows_lean_kernel(const LeanArgs a) {
  pdl_trigger_early();
  if constexpr (EPI ? HINTS : HALO_PF_NORM != 0) {
    if (threadIdx.x == 0) {  // the CTA's rows are one contiguous span per tensor
      const size_t span = static_cast<size_t>(kBlock >> a.lg) * a.d;
      prefetch_l2_span(static_cast<const XT*>(a.x) + blockIdx.x * span, static_cast<unsigned>(span * sizeof(XT)));
      if constexpr (ADD)
        prefetch_l2_span(static_cast<const XT*>(a.delta) + blockIdx.x * span, static_cast<unsigned>(span * sizeof(XT)));
    }
  }
  pdl_wait_and_trigger();
  __shared__ float scratch[WIDE ? kBlock / 32 : 1];
  // Q8_0 staging: the 32 octets of a warp's slab are 8 blocks = 272 contiguous output bytes that
  // start on a 16-byte boundary (272 = 17 * 16), so the warp assembles them in shared memory
  // with 2-byte stores and 17 lanes write them out as 16-byte stores; the 2-byte global stores
  // this replaces cost 4-5 store instructions per thread, each touching 32 separate sectors.
  __shared__ __align__(16) uint8_t stage[EPI ? kBlock / 32 : 1][EPI ? K : 1][EPI ? 272 : 16];
  const unsigned lg = a.lg, g = 1u << lg;
  const unsigned lir = threadIdx.x & (g - 1);
  const uint32_t row = blockIdx.x * (kBlock >> lg) + (threadIdx.x >> lg);
  const size_t off = static_cast<size_t>(row) * a.d;
  const XT* x = static_cast<const XT*>(a.x) + off;
  Raw<XT> rx[K];
  Raw<XT> rd[ADD ? K : 1];
#pragma unroll
  for (int k = 0; k < K; ++k) rx[k] = raw_load(x + (((k << lg) + lir) << 3));
  if constexpr (ADD) {
    const XT* dl = static_cast<const XT*>(a.delta) + off;
#pragma unroll
    for (int k = 0; k < K; ++k) rd[k] = raw_load(dl + (((k << lg) + lir) << 3));
  }
  if constexpr (EPI ? HINTS : HALO_PF_AHEAD_NORM != 0) {
    if (threadIdx.x == 0 && a.ahead != 0 && blockIdx.x + a.ahead < gridDim.x) {
      const size_t span = static_cast<size_t>(kBlock >> lg) * a.d;
      prefetch_l2_span(static_cast<const XT*>(a.x) + (blockIdx.x + a.ahead) * span, static_cast<unsigned>(span * sizeof(XT)));
      if constexpr (ADD)
        prefetch_l2_span(static_cast<const XT*>(a.delta) + (blockIdx.x + a.ahead) * span, static_cast<unsigned>(span * sizeof(XT)));
    }
  }
  norm_lean_row<XT, YT, K, ADD, EPI, WIDE, MODE>(a, rx, rd, row, scratch, stage);
}

template <typename XT, typename YT, int K, bool ADD, bool WIDE>
void LaunchLeanMode(const LeanArgs& l, bool epi, int mode, unsigned grid, cudaStream_t s) {
  // the fixed epilogue modes on 16-bit rows carry the L2 hints in launches that give every SM a CTA and are short
  // enough for the look-ahead (beyond that the unhinted kernel measured 2 % faster: 154 against 157 us at 65 536 tokens)
  const bool hints = HALO_PF_NORM_EPI != 0 && sizeof(XT) == 2 && grid >= kSms && l.ahead != 0;
  if (epi && mode == 4 && hints) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 4, true>, grid, kBlock, 0, s, l);
  else if (epi && mode == 5 && hints) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 5, true>, grid, kBlock, 0, s, l);
  else if (epi && mode == 6 && hints) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 6, true>, grid, kBlock, 0, s, l);
  else if (epi && mode == 7 && hints) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 7, true>, grid, kBlock, 0, s, l);
  else if (epi && mode == 4) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 4>, grid, kBlock, 0, s, l);
  else if (epi && mode == 5) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 5>, grid, kBlock, 0, s, l);
  else if (epi && mode == 6) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 6>, grid, kBlock, 0, s, l);
  else if (epi && mode == 7) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 7>, grid, kBlock, 0, s, l);
  else if (epi) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, true, WIDE, 0>, grid, kBlock, 0, s, l);
  else if (mode == 2) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, false, WIDE, 2>, grid, kBlock, 0, s, l);
  else if (mode == 1) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, false, WIDE, 1>, grid, kBlock, 0, s, l);
  else if (mode == 3) LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, false, WIDE, 3>, grid, kBlock, 0, s, l);
  else LaunchKernel(norm_rows_lean_kernel<XT, YT, K, ADD, false, WIDE, 0>, grid, kBlock, 0, s, l);
}

template <typename XT, typename YT, int K, bool ADD>
cudaError_t LaunchLean(const NormArgs& a, const Shape& sh, unsigned grid, cudaStream_t s) {
  LeanArgs l;
  l.x = a.x;
  l.delta = a.delta;
  l.res = a.res;
  l.w = a.w;
  l.y = a.y;
  l.q8_0 = a.q8_0;
  l.xq = a.xq;
  l.xd = a.xd;
  l.d = a.d;
  l.eps = a.eps;
  l.inv_d = 1.0f / static_cast<float>(a.d);
  l.lg = sh.lg;
  l.one_plus = a.one_plus;
  l.l2 = a.l2;
  // The residual is asked to stay in L2 when it is small enough to survive there until the next add + norm:
  // 4096 x 2048 bf16 is 16.8 MB of the 126 MB. (Keeping the normalized rows as well measured no gain at 4096
  // tokens and cost 3 % at 65 536, where the two buffers are 537 MB.)
  l.keep_res = ADD && a.keep_hint && static_cast<size_t>(a.rows) * a.d * sizeof(XT) <= (40u << 20);
  // a warp's 32 octets must be consecutive in the output: rows of at least a warp, or one octet per thread
  l.stage_q8 = a.q8_0 && (reinterpret_cast<uintptr_t>(a.q8_0) & 15u) == 0 && (sh.lg >= 5 || K == 1);
  const bool epi = a.q8_0 || a.xq;
  // one wave of resident CTAs (the kernel's launch bounds), for launches short enough to run in step (see common.cuh)
  const unsigned wave = kSms * ((K > 2 || sizeof(XT) == 4) ? 4u : 6u);
  l.ahead = grid <= kAheadMaxWaves * wave ? wave : 0u;  // read by the kernels that carry the hints
  const int mode = (!epi && a.w && a.y && !a.l2)    ? (a.one_plus ? 2 : 1)
                   : (!epi && !a.w && a.y && a.l2) ? 3
                   : (epi && a.w && a.one_plus && !a.l2 && l.stage_q8 && !a.xq) ? (a.y ? 4 : 5)
                   : (epi && a.w && a.one_plus && !a.l2 && !a.q8_0 && a.xq)     ? (a.y ? 6 : 7)
                                                                                  : 0;
  if constexpr (K == 3 || K == 5) {  // rows of 3 g or 5 g octets, g >= 64 (PickOddShape): always wider than a warp
    LaunchLeanMode<XT, YT, K, ADD, true>(l, epi, mode, grid, s);
    return cudaGetLastError();
  }
  if constexpr (K <= 2) {  // rows wider than a warp per row exist only with one or two octets per thread
    if (sh.lg > 5) {
      LaunchLeanMode<XT, YT, K, ADD, true>(l, epi, mode, grid, s);
      return cudaGetLastError();
    }
  }
  LaunchLeanMode<XT, YT, K, ADD, false>(l, epi, mode, grid, s);
  return cudaGetLastError();
}

}  // namespace
}  // namespace halo_b200

#endif  // HALO_B200_NORM_LEAN_CUH_
