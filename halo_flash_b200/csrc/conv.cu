// Causal depthwise conv (kernel 4) + SiLU + per-head L2 norm for sm_100a: the step of a Gated
// DeltaNet layer just before the q / k L2 norm, fused with it. Replaces halo_conv_step,
// halo_conv_l2norm, halo_conv_l2norm_prefill, halo_conv_l2norm_prefill8(_h, _hh) and
// halo_conv_state_advance(_h) (src/kernels/core.hip:445-456, 3002-3028, 3486-3611); arithmetic
// follows Qwen35Reference::Linear, src/model/qwen35.cpp:180-198.
//
// in, out are [tokens][channels]; channel ch of token t sees the inputs t-3 .. t, the ones before
// the chunk from the conv state [3][channels] (oldest first, fp32). The first l2_channels channels
// (q and k) are L2-normalized per head of d channels; the rest (v) are only convolved.
//
// A thread owns one octet of channels for kTile consecutive tokens: the window slides through its
// registers (kTile + 3 loads for kTile outputs; the 3 halo rows are the neighbour tile's own rows, so
// they come from L2), all loads are issued first, and a head of d channels is d / 8 neighbouring
// lanes, so each token's sum of squares is a shuffle reduction with no barrier.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "stage.cuh"

namespace halo_b200 {
namespace {

// Tokens per tile of the staged kernel and its resident CTAs per SM. 16-bit inputs: four tokens (two buffers of 7 rows =
// 56 KB) and three CTAs of 80 registers measured best - 31.2 us for 4096 tokens x 8192 channels against 32.4 with eight
// tokens and two CTAs of 128 registers (five tokens 31.6, six 34.8, four tokens with four CTAs of 64 registers 50.1:
// spills). fp32 inputs: eight tokens (176 KB) and one CTA; four tokens and two CTAs measured slower (53.8 against 49.1 us).
#ifndef HALO_CONV_TILE16
#define HALO_CONV_TILE16 4
#endif
#ifndef HALO_CONV_T4_CTAS
#define HALO_CONV_T4_CTAS 3
#endif
constexpr int kTaps = 4;

// acc = w[3] x[t]; acc += w[0] x[t-3]; += w[1] x[t-2]; += w[2] x[t-1] (the order of qwen35.cpp:183-186),
// each step one packed FMA. The step, prefill and scalar kernels all use this one recipe, so a token's
// output does not depend on how the chunk was tiled.
__device__ __forceinline__ Oct conv4(const Oct (&w)[kTaps], const Oct& x0, const Oct& x1, const Oct& x2, const Oct& x3) {
  Oct acc;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 v = __fmul2_rn(w[3].p[i], x3.p[i]);
    v = __ffma2_rn(w[0].p[i], x0.p[i], v);
    v = __ffma2_rn(w[1].p[i], x1.p[i], v);
    v = __ffma2_rn(w[2].p[i], x2.p[i], v);
    acc.p[i] = v;
  }
  return acc;
}

// HL: lanes per head (d / 8), a compile-time constant so that the shuffle steps carry no branch and the
// eight tokens' reductions, which are independent, interleave. FULL: the tile and its three rows of
// history lie inside the chunk and the thread owns a real octet, so nothing is predicated and the row
// addresses are one pointer stepped by `channels` (the predicated form spent more instructions on
// address arithmetic and guards than on the convolution).
template <typename IT, typename OT, unsigned HL, int kTile, bool FULL>
__device__ __forceinline__ void conv_tile(const ConvArgs& a, const unsigned c0, const uint32_t t0, const bool live) {
  const IT* in = static_cast<const IT*>(a.in);
  // window rows j = 0 .. kTile + 2 hold input t0 - 3 + j
  Raw<IT> raw[kTile + 3];
  if constexpr (FULL) {
    const IT* p = in + static_cast<size_t>(t0 - 3) * a.channels + c0;
#pragma unroll
    for (int j = 0; j < kTile + 3; ++j, p += a.channels) raw[j] = raw_load(p);
  } else {
#pragma unroll
    for (int j = 0; j < kTile + 3; ++j) {
      const int64_t i = static_cast<int64_t>(t0) - 3 + j;
      const bool from_chunk = live && i >= 0 && i < static_cast<int64_t>(a.tokens);
      if (from_chunk) raw[j] = raw_load(in + static_cast<size_t>(i) * a.channels + c0);
      else if constexpr (std::is_same_v<IT, float>) raw[j].a = raw[j].b = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      else raw[j].u = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  // taps: w[ch][4] -> four octets, tap k of the thread's 8 channels
  Oct w[kTaps];
  {
    float4 wl[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
      wl[c] = (FULL || live) ? __ldg(reinterpret_cast<const float4*>(a.w + static_cast<size_t>(c0 + c) * kTaps))
                             : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[0].p[i] = make_float2(wl[2 * i].x, wl[2 * i + 1].x);
      w[1].p[i] = make_float2(wl[2 * i].y, wl[2 * i + 1].y);
      w[2].p[i] = make_float2(wl[2 * i].z, wl[2 * i + 1].z);
      w[3].p[i] = make_float2(wl[2 * i].w, wl[2 * i + 1].w);
    }
  }
  // the three rows of history before the tile: from the chunk, or for the first tile from the conv state
  Oct x0 = raw_unpack(raw[0]), x1 = raw_unpack(raw[1]), x2 = raw_unpack(raw[2]);
  if constexpr (!FULL) {
    if (t0 == 0 && live && a.state) {
      x0 = oct_load(a.state + c0);
      x1 = oct_load(a.state + static_cast<size_t>(a.channels) + c0);
      x2 = oct_load(a.state + 2 * static_cast<size_t>(a.channels) + c0);
    }
  }
  const bool l2 = c0 < a.l2_channels;
  OT* out = static_cast<OT*>(a.out) + static_cast<size_t>(t0) * a.channels + c0;
#pragma unroll
  for (int t = 0; t < kTile; ++t, out += a.channels) {
    const Oct x3 = raw_unpack(raw[t + 3]);
    Oct v = conv4(w, x0, x1, x2, x3);
    x0 = x1, x1 = x2, x2 = x3;
#pragma unroll
    for (int i = 0; i < 4; ++i) v.p[i] = silu2_f(v.p[i]);
    if constexpr (HL > 0) {
      // all lanes shuffle (a warp may hold normalized and plain heads); only q / k lanes use the sum
      const float2 acc = oct_sumsq(v, make_float2(0.0f, 0.0f));
      float ss = acc.x + acc.y;
#pragma unroll
      for (unsigned of = 16; of > 0; of >>= 1)
        if (of < HL) ss += __shfl_xor_sync(kFullMask, ss, of);
      if (l2) v = oct_scale(v, rsqrtf(ss + a.eps));
    }
    if (FULL || (live && t0 + t < a.tokens)) oct_store(out, v);
  }
}

template <typename IT, typename OT, unsigned HL, int kTile>
__global__ void __launch_bounds__(kBlock, kTile >= 8 ? 2 : 3) conv_l2norm_kernel(const ConvArgs a) {
  pdl_begin();
  const unsigned oc = blockIdx.x * kBlock + threadIdx.x;  // channel octet
  const bool live = oc < (a.channels >> 3);
  const unsigned c0 = (live ? oc : 0u) << 3;
  const uint32_t t0 = blockIdx.y * kTile;
  // CTA-uniform except in the last CTA of a row of the grid; a warp there may run both forms in turn
  // (the shuffles of a head stay together: heads do not straddle the live / dead boundary)
  const bool full = t0 >= 3 && t0 + kTile <= a.tokens && (blockIdx.x + 1) * kBlock <= (a.channels >> 3);
  if (full) conv_tile<IT, OT, HL, kTile, true>(a, c0, t0, true);
  else conv_tile<IT, OT, HL, kTile, false>(a, c0, t0, live);
}

// ---- the same tile with its rows staged in shared memory by bulk asynchronous copies --------------
// The register form above holds its eleven input rows in registers to keep enough loads in flight
// (128 registers, 16 resident warps per SM) and then computes with nothing in flight: it measured
// 36 % issue-active. Here a CTA is persistent: it walks over tiles, and while it computes tile n out of
// one shared-memory buffer, the copy engine fills the other with tile n + 1 (cp.async.bulk, one 1-D copy
// of the CTA's channel slice per row, completion counted on an mbarrier per buffer). Bytes in flight
// cost no registers and the loads of the next tile overlap the arithmetic of this one.
//
// Every wait is bounded (stage.cuh): a CTA whose wait ran out counts it in g_stage_timeouts, gives the copies
// it has in flight one more bounded wait and all of its threads return together without writing further
// tiles. Rows outside the chunk are not copied; their lanes read zeros (or the conv state).
__device__ unsigned int g_stage_timeouts = 0;

// MODE 0: per-thread q/k test, 1: all q/k, 2: none. FULL: the tile and its three rows of history lie inside the
// chunk and every thread owns a real octet, so no load or store is predicated and the eight tokens form ONE
// straight-line block: their convolutions, gates and head reductions are independent and the compiler
// interleaves them (with the bounds tests in the loop each token was a block of its own, and a warp issued
// once in fifteen cycles, stalled on its own dependent chain).
template <typename IT, typename OT, unsigned HL, int kTile, int MODE, bool FULL>
__device__ __forceinline__ void conv_stage_compute(const ConvArgs& a, const Oct (&w)[kTaps], const IT* tile,
                                                   const unsigned row_elems, const unsigned c0, const uint32_t t0,
                                                   const bool live, const uint32_t first_row, const uint32_t last_row) {
  const IT* mine = tile + threadIdx.x * 8;
  // window row j holds input t0 - 3 + j; rows [first_row, last_row) were copied, the rest read as zero
  auto row = [&](int j) -> Oct {
    if (FULL || (static_cast<uint32_t>(j) >= first_row && static_cast<uint32_t>(j) < last_row)) {
      if constexpr (std::is_same_v<IT, float>) {
        const float4 lo = *reinterpret_cast<const float4*>(mine + static_cast<size_t>(j) * row_elems);
        const float4 hi = *reinterpret_cast<const float4*>(mine + static_cast<size_t>(j) * row_elems + 4);
        Oct o;
        o.p[0] = make_float2(lo.x, lo.y), o.p[1] = make_float2(lo.z, lo.w);
        o.p[2] = make_float2(hi.x, hi.y), o.p[3] = make_float2(hi.z, hi.w);
        return o;
      } else {
        const uint4 u = *reinterpret_cast<const uint4*>(mine + static_cast<size_t>(j) * row_elems);
        if constexpr (std::is_same_v<IT, bf16>) return oct_unpack_bf16(u);
        else return oct_unpack_f16(u);
      }
    }
    return oct_zero();
  };
  Oct x0 = row(0), x1 = row(1), x2 = row(2);
  if (!FULL && t0 == 0 && live && a.state) {
    x0 = oct_load(a.state + c0);
    x1 = oct_load(a.state + static_cast<size_t>(a.channels) + c0);
    x2 = oct_load(a.state + 2 * static_cast<size_t>(a.channels) + c0);
  }
  const bool l2 = MODE == 1 || (MODE == 0 && c0 < a.l2_channels);
  OT* out = static_cast<OT*>(a.out) + static_cast<size_t>(t0) * a.channels + c0;
#pragma unroll
  for (int t = 0; t < kTile; ++t, out += a.channels) {
    const Oct x3 = row(t + 3);
    Oct v = conv4(w, x0, x1, x2, x3);
    x0 = x1, x1 = x2, x2 = x3;
#pragma unroll
    for (int i = 0; i < 4; ++i) v.p[i] = silu2_f(v.p[i]);
    if constexpr (MODE != 2 && HL > 0) {
      const float2 acc = oct_sumsq(v, make_float2(0.0f, 0.0f));
      float ss = acc.x + acc.y;
#pragma unroll
      for (unsigned of = 16; of > 0; of >>= 1)
        if (of < HL) ss += __shfl_xor_sync(kFullMask, ss, of);
      if (l2) v = oct_scale(v, rsqrtf(ss + a.eps));
    }
    if (FULL || (live && t0 + t < a.tokens)) oct_store(out, v);
  }
}

// Rows of tile (slice, by) wanted by the window: [first_row, last_row) of the kTile + 3 window rows.
template <int kTile>
__device__ __forceinline__ void tile_rows(uint32_t t0, uint32_t tokens, uint32_t* first_row, uint32_t* last_row) {
  *first_row = t0 >= 3 ? 0u : 3u - t0;
  const uint32_t avail = tokens + 3u - t0;  // window rows before the chunk's end
  *last_row = avail < static_cast<uint32_t>(kTile + 3) ? avail : static_cast<uint32_t>(kTile + 3);
}

// grid.x = a multiple of `slices` (CTA c always works on channel slice c % slices, so its taps are loaded
// once); CTA c takes the token tiles c / slices, c / slices + grid.x / slices, ...
template <typename IT, typename OT, unsigned HL, int kTile>
__global__ void __launch_bounds__(kBlock, (kTile < 8 && sizeof(IT) == 2) ? HALO_CONV_T4_CTAS : 2) conv_l2norm_staged_kernel(const ConvArgs a, const uint32_t slices,
                                                                    const uint32_t token_tiles) {
  pdl_launch_dependents();  // persistent and GPU-filling whatever its grid: the successor may be scheduled at once
  extern __shared__ __align__(128) uint8_t conv_smem[];
  __shared__ __align__(8) unsigned long long bars[2];
  const unsigned octs = a.channels >> 3;
  const uint32_t slice = blockIdx.x % slices, lane_of_slice = blockIdx.x / slices, stride = gridDim.x / slices;
  const unsigned oc0 = slice * kBlock;                           // first channel octet of the CTA's slice
  const unsigned slice_octs = min(static_cast<unsigned>(kBlock), octs - oc0);
  constexpr unsigned row_elems = kBlock * 8;                     // elements between two staged rows
  constexpr unsigned buf_elems = (kTile + 3) * row_elems;
  const bool live = threadIdx.x < slice_octs;
  const unsigned c0 = (oc0 + (live ? threadIdx.x : 0u)) << 3;
  IT* bufs = reinterpret_cast<IT*>(conv_smem);
  const unsigned row_bytes = slice_octs * 8u * static_cast<unsigned>(sizeof(IT));  // a multiple of 16

  uint32_t by = lane_of_slice;
  // before the wait for the kernel ahead: the barriers, and a hint to L2 for the rows of the CTA's first tile
  if (threadIdx.x == 0) stage_init(bars, 2);
  if (HALO_PF_CONV != 0 && by < token_tiles) {
    uint32_t first_row, last_row;
    tile_rows<kTile>(by * kTile, a.tokens, &first_row, &last_row);
    if (threadIdx.x < last_row - first_row)
      prefetch_l2_span(static_cast<const IT*>(a.in) + static_cast<size_t>(by * kTile + first_row + threadIdx.x - 3u) * a.channels +
                           (static_cast<size_t>(oc0) << 3), row_bytes);
  }
  pdl_wait_and_trigger();
  __syncthreads();

  // thread 0 asks the copy engine for the rows of token tile `by` into buffer `b`
  auto request = [&](uint32_t by, unsigned b) {
    uint32_t first_row, last_row;
    tile_rows<kTile>(by * kTile, a.tokens, &first_row, &last_row);
    const unsigned bar = smem_addr(&bars[b]);
    stage_expect(bar, (last_row - first_row) * row_bytes);
    const IT* src = static_cast<const IT*>(a.in) + static_cast<size_t>(by * kTile + first_row - 3u) * a.channels +
                    (static_cast<size_t>(oc0) << 3);
    unsigned dst = smem_addr(bufs + b * buf_elems + first_row * row_elems);
    for (uint32_t j = first_row; j < last_row; ++j, src += a.channels, dst += row_elems * sizeof(IT))
      stage_copy(dst, src, row_bytes, bar);
  };

  if (by >= token_tiles) return;  // uniform: the whole CTA has no tile
  if (threadIdx.x == 0) request(by, 0);

  // taps: w[ch][4] -> four octets, tap k of the thread's 8 channels; loaded once, while the first tile arrives
  Oct w[kTaps];
  {
    float4 wl[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
      wl[c] = live ? __ldg(reinterpret_cast<const float4*>(a.w + static_cast<size_t>(c0 + c) * kTaps))
                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[0].p[i] = make_float2(wl[2 * i].x, wl[2 * i + 1].x);
      w[1].p[i] = make_float2(wl[2 * i].y, wl[2 * i + 1].y);
      w[2].p[i] = make_float2(wl[2 * i].z, wl[2 * i + 1].z);
      w[3].p[i] = make_float2(wl[2 * i].w, wl[2 * i + 1].w);
    }
  }
  const unsigned slice_lo = oc0 << 3, slice_hi = (oc0 + slice_octs) << 3;
  const int mode = (HL == 0 || slice_lo >= a.l2_channels) ? 2 : (slice_hi <= a.l2_channels ? 1 : 0);

  for (uint32_t n = 0; by < token_tiles; ++n, by += stride) {
    const unsigned b = n & 1u;
    // the other buffer was last read in iteration n - 1, which ended with a CTA barrier: refill it now
    if (threadIdx.x == 0 && by + stride < token_tiles) request(by + stride, b ^ 1u);
    // wait for this buffer's bytes: its (n / 2)-th use, so phase parity (n / 2) & 1; bounded (see stage_wait)
    const bool prefetched = by + stride < token_tiles;
    const unsigned done = stage_wait(smem_addr(&bars[b]), (n >> 1) & 1u);
    if (!__syncthreads_and(static_cast<int>(done))) {
      // Never seen. All threads leave together, and nothing more is requested; but the CTA must not hand its shared
      // memory back while a copy into it may still be in flight, so this buffer and the prefetch issued above (the
      // other buffer's ((n + 1) / 2)-th use) each get one more bounded wait first. The output tiles this CTA still
      // owned stay unwritten: the counter is how the host learns that the call's results are invalid.
      stage_wait(smem_addr(&bars[b]), (n >> 1) & 1u);
      if (prefetched) stage_wait(smem_addr(&bars[b ^ 1u]), ((n + 1) >> 1) & 1u);
      if (threadIdx.x == 0) atomicAdd(&g_stage_timeouts, 1u);
      return;
    }
    uint32_t first_row, last_row;
    tile_rows<kTile>(by * kTile, a.tokens, &first_row, &last_row);
    const IT* tile = bufs + b * buf_elems;
    const bool full = first_row == 0 && last_row == static_cast<uint32_t>(kTile + 3) && slice_octs == kBlock &&
                      by * kTile + kTile <= a.tokens;  // uniform over the CTA
    if (full) {
      if (mode == 2) conv_stage_compute<IT, OT, HL, kTile, 2, true>(a, w, tile, row_elems, c0, by * kTile, live, first_row, last_row);
      else if (mode == 1) conv_stage_compute<IT, OT, HL, kTile, 1, true>(a, w, tile, row_elems, c0, by * kTile, live, first_row, last_row);
      else conv_stage_compute<IT, OT, HL, kTile, 0, true>(a, w, tile, row_elems, c0, by * kTile, live, first_row, last_row);
    } else {
      if (mode == 2) conv_stage_compute<IT, OT, HL, kTile, 2, false>(a, w, tile, row_elems, c0, by * kTile, live, first_row, last_row);
      else if (mode == 1) conv_stage_compute<IT, OT, HL, kTile, 1, false>(a, w, tile, row_elems, c0, by * kTile, live, first_row, last_row);
      else conv_stage_compute<IT, OT, HL, kTile, 0, false>(a, w, tile, row_elems, c0, by * kTile, live, first_row, last_row);
    }
    __syncthreads();  // every thread is done reading this buffer before it is refilled
  }
}

// Any kernel length, head size and alignment: one CTA per (head, token), one channel per thread.
template <typename IT, typename OT>
__global__ void __launch_bounds__(1024) conv_l2norm_scalar_kernel(const ConvArgs a) {
  pdl_begin();
  __shared__ float scratch[32];
  __shared__ float total;
  const uint32_t t = blockIdx.y;
  const uint32_t ch = blockIdx.x * a.d + threadIdx.x;
  const bool live = threadIdx.x < a.d && ch < a.channels;
  const IT* in = static_cast<const IT*>(a.in);
  float v = 0.0f;
  if (live) {
    const float* w = a.w + static_cast<size_t>(ch) * a.kern;
    float acc = __fmul_rn(w[a.kern - 1], to_f32(in[static_cast<size_t>(t) * a.channels + ch]));
    for (uint32_t k = 0; k + 1 < a.kern; ++k) {
      const int64_t i = static_cast<int64_t>(t) - static_cast<int64_t>(a.kern - 1) + k;  // window slot k
      float x = 0.0f;
      if (i >= 0) x = to_f32(in[static_cast<size_t>(i) * a.channels + ch]);
      else if (a.state) x = a.state[static_cast<size_t>(i + a.kern - 1) * a.channels + ch];
      acc = __fmaf_rn(w[k], x, acc);
    }
    v = silu_f(acc);
  }
  if (blockIdx.x * a.d < a.l2_channels) {  // CTA-uniform
    float ss = warp_sum(live ? __fmul_rn(v, v) : 0.0f);
    if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.0f;
      for (unsigned i = 0; i < (blockDim.x + 31) / 32; ++i) s += scratch[i];
      total = s;
    }
    __syncthreads();
    v *= rsqrtf(total + a.eps);
  }
  if (live) static_cast<OT*>(a.out)[static_cast<size_t>(t) * a.channels + ch] = from_f32<OT>(v);
}

// One decode step of `entries` sessions (src/kernels/core.hip:3005-3028, src/kernels/batch_decode.hip:1741-1748):
// the conv over the session's state and its new input, the state shifted by one with the input appended, SiLU,
// and the L2 norm of the q/k heads, in one launch. One CTA per (head, entry), one channel per thread: a thread
// reads its own state column before it writes it, so nothing else orders the update.
template <typename IT, typename OT>
__global__ void __launch_bounds__(1024) conv_step_kernel(const ConvArgs a) {
  pdl_begin();
  __shared__ float scratch[32];
  __shared__ float total;
  const uint32_t e = blockIdx.y;
  const uint32_t ch = blockIdx.x * a.d + threadIdx.x;
  const bool live = threadIdx.x < a.d && ch < a.channels;
  const IT* in = static_cast<const IT*>(a.in) + static_cast<size_t>(e) * a.entry_stride;
  OT* out = static_cast<OT*>(a.out) + static_cast<size_t>(e) * a.entry_stride;
  float* state = a.state_tab ? reinterpret_cast<float*>(a.state_tab[static_cast<size_t>(e) * a.tstride + a.tslot]) : a.state;
  float v = 0.0f;
  if (live) {
    const float* w = a.w + static_cast<size_t>(ch) * a.kern;
    const float x = to_f32(in[ch]);
    float acc = __fmul_rn(w[a.kern - 1], x);
    float older[8];  // kern <= 9
#pragma unroll
    for (uint32_t k = 0; k < 8; ++k)
      if (k + 1 < a.kern) {
        older[k] = state[static_cast<size_t>(k) * a.channels + ch];
        acc = __fmaf_rn(w[k], older[k], acc);
      }
#pragma unroll
    for (uint32_t k = 0; k < 7; ++k)
      if (k + 2 < a.kern) state[static_cast<size_t>(k) * a.channels + ch] = older[k + 1];
    if (a.kern > 1) state[static_cast<size_t>(a.kern - 2) * a.channels + ch] = x;
    v = silu_f(acc);
  }
  if (blockIdx.x * a.d < a.l2_channels) {  // CTA-uniform
    const float ss = warp_sum(live ? __fmul_rn(v, v) : 0.0f);
    if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.0f;
      for (unsigned i = 0; i < (blockDim.x + 31) / 32; ++i) s += scratch[i];
      total = s;
    }
    __syncthreads();
    v *= rsqrtf(total + a.eps);
  }
  if (live) out[ch] = from_f32<OT>(v);
}

// The conv state after a chunk: the last kern - 1 inputs, the older ones from the previous state when
// the chunk is shorter than that (src/kernels/core.hip:3578-3611). One thread per channel.
template <typename IT>
__global__ void __launch_bounds__(kBlock) conv_state_advance_kernel(const ConvArgs a) {
  pdl_begin();
  const uint32_t ch = blockIdx.x * kBlock + threadIdx.x;
  if (ch >= a.channels || a.kern < 2) return;
  const IT* in = static_cast<const IT*>(a.in);
  float next[8];  // kern <= 9: every row is read before any is written
  for (uint32_t k = 0; k + 1 < a.kern; ++k) {
    const int64_t i = static_cast<int64_t>(a.tokens) - static_cast<int64_t>(a.kern - 1) + k;
    next[k] = i >= 0 ? to_f32(in[static_cast<size_t>(i) * a.channels + ch])
                     : a.state[static_cast<size_t>(i + a.kern - 1) * a.channels + ch];
  }
  for (uint32_t k = 0; k + 1 < a.kern; ++k) a.state[static_cast<size_t>(k) * a.channels + ch] = next[k];
}

template <typename IT, typename OT, int TILE>
cudaError_t LaunchConvTile(const ConvArgs& a, unsigned head_octs, cudaStream_t s) {
  const dim3 grid((a.channels / 8 + kBlock - 1) / kBlock, (a.tokens + TILE - 1) / TILE);
  if (grid.y > 65535u) return cudaErrorInvalidValue;
  switch (a.l2_channels ? head_octs : 0u) {
    case 0: return LaunchKernel(conv_l2norm_kernel<IT, OT, 0, TILE>, grid, kBlock, 0, s, a);
    case 1: return LaunchKernel(conv_l2norm_kernel<IT, OT, 1, TILE>, grid, kBlock, 0, s, a);
    case 2: return LaunchKernel(conv_l2norm_kernel<IT, OT, 2, TILE>, grid, kBlock, 0, s, a);
    case 4: return LaunchKernel(conv_l2norm_kernel<IT, OT, 4, TILE>, grid, kBlock, 0, s, a);
    case 8: return LaunchKernel(conv_l2norm_kernel<IT, OT, 8, TILE>, grid, kBlock, 0, s, a);
    case 16: return LaunchKernel(conv_l2norm_kernel<IT, OT, 16, TILE>, grid, kBlock, 0, s, a);
    default: return LaunchKernel(conv_l2norm_kernel<IT, OT, 32, TILE>, grid, kBlock, 0, s, a);
  }
}

template <typename IT, typename OT, unsigned HL>
cudaError_t LaunchConvStagedHL(const ConvArgs& a, unsigned grid, uint32_t slices, uint32_t token_tiles, size_t smem,
                               cudaStream_t s) {
  auto kernel = conv_l2norm_staged_kernel<IT, OT, HL, (sizeof(IT) == 2 ? HALO_CONV_TILE16 : 8)>;
  // more than 48 KB of dynamic shared memory has to be asked for
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  return LaunchKernel(kernel, grid, kBlock, smem, s, a, slices, token_tiles);
}

// Persistent CTAs, three per SM for 16-bit inputs (the two four-token tile buffers of a CTA take 56 KB) and one for
// fp32 (eight-token buffers, 176 KB), rounded to a multiple of the number of channel slices.
template <typename IT, typename OT>
cudaError_t LaunchConvStaged(const ConvArgs& a, unsigned head_octs, cudaStream_t s) {
  constexpr unsigned kT = sizeof(IT) == 2 ? HALO_CONV_TILE16 : 8;
  const uint32_t slices = (a.channels / 8 + kBlock - 1) / kBlock, token_tiles = (a.tokens + kT - 1) / kT;
  const size_t smem = 2 * static_cast<size_t>(kT + 3) * kBlock * 8 * sizeof(IT);
  const unsigned resident = 148u * (sizeof(IT) == 2 ? (kT < 8 ? HALO_CONV_T4_CTAS : 2u) : 1u);
  if (slices > resident) return cudaErrorNotSupported;  // wider than the persistent grid: the register form runs
  unsigned per_slice = resident / slices;
  if (per_slice > token_tiles) per_slice = token_tiles;
  const unsigned grid = per_slice * slices;
  switch (a.l2_channels ? head_octs : 0u) {
    case 0: return LaunchConvStagedHL<IT, OT, 0>(a, grid, slices, token_tiles, smem, s);
    case 1: return LaunchConvStagedHL<IT, OT, 1>(a, grid, slices, token_tiles, smem, s);
    case 2: return LaunchConvStagedHL<IT, OT, 2>(a, grid, slices, token_tiles, smem, s);
    case 4: return LaunchConvStagedHL<IT, OT, 4>(a, grid, slices, token_tiles, smem, s);
    case 8: return LaunchConvStagedHL<IT, OT, 8>(a, grid, slices, token_tiles, smem, s);
    case 16: return LaunchConvStagedHL<IT, OT, 16>(a, grid, slices, token_tiles, smem, s);
    default: return LaunchConvStagedHL<IT, OT, 32>(a, grid, slices, token_tiles, smem, s);
  }
}

template <typename IT, typename OT>
cudaError_t LaunchConvT(const ConvArgs& a, cudaStream_t s) {
  const unsigned head_octs = a.d / 8;
  const bool head_pow2 = head_octs >= 1 && head_octs <= 32 && (head_octs & (head_octs - 1)) == 0 && a.d % 8 == 0;
  if (a.vec && a.kern == kTaps && (a.l2_channels == 0 || head_pow2)) {
    if (a.staged) {
      const cudaError_t e = LaunchConvStaged<IT, OT>(a, head_octs, s);
      if (e != cudaErrorNotSupported) return e;
    }
    return a.tile == 4 ? LaunchConvTile<IT, OT, 4>(a, head_octs, s) : LaunchConvTile<IT, OT, 8>(a, head_octs, s);
  }
  if (a.d == 0 || a.d > 1024 || a.tokens > 65535u) return cudaErrorInvalidValue;
  const dim3 grid((a.channels + a.d - 1) / a.d, a.tokens);
  return LaunchKernel(conv_l2norm_scalar_kernel<IT, OT>, grid, dim3((a.d + 31) / 32 * 32), 0, s, a);
}

}  // namespace

cudaError_t LaunchConvL2norm(const ConvArgs& a, cudaStream_t s) {
  if (a.tokens == 0 || a.channels == 0) return cudaSuccess;
  const int i = a.in_dtype, o = a.out_dtype;
  if (i == kF32 && o == kF32) return LaunchConvT<float, float>(a, s);
  if (i == kF16 && o == kF32) return LaunchConvT<f16, float>(a, s);
  if (i == kF16 && o == kF16) return LaunchConvT<f16, f16>(a, s);
  if (i == kBF16 && o == kBF16) return LaunchConvT<bf16, bf16>(a, s);
  if (i == kBF16 && o == kF32) return LaunchConvT<bf16, float>(a, s);
  return cudaErrorInvalidValue;
}

template <typename IT, typename OT>
cudaError_t LaunchConvStepT(const ConvArgs& a, cudaStream_t s) {
  const dim3 grid((a.channels + a.d - 1) / a.d, a.entries);
  return LaunchKernel(conv_step_kernel<IT, OT>, grid, dim3((a.d + 31) / 32 * 32), 0, s, a);
}

cudaError_t LaunchConvStep(const ConvArgs& a, cudaStream_t s) {
  if (a.entries == 0 || a.channels == 0) return cudaSuccess;
  if (a.d == 0 || a.d > 1024 || a.entries > 65535u || a.kern < 1 || a.kern > 9) return cudaErrorInvalidValue;
  const int i = a.in_dtype, o = a.out_dtype;
  if (i == kF32 && o == kF32) return LaunchConvStepT<float, float>(a, s);
  if (i == kF16 && o == kF32) return LaunchConvStepT<f16, float>(a, s);
  if (i == kF16 && o == kF16) return LaunchConvStepT<f16, f16>(a, s);
  if (i == kBF16 && o == kBF16) return LaunchConvStepT<bf16, bf16>(a, s);
  if (i == kBF16 && o == kF32) return LaunchConvStepT<bf16, float>(a, s);
  return cudaErrorInvalidValue;
}

cudaError_t ReadConvStageTimeouts(unsigned int* out) {
  return cudaMemcpyFromSymbol(out, g_stage_timeouts, sizeof(unsigned int));
}

cudaError_t LaunchConvStateAdvance(const ConvArgs& a, cudaStream_t s) {
  if (a.channels == 0 || a.kern < 2) return cudaSuccess;
  const unsigned grid = (a.channels + kBlock - 1) / kBlock;
  switch (a.in_dtype) {
    case kF32: return LaunchKernel(conv_state_advance_kernel<float>, grid, kBlock, 0, s, a);
    case kF16: return LaunchKernel(conv_state_advance_kernel<f16>, grid, kBlock, 0, s, a);
    case kBF16: return LaunchKernel(conv_state_advance_kernel<bf16>, grid, kBlock, 0, s, a);
  }
  return cudaErrorInvalidValue;
}

}  // namespace halo_b200
