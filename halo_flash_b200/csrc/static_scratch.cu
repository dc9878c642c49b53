// halo_b200_norm_rope_qk_noalloc: fused Q/K per-head RMSNorm + RoPE for callers that cannot
// allocate device memory and have no spare buffer to lend.
//
// The fast form of the fused kernel reads cos / sin from a rotation table (one entry per token and
// frequency) that a small kernel fills first. halo_b200_rope_table_ex + halo_b200_norm_rope_qk_table_ex
// leave that table to the caller. This entry point keeps it instead in a fixed array inside the
// library, so the caller passes only its inputs and outputs and nothing is allocated, ever.
//
// Who needs that: an engine that committed all of its device memory up front (weights, KV pages
// mapped page by page, a scratch arena sized at load time) and accounts for every byte itself, as
// halo-flash does through rt::Device::Alloc / AvailableBytes; a serving loop where cudaMalloc's
// implicit device synchronisation would stall every session; a host that forbids allocation after
// start-up altogether. None of them can call cudaMalloc mid-step, and a library that did so behind
// their back would break their accounting or their latency.
//
// Costs and rules, all consequences of the array being one fixed, shared object:
//   * 4 MiB of device memory on every GPU that loads the library, held until the process exits.
//   * tokens * rotary_dim <= kMaxTableFloats, else the call fails with a message.
//   * The arguments are validated before anything is enqueued: a call that returns -1 has launched nothing and
//     has not touched the array. Shapes the table form cannot take (rows that are not 16-byte aligned, d or
//     rotary_dim / 2 not multiples of 8, no rotation at all) are forwarded to halo_b200_norm_rope_qk_ex, which
//     needs no table and allocates nothing either, so the accepted arguments are exactly that call's.
//   * The array keeps the previous call's table. Nothing in it has to start at zero - each call
//     overwrites every entry it later reads - but two calls whose kernels overlap on the GPU
//     (different streams, or the same graph launched twice concurrently) race on it. Calls on one
//     stream are ordered and safe.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current). Make that first call outside any stream capture.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/halo_b200.h"
#include "kernels.h"

namespace {

constexpr size_t kMaxTableFloats = size_t{1} << 20;  // 4 MiB: e.g. 16384 tokens at rotary_dim 64
constexpr int kMaxDevices = 64;

// The scratch itself. In host code this name is only a handle for the runtime, not an address a
// kernel could use: the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_rope_table_scratch[kMaxTableFloats];

std::mutex g_mutex;
float* g_device_address[kMaxDevices] = {};

int Fail(char* err, size_t errlen, const char* msg, const char* detail) {
  if (err && errlen) std::snprintf(err, errlen, "halo_norm_rope_qk_noalloc: %s%s", msg, detail ? detail : "");
  return -1;
}

// Device address of the scratch array on the current device (looked up once per device).
int ScratchAddress(float** out, char* err, size_t errlen) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return Fail(err, errlen, "cudaGetDevice: ", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return Fail(err, errlen, "device ordinal out of range", nullptr);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_device_address[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_rope_table_scratch);
    if (e != cudaSuccess) return Fail(err, errlen, "cudaGetSymbolAddress: ", cudaGetErrorString(e));
    if (p == nullptr) return Fail(err, errlen, "cudaGetSymbolAddress returned a null address", nullptr);
    g_device_address[dev] = static_cast<float*>(p);
  }
  *out = g_device_address[dev];
  return 0;
}

}  // namespace

extern "C" int halo_b200_norm_rope_qk_noalloc(halo_b200_stream stream, const void* q_in, uint64_t q_row_stride,
                                              void* q_out, void* q_gate, const float* w_q, uint32_t q_heads,
                                              const void* k_in, void* k_out, void* k_cache, const float* w_k,
                                              uint32_t k_heads, int in_dtype, int out_dtype, int one_plus, float eps,
                                              uint32_t d, uint32_t rotary_dim, uint32_t tokens, float theta,
                                              const uint32_t* params, uint32_t pstride, uint32_t slot, uint32_t pos0,
                                              uint32_t scale, uint32_t* pos_out, char* err, size_t errlen) {
  if (tokens == 0) {
    if (err && errlen) err[0] = '\0';
    return 0;
  }
  // Validate first: nothing may be enqueued (and the shared array must stay untouched) when the call fails.
  const int form = halo_b200::CheckNormRopeQk(q_in, q_row_stride, q_out, q_gate, w_q, q_heads, k_in, k_out, k_cache, w_k,
                                              k_heads, in_dtype, out_dtype, d, rotary_dim, tokens, theta, err, errlen);
  if (form < 0) return -1;
  if (form == 1 || rotary_dim < 2)  // no table can serve these rows: the table-free form (it allocates nothing either)
    return halo_b200_norm_rope_qk_ex(stream, q_in, q_row_stride, q_out, q_gate, w_q, q_heads, k_in, k_out, k_cache, w_k,
                                     k_heads, in_dtype, out_dtype, one_plus, eps, d, rotary_dim, tokens, theta, params,
                                     pstride, slot, pos0, scale, pos_out, err, errlen);
  if (static_cast<uint64_t>(tokens) * rotary_dim > kMaxTableFloats) {
    char detail[128];
    std::snprintf(detail, sizeof detail, " (tokens %u x rotary_dim %u; limit %zu floats)", tokens, rotary_dim,
                  kMaxTableFloats);
    return Fail(err, errlen, "rotation table exceeds the built-in scratch", detail);
  }
  float* table = nullptr;
  if (ScratchAddress(&table, err, errlen) != 0) return -1;
  // Both steps only enqueue kernels on `stream`: the table into the scratch, then the fused kernel
  // reading it. Stream order makes the second see the first.
  if (halo_b200_rope_table_ex(stream, table, tokens, rotary_dim, theta, params, pstride, slot, pos0, scale, pos_out,
                              err, errlen) != 0)
    return -1;
  return halo_b200_norm_rope_qk_table_ex(stream, q_in, q_row_stride, q_out, q_gate, w_q, q_heads, k_in, k_out, k_cache,
                                         w_k, k_heads, in_dtype, out_dtype, one_plus, eps, d, rotary_dim, tokens, table,
                                         err, errlen);
}
