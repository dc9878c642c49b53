// Drives the sm_100a replacement kernels through halo-flash's own device interface (halo::rt::Device,
// src/rt/device.hpp) and checks them against halo-flash's own CPU operators, the way the reference's
// kernel tests do (tests/gpu/quant_gpu_test.cpp): LCG-seeded inputs, Upload, Kernel(name) + Launch with
// the reference kernel's grid, block and argument list, Download, compare. Built only where the
// reference checkout is present (its headers and CPU sources are compiled from where they lie).
//
// Prints one line per check and exits non-zero on the first failure.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <span>
#include <string>
#include <vector>

#include "core/lowbit.hpp"
#include "model/cpu_ops.hpp"
#include "model/weights.hpp"
#include "rt/device.hpp"

#include "cuda_device.hpp"

namespace rt = halo::rt;
namespace cpu = halo::model::cpu;

namespace {

int g_failures = 0;

void Report(const char* what, bool ok, const std::string& detail = "") {
  std::printf("%s %s%s%s\n", ok ? "PASS" : "FAIL", what, detail.empty() ? "" : ": ", detail.c_str());
  if (!ok) ++g_failures;
}

std::uint32_t g_seed = 12345;
std::vector<float> Lcg(std::size_t n, float amp) {  // tests/gpu/quant_gpu_test.cpp:2373-2377
  std::vector<float> v(n);
  for (auto& x : v) {
    g_seed = g_seed * 1664525u + 1013904223u;
    x = amp * (static_cast<float>(g_seed >> 8) / 16777216.0f - 0.5f);
  }
  return v;
}

// |got - want| <= 1e-5 * max(|want|, rms(want row)) on rows of d values
bool RowsClose(const std::vector<float>& got, const std::vector<float>& want, std::size_t d, std::string* detail) {
  for (std::size_t r = 0; r * d < want.size(); ++r) {
    double ss = 0;
    for (std::size_t i = 0; i < d; ++i) ss += static_cast<double>(want[r * d + i]) * want[r * d + i];
    const float rms = static_cast<float>(std::sqrt(ss / static_cast<double>(d)));
    for (std::size_t i = 0; i < d; ++i) {
      const float w = want[r * d + i], g = got[r * d + i];
      if (!(std::fabs(g - w) <= 1e-5f * std::fmax(std::fabs(w), rms) + 1e-30f)) {
        *detail = "row " + std::to_string(r) + " col " + std::to_string(i) + ": got " + std::to_string(g) + " want " +
                  std::to_string(w);
        return false;
      }
    }
  }
  return true;
}

struct Dev {
  rt::Device* d;
  std::string err;
  rt::Buffer Up(const void* p, std::size_t bytes) {
    rt::Buffer b = d->Alloc(bytes, &err);
    if (!b || !d->Upload(b, 0, p, bytes, &err)) {
      std::printf("FAIL upload: %s\n", err.c_str());
      std::exit(2);
    }
    return b;
  }
  template <typename T>
  rt::Buffer Up(const std::vector<T>& v) { return Up(v.data(), v.size() * sizeof(T)); }
  template <typename T>
  std::vector<T> Down(const rt::Buffer& b, std::size_t n) {
    std::vector<T> v(n);
    if (!d->Download(b, 0, v.data(), n * sizeof(T), &err)) {
      std::printf("FAIL download: %s\n", err.c_str());
      std::exit(2);
    }
    return v;
  }
  bool Launch(const char* name, rt::Dim3 grid, rt::Dim3 block, std::vector<rt::Arg> args) {
    const rt::KernelId k = d->Kernel(name, &err);
    return k >= 0 && d->Launch(k, grid, block, args, &err);
  }
};

void CheckGroupedNormRows(Dev& dv) {
  const std::uint32_t T = 6, hc = 4, d = 320;
  auto x = Lcg(T * hc * d, 6.0f), w = Lcg(hc * d, 2.0f);
  rt::Buffer bx = dv.Up(x), bw = dv.Up(w), by = dv.d->Alloc(x.size() * 4, &dv.err);
  const bool ok = dv.Launch("halo_rmsnorm_rows", {T * hc}, {256},
                            {rt::Arg::Buf(bx), rt::Arg::Buf(bw), rt::Arg::Buf(by), rt::Arg::Val(d), rt::Arg::Val(1e-6f),
                             rt::Arg::Val(d), rt::Arg::Val(hc)});
  std::vector<float> want = x;
  for (std::uint32_t r = 0; r < T * hc; ++r) cpu::RmsNorm(std::span<float>(want.data() + r * d, d), w.data() + (r % hc) * d, 1e-6f);
  std::string detail = dv.err;
  Report("halo_rmsnorm_rows through rt::Device", ok && RowsClose(dv.Down<float>(by, x.size()), want, d, &detail), detail);
}

// A decode step recorded once and replayed at two different (token, position) pairs held in device
// memory (src/kernels/step_params.h): embedding gather, RMSNorm, RoPE, SwiGLU.
void CheckCapturedDecodeStep(Dev& dv) {
  const std::uint32_t vocab = 64, H = 256, heads = 4, hd = 64, rot = 16;
  const float theta = 1e7f, eps = 1e-6f;
  const std::size_t row_bytes = H / 32 * 34;
  std::vector<std::uint8_t> table(vocab * row_bytes);
  for (std::uint32_t v = 0; v < vocab; ++v) {
    auto row = Lcg(H, 3.0f);
    halo::quant::lowbit::EncodeQ8_0(row.data(), H, table.data() + v * row_bytes);
  }
  auto gamma = Lcg(H, 1.0f);
  for (auto& g : gamma) g += 1.0f;
  auto up = Lcg(H, 4.0f);
  std::vector<std::uint32_t> params(16, 0);
  rt::Buffer btab = dv.Up(table), bg = dv.Up(gamma), bup = dv.Up(up), bpar = dv.Up(params);
  rt::Buffer bx = dv.d->Alloc(H * 4, &dv.err);
  bool ok = dv.d->BeginCapture(&dv.err);
  std::string during;
  const bool refused = !dv.d->Upload(bpar, 0, params.data(), 64, &during);  // not capturable: must fail
  ok = ok && dv.Launch("halo_matvec_q8_0_embed_p", {(H + 255) / 256}, {256},
                       {rt::Arg::Buf(btab), rt::Arg::Buf(bx), rt::Arg::Buf(bpar), rt::Arg::Val(H),
                        rt::Arg::Val(static_cast<std::uint64_t>(row_bytes))});
  ok = ok && dv.Launch("halo_rmsnorm", {1}, {256},
                       {rt::Arg::Buf(bx), rt::Arg::Buf(bg), rt::Arg::Buf(bx), rt::Arg::Val(H), rt::Arg::Val(eps),
                        rt::Arg::Val(std::uint32_t{0})});
  ok = ok && dv.Launch("halo_rope_neox_p", {heads}, {64},
                       {rt::Arg::Buf(bx), rt::Arg::Buf(bpar), rt::Arg::Val(hd), rt::Arg::Val(rot), rt::Arg::Val(std::uint32_t{1}),
                        rt::Arg::Val(std::uint32_t{1}), rt::Arg::Val(theta)});
  ok = ok && dv.Launch("halo_silu_mul", {1}, {256}, {rt::Arg::Buf(bx), rt::Arg::Buf(bup), rt::Arg::Val(H)});
  rt::Graph graph;
  ok = ok && dv.d->EndCapture(&graph, &dv.err);
  Report("Upload is refused while capturing", refused, during);
  std::string detail = dv.err;
  const std::uint32_t steps[2][2] = {{5, 17}, {63, 262143}};
  for (const auto& st : steps) {
    params[0] = st[0];
    params[1] = st[1];
    ok = ok && dv.d->Upload(bpar, 0, params.data(), 64, &dv.err) && dv.d->LaunchGraph(graph, &dv.err);
    std::vector<float> want(H);
    halo::model::TensorRef ref;
    ref.data = table.data();
    ref.type = halo::core::GgmlType::kQ8_0;
    ref.cols = H;
    ref.rows = vocab;
    cpu::DequantizeRow(ref, 0, st[0], want.data());
    cpu::RmsNorm(want, gamma.data(), eps);
    cpu::Rope(want.data(), heads, hd, rot, st[1], theta);
    for (std::uint32_t i = 0; i < H; ++i) want[i] = cpu::Silu(want[i]) * up[i];
    ok = ok && RowsClose(dv.Down<float>(bx, H), want, hd, &detail);
  }
  dv.d->FreeGraph(graph);
  Report("captured decode step replayed at two positions", ok, detail);
}

void CheckErrors(Dev& dv) {
  std::string err;
  Report("a kernel outside the path is reported absent", dv.d->Kernel("halo_attention_decode", &err) < 0 && !err.empty(), err);
  err.clear();
  const rt::KernelId k = dv.d->Kernel("halo_l2norm", &err);
  rt::Buffer b = dv.d->Alloc(1024, &err);
  const bool refused = k >= 0 && !dv.d->Launch(k, {4}, {64}, std::vector<rt::Arg>{rt::Arg::Buf(b)}, &err);
  Report("a wrong argument list is refused with a message", refused && !err.empty(), err);
  dv.d->Free(b);
}

}  // namespace

int main() {
  std::string err;
  auto device = rt::CreateCudaDevice(0, &err);
  if (!device) {
    std::printf("FAIL no device: %s\n", err.c_str());
    return 2;
  }
  Dev dv{device.get(), {}};
  CheckGroupedNormRows(dv);
  CheckCapturedDecodeStep(dv);
  CheckErrors(dv);
  std::printf("%s\n", g_failures ? "FAILED" : "ALL PASS");
  return g_failures ? 1 : 0;
}
