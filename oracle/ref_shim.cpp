// Thin extern "C" shim over halo-flash's OWN CPU operators. TEST INFRASTRUCTURE ONLY.
//
// This file contains no arithmetic: every function loops over rows / heads and
// calls the reference's scalar operators (halo::model::cpu::*, halo::quant::*),
// which oracle/Makefile compiles unmodified from the reference checkout into
// oracle/_ref/libhalo_ref.so. It exports the same orc_* names as
// oracle/halo_oracle.cpp so the two can be compared bit for bit and either can
// serve as the checker or as the timed CPU baseline.

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <span>
#include <thread>
#include <vector>

#include "core/lowbit.hpp"
#include "core/quant.hpp"
#include "model/cpu_ops.hpp"

namespace {

namespace cpu = halo::model::cpu;

template <typename Fn>
void ForRows(std::size_t rows, int threads, Fn fn) {
  if (threads <= 1 || rows < 2) {
    fn(0, rows);
    return;
  }
  const std::size_t nt = std::min<std::size_t>(static_cast<std::size_t>(threads), rows);
  const std::size_t chunk = (rows + nt - 1) / nt;
  std::vector<std::thread> pool;
  for (std::size_t b = 0; b < rows; b += chunk) pool.emplace_back(fn, b, std::min(rows, b + chunk));
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

const char* orc_kind() { return "reference"; }

float orc_fp16_to_float(std::uint16_t h) { return halo::quant::Fp16ToFloat(h); }
float orc_bf16_to_float(std::uint16_t h) { return halo::quant::Bf16ToFloat(h); }
float orc_sigmoid(float x) { return cpu::Sigmoid(x); }
float orc_silu(float x) { return cpu::Silu(x); }

void orc_rmsnorm_rows(float* x, const float* g, std::size_t rows, std::size_t d, float eps, std::size_t w_stride,
                      std::size_t w_period, int threads) {
  if (w_period == 0) w_period = 1;
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r)
      cpu::RmsNorm(std::span<float>(x + r * d, d), g ? g + (r % w_period) * w_stride : nullptr, eps);
  });
}

void orc_l2norm_rows(float* x, std::size_t rows, std::size_t d, float eps, int threads) {
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r) cpu::L2Norm(std::span<float>(x + r * d, d), eps);
  });
}

// The call sequence of Qwen35Reference::Linear's output norm: RmsNorm with the
// plain weight, then o[j] *= Silu(z[j]) (mode 0) or Sigmoid(z[j]) (mode 1).
void orc_gated_norm_rows(float* o, const float* w, const float* z, std::size_t rows, std::size_t d, float eps,
                         std::uint32_t mode, int threads) {
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r) {
      float* ov = o + r * d;
      const float* zv = z + r * d;
      cpu::RmsNorm(std::span<float>(ov, d), w, eps);
      for (std::size_t j = 0; j < d; ++j) ov[j] *= mode == 0 ? cpu::Silu(zv[j]) : cpu::Sigmoid(zv[j]);
    }
  });
}

void orc_rope_rows(float* x, std::size_t tokens, std::uint32_t heads, std::uint32_t hd, std::uint32_t rot,
                   const std::uint32_t* pos, float theta, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t) cpu::Rope(x + t * heads * hd, heads, hd, rot, pos[t], theta);
  });
}

void orc_silu_mul(float* g, const float* up, std::size_t n, int threads) {
  ForRows(n, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t i = b; i < e; ++i) g[i] = cpu::Silu(g[i]) * up[i];
  });
}

void orc_embed_q8_0_rows(const std::uint8_t* table, const std::uint32_t* ids, std::size_t tokens, std::size_t cols,
                         std::size_t row_bytes, float* out, int threads) {
  (void)row_bytes;  // TensorRef::RowBytes() derives it from the format and cols
  halo::model::TensorRef t;
  t.data = table;
  t.type = halo::core::GgmlType::kQ8_0;
  t.cols = cols;
  t.rows = 1;  // rows are addressed directly; Expert(0) is the base
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t i = b; i < e; ++i) cpu::DequantizeRow(t, 0, ids[i], out + i * cols);
  });
}

void orc_dequant_f16(const std::uint8_t* src, float* dst, std::size_t k) {
  halo::model::TensorRef t;
  t.data = src;
  t.type = halo::core::GgmlType::kF16;
  t.cols = k;
  cpu::DequantizeRow(t, 0, 0, dst);
}
void orc_dequant_bf16(const std::uint8_t* src, float* dst, std::size_t k) {
  halo::model::TensorRef t;
  t.data = src;
  t.type = halo::core::GgmlType::kBF16;
  t.cols = k;
  cpu::DequantizeRow(t, 0, 0, dst);
}

void orc_encode_q8_0_rows(const float* x, std::size_t rows, std::size_t cols, std::uint8_t* out, int threads) {
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r)
      halo::quant::lowbit::EncodeQ8_0(x + r * cols, cols, out + r * (cols / 32) * 34);
  });
}

}  // extern "C"
