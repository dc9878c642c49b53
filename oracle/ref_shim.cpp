// Thin extern "C" shim over halo-flash's OWN CPU operators. TEST INFRASTRUCTURE ONLY.
//
// This file contains no arithmetic: every function loops over rows / heads and
// calls the reference's scalar operators (halo::model::cpu::*, halo::quant::*),
// which oracle/Makefile compiles unmodified from the reference checkout into
// oracle/_ref/libhalo_ref.so. It exports the same orc_* names as
// oracle/halo_oracle.cpp so the two can be compared bit for bit and either can
// serve as the checker or as the timed CPU baseline.

#include "row_pool.hpp"
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <span>
#include <thread>
#include <vector>

#include "core/lowbit.hpp"
#include "core/quant.hpp"
#include "model/cpu_ops.hpp"
#include "model/weights.hpp"

namespace {

namespace cpu = halo::model::cpu;

using halo_oracle::ForRows;  // persistent row-parallel workers (row_pool.hpp)

// What a bf16 residual buffer holds after a store of v: round to nearest even on the upper 16 bits
// (the GPU side's HaloBf16 store, src/kernels/core.hip:62-73), decoded by the reference's Bf16ToFloat.
float StoredBf16(float v) {
  std::uint32_t u;
  std::memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return v;
  u += 0x7fffu + ((u >> 16) & 1u);
  return halo::quant::Bf16ToFloat(static_cast<std::uint16_t>(u >> 16));
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

// ---- hyper-connection residual (Flash-Next) ------------------------------------------------
// ReferenceModel::HcCombine, GroupedNorm, HcMix and Moe (src/model/reference.cpp:151-202, 529-578) are
// members (or file-local helpers) of a class that needs a loaded model, so they cannot be called from
// here. These four functions repeat their loops around the reference's own scalar operators: the norm is
// cpu::RmsNorm, the gates are cpu::Sigmoid, the inject projection is cpu::MatVec over an F32 TensorRef;
// the only arithmetic written here is the `dst += out * a` / `m += x * gate` accumulation of those loops.
void orc_hc_combine_norm(float* res, const float* out, const float* inject, const float* w, float* y,
                         std::size_t tokens, std::size_t hc, std::size_t h, float eps, int round, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t)
      for (std::size_t s = 0; s < hc; ++s) {
        float* dst = res + (t * hc + s) * h;
        if (out != nullptr) {
          const float a = 2.0F * cpu::Sigmoid(inject[t * hc + s] / static_cast<float>(hc));
          for (std::size_t i = 0; i < h; ++i) dst[i] += out[t * h + i] * a;
        }
        if (round == 1)
          for (std::size_t i = 0; i < h; ++i) dst[i] = StoredBf16(dst[i]);
        if (round == 2)
          for (std::size_t i = 0; i < h; ++i) dst[i] = static_cast<float>(static_cast<_Float16>(dst[i]));
        float* yr = y + (t * hc + s) * h;
        std::copy(dst, dst + h, yr);
        cpu::RmsNorm(std::span<float>(yr, h), w + s * h, eps);
      }
  });
}

void orc_hc_inject(const float* xn, const float* iw, float* inject, std::size_t tokens, std::size_t cols,
                   std::size_t irows, int threads) {
  halo::model::TensorRef ref;
  ref.data = iw;
  ref.type = halo::core::GgmlType::kF32;
  ref.cols = cols;
  ref.rows = irows;
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t)
      cpu::MatVec(ref, 0, std::span<const float>(xn + t * cols, cols), std::span<float>(inject + t * irows, irows));
  });
}

void orc_hc_mix(const float* xn, const float* gate, float* mixed, std::size_t tokens, std::size_t hc, std::size_t h,
                int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t) {
      float* m = mixed + t * h;
      std::fill(m, m + h, 0.0F);
      for (std::size_t s = 0; s < hc; ++s) {
        const std::size_t base = (t * hc + s) * h;
        for (std::size_t i = 0; i < h; ++i) m[i] += xn[base + i] * cpu::Sigmoid(gate[base + i]);
      }
      for (std::size_t i = 0; i < h; ++i) m[i] /= static_cast<float>(hc);
    }
  });
}

void orc_moe_combine(const float* yp, const std::uint32_t* pos, const float* mw, const float* sx, const float* sg,
                     float* out, std::size_t tokens, std::size_t k, std::size_t h, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t) {
      float* o = out + t * h;
      std::fill(o, o + h, 0.0F);
      for (std::size_t s = 0; s < k; ++s) {
        const float weight = mw[t * k + s];
        const float* down = yp + static_cast<std::size_t>(pos[t * k + s]) * h;
        for (std::size_t j = 0; j < h; ++j) o[j] += weight * down[j];
      }
      if (sx == nullptr) continue;  // routed experts only
      const float g = cpu::Sigmoid(sg[t]);
      for (std::size_t j = 0; j < h; ++j) o[j] += g * sx[t * h + j];
    }
  });
}

// Qwen35Reference::Linear (src/model/qwen35.cpp:180-198) is a member of a class that needs a loaded
// model; its conv loop is repeated here around the reference's own cpu::Silu and cpu::L2Norm.
void orc_conv_l2norm(const float* in, float* state, const float* w, float* out, std::size_t tokens,
                     std::size_t channels, std::size_t kern, std::size_t l2_channels, std::size_t d, float eps) {
  for (std::size_t t = 0; t < tokens; ++t) {
    const float* x = in + t * channels;
    float* o = out + t * channels;
    for (std::size_t ch = 0; ch < channels; ++ch) {
      float acc = w[ch * kern + kern - 1] * x[ch];
      for (std::size_t k = 0; k + 1 < kern; ++k) acc += w[ch * kern + k] * state[k * channels + ch];
      o[ch] = cpu::Silu(acc);
    }
    if (kern > 1) {
      std::copy(state + channels, state + (kern - 1) * channels, state);
      std::copy(x, x + channels, state + (kern - 2) * channels);
    }
    for (std::size_t h = 0; h * d < l2_channels; ++h) cpu::L2Norm(std::span<float>(o + h * d, d), eps);
  }
}

}  // extern "C"
