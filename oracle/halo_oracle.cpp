// CPU oracle for the fused per-layer elementwise path. TEST INFRASTRUCTURE ONLY.
//
// A plain scalar restatement of halo-flash's CPU operators for the five op
// groups the CUDA library implements. Nothing here is shipped or measured as
// the product: it is the checker the parity tests, the smoke test and the
// benchmark's cpu_baseline leg compare against. Each function cites the
// reference file:line whose arithmetic (and evaluation order) it follows.
//
// Parity pin: this restatement is checked bit-for-bit against the reference's
// own sources compiled unmodified (oracle/_ref, built by oracle/Makefile) on
// seeded inputs, and against the reference's gguf-py golden blocks
// (tests/core/data/quant.tsv: Q8_0, F16, BF16 rows) and its known-answer
// tests for the fp16 conversion.
//
// Build: g++ -std=c++20 -O2 (no -march, no -ffast-math: x86-64 baseline has no
// FMA, so every multiply and add rounds separately, as in the reference build).

#include "row_pool.hpp"
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// src/core/quant.cpp:13-39 Fp16ToFloat: field-wise decode, subnormals as
// (mant / 1024) * 2^-14, inf/NaN keep the payload shifted left by 13.
float HalfBitsToFloat(std::uint16_t h) {
  const std::uint32_t sign = static_cast<std::uint32_t>(h & 0x8000u) << 16;
  const std::uint32_t e = (h >> 10) & 0x1Fu;
  const std::uint32_t m = h & 0x3FFu;
  std::uint32_t bits;
  if (e == 0) {
    if (m == 0) {
      bits = sign;
    } else {
      const float f = (static_cast<float>(m) / 1024.0f) * std::ldexp(1.0f, -14);
      return (h & 0x8000u) ? -f : f;
    }
  } else if (e == 31) {
    bits = sign | 0x7F800000u | (m << 13);
  } else {
    bits = sign | ((e + 112u) << 23) | (m << 13);
  }
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}

// src/core/quant.cpp:691-696 Bf16ToFloat and src/kernels/core.hip:66: bits << 16.
float Bf16BitsToFloat(std::uint16_t h) {
  const std::uint32_t bits = static_cast<std::uint32_t>(h) << 16;
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}

// src/kernels/core.hip:70-73 RSt(HaloBf16*): round to nearest even on the bit pattern.
std::uint16_t FloatToBf16Bits(float v) {
  std::uint32_t u;
  std::memcpy(&u, &v, 4);
  return static_cast<std::uint16_t>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// src/core/lowbit.cpp:14-20 ToHalf / Half: the compiler's _Float16 conversion (RNE).
std::uint16_t FloatToHalfBits(float v) {
  const auto h = static_cast<_Float16>(v);
  std::uint16_t bits;
  std::memcpy(&bits, &h, 2);
  return bits;
}
float RoundToHalf(float v) { return static_cast<float>(static_cast<_Float16>(v)); }

// src/model/cpu_ops.cpp:158-163.
float SigmoidF(float x) { return 1.0f / (1.0f + std::exp(-x)); }
float SiluF(float x) { return x * SigmoidF(x); }

// src/model/cpu_ops.cpp:134-145 RmsNorm: double sum of squares,
// scale = 1 / sqrt(float(ss / n) + eps), y = x * scale * w (w null -> 1).
void RmsNormRow(float* x, std::size_t n, const float* w, float eps) {
  double ss = 0.0;
  for (std::size_t i = 0; i < n; ++i) ss += static_cast<double>(x[i]) * x[i];
  const float scale = 1.0f / std::sqrt(static_cast<float>(ss / static_cast<double>(n)) + eps);
  for (std::size_t i = 0; i < n; ++i) x[i] = x[i] * scale * (w != nullptr ? w[i] : 1.0f);
}

// src/model/cpu_ops.cpp:147-156 L2Norm: eps is added to the sum, not the mean.
void L2NormRow(float* x, std::size_t n, float eps) {
  double ss = 0.0;
  for (std::size_t i = 0; i < n; ++i) ss += static_cast<double>(x[i]) * x[i];
  const float scale = 1.0f / std::sqrt(static_cast<float>(ss) + eps);
  for (std::size_t i = 0; i < n; ++i) x[i] *= scale;
}

// src/model/cpu_ops.cpp:168-185 Rope: NEOX pairs (i, i + rot/2) on the first
// `rot` dims of each head; freq = pow(theta, -2 i / rot) in fp32.
void RopeToken(float* x, std::uint32_t heads, std::uint32_t hd, std::uint32_t rot, std::uint32_t pos, float theta) {
  const std::uint32_t half = rot / 2;
  for (std::uint32_t h = 0; h < heads; ++h) {
    float* v = x + static_cast<std::size_t>(h) * hd;
    for (std::uint32_t i = 0; i < half; ++i) {
      const float freq = std::pow(theta, -2.0f * static_cast<float>(i) / static_cast<float>(rot));
      const float angle = static_cast<float>(pos) * freq;
      const float c = std::cos(angle), s = std::sin(angle);
      const float a = v[i], b = v[i + half];
      v[i] = a * c - b * s;
      v[i + half] = a * s + b * c;
    }
  }
}

// Rows [begin, end) of `fn` on `threads` host threads, contiguous chunks. The
// reference threads only its MatVec (src/model/cpu_ops.cpp:120-131); its
// trainer splits norm rows the same way (src/train/last_k.cpp:41-52).
using halo_oracle::ForRows;  // persistent row-parallel workers (row_pool.hpp)

}  // namespace

extern "C" {

const char* orc_kind() { return "port"; }

float orc_fp16_to_float(std::uint16_t h) { return HalfBitsToFloat(h); }
float orc_bf16_to_float(std::uint16_t h) { return Bf16BitsToFloat(h); }
std::uint16_t orc_float_to_bf16(float v) { return FloatToBf16Bits(v); }
std::uint16_t orc_float_to_fp16(float v) { return FloatToHalfBits(v); }
float orc_sigmoid(float x) { return SigmoidF(x); }
float orc_silu(float x) { return SiluF(x); }

// y[i] += x[i]: src/model/qwen35.cpp:322,329 (res += out).
void orc_add(float* y, const float* x, std::size_t n, int threads) {
  ForRows(n, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t i = b; i < e; ++i) y[i] += x[i];
  });
}

// In-place RMSNorm over `rows` vectors of length d. Row r uses gamma
// g + (r % w_period) * w_stride (src/kernels/core.hip:4049; w_stride 0 = shared);
// g null keeps the raw scale.
void orc_rmsnorm_rows(float* x, const float* g, std::size_t rows, std::size_t d, float eps, std::size_t w_stride,
                      std::size_t w_period, int threads) {
  if (w_period == 0) w_period = 1;
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r) RmsNormRow(x + r * d, d, g ? g + (r % w_period) * w_stride : nullptr, eps);
  });
}

void orc_l2norm_rows(float* x, std::size_t rows, std::size_t d, float eps, int threads) {
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r) L2NormRow(x + r * d, d, eps);
  });
}

// Gated RMSNorm, in place on o: src/model/qwen35.cpp:232-234 (RmsNorm with a
// plain per-dim weight shared by all heads, then *= Silu(z)); mode 1 uses
// Sigmoid(z) as src/model/reference.cpp:359-363.
void orc_gated_norm_rows(float* o, const float* w, const float* z, std::size_t rows, std::size_t d, float eps,
                         std::uint32_t mode, int threads) {
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r) {
      float* ov = o + r * d;
      const float* zv = z + r * d;
      RmsNormRow(ov, d, w, eps);
      for (std::size_t j = 0; j < d; ++j) ov[j] *= mode == 0 ? SiluF(zv[j]) : SigmoidF(zv[j]);
    }
  });
}

// x is [T][heads][hd]; token t rotates at position pos[t].
void orc_rope_rows(float* x, std::size_t tokens, std::uint32_t heads, std::uint32_t hd, std::uint32_t rot,
                   const std::uint32_t* pos, float theta, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t) RopeToken(x + t * heads * hd, heads, hd, rot, pos[t], theta);
  });
}

// pow(theta, -2 i / rot) for i < rot/2, the expression of cpu_ops.cpp:174-175.
void orc_rope_inv_freq(float* out, std::uint32_t rot, float theta) {
  for (std::uint32_t i = 0; i < rot / 2; ++i)
    out[i] = std::pow(theta, -2.0f * static_cast<float>(i) / static_cast<float>(rot));
}

// g = Silu(g) * up: src/model/qwen35.cpp:327.
void orc_silu_mul(float* g, const float* up, std::size_t n, int threads) {
  ForRows(n, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t i = b; i < e; ++i) g[i] = SiluF(g[i]) * up[i];
  });
}

// Row ids[t] of a Q8_0 table -> out[t][cols]: src/model/cpu_ops.cpp:47-72
// (DequantizeRow) and src/core/quant.cpp:411-421 (d * float(q) per 34-byte block).
void orc_embed_q8_0_rows(const std::uint8_t* table, const std::uint32_t* ids, std::size_t tokens, std::size_t cols,
                         std::size_t row_bytes, float* out, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t) {
      const std::uint8_t* row = table + static_cast<std::size_t>(ids[t]) * row_bytes;
      float* dst = out + t * cols;
      for (std::size_t blk = 0; blk < cols / 32; ++blk) {
        const std::uint8_t* p = row + blk * 34;
        std::uint16_t dh;
        std::memcpy(&dh, p, 2);
        const float d = HalfBitsToFloat(dh);
        for (std::size_t i = 0; i < 32; ++i) dst[blk * 32 + i] = d * static_cast<float>(static_cast<std::int8_t>(p[2 + i]));
      }
    }
  });
}

// F16 / BF16 rows to fp32 (cpu_ops.cpp:56-70), used against the golden blocks.
void orc_dequant_f16(const std::uint8_t* src, float* dst, std::size_t k) {
  for (std::size_t i = 0; i < k; ++i) {
    std::uint16_t h;
    std::memcpy(&h, src + 2 * i, 2);
    dst[i] = HalfBitsToFloat(h);
  }
}
void orc_dequant_bf16(const std::uint8_t* src, float* dst, std::size_t k) {
  for (std::size_t i = 0; i < k; ++i) {
    std::uint16_t h;
    std::memcpy(&h, src + 2 * i, 2);
    dst[i] = Bf16BitsToFloat(h);
  }
}

// True Q8_0 encode, src/core/lowbit.cpp:285-298: d = half(amax / 127),
// q = clamp(nearbyint(x / d), +-127) (0 when d == 0), block = LE fp16 d + 32 int8.
void orc_encode_q8_0_rows(const float* x, std::size_t rows, std::size_t cols, std::uint8_t* out, int threads) {
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r) {
      const float* xr = x + r * cols;
      std::uint8_t* orow = out + r * (cols / 32) * 34;
      for (std::size_t j = 0; j < cols / 32; ++j) {
        float amax = 0;
        for (std::size_t i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(xr[32 * j + i]));
        const float d = RoundToHalf(amax / 127.0f);
        std::uint8_t* blk = orow + 34 * j;
        const std::uint16_t dh = FloatToHalfBits(d);
        std::memcpy(blk, &dh, 2);
        for (std::size_t i = 0; i < 32; ++i) {
          const float q = d > 0 ? std::clamp(std::nearbyint(xr[32 * j + i] / d), -127.0f, 127.0f) : 0.0f;
          blk[2 + i] = static_cast<std::uint8_t>(static_cast<std::int8_t>(q));
        }
      }
    }
  });
}

// int8 activation form: scale = amax / 127 kept in fp32, q = rint(v / scale)
// (0 when scale == 0). Device recipe src/kernels/core.hip:3086-3101; the host
// check the reference's test applies is tests/gpu/quant_gpu_test.cpp:2482-2491.
// Row-major xq [rows][cols], xd [rows][cols / 32].
void orc_quantize_i8_rows(const float* x, std::size_t rows, std::size_t cols, std::int8_t* xq, float* xd,
                          int threads) {
  ForRows(rows, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t r = b; r < e; ++r)
      for (std::size_t j = 0; j < cols / 32; ++j) {
        float amax = 0.0f;
        for (std::size_t c = j * 32; c < j * 32 + 32; ++c) amax = std::max(amax, std::fabs(x[r * cols + c]));
        const float scale = amax / 127.0f;
        xd[r * (cols / 32) + j] = scale;
        for (std::size_t c = j * 32; c < j * 32 + 32; ++c)
          xq[r * cols + c] =
              static_cast<std::int8_t>(scale > 0.0f ? static_cast<int>(std::rint(x[r * cols + c] / scale)) : 0);
      }
  });
}

// Element-wise rounding helpers for 16-bit storage (residual stored in bf16:
// the norm reads the rounded value, src/kernels/core.hip:4132-4135).
void orc_round_bf16(float* x, std::size_t n) {
  for (std::size_t i = 0; i < n; ++i) x[i] = Bf16BitsToFloat(FloatToBf16Bits(x[i]));
}
void orc_round_fp16(float* x, std::size_t n) {
  for (std::size_t i = 0; i < n; ++i) x[i] = RoundToHalf(x[i]);
}

// ---- hyper-connection residual (Flash-Next) ------------------------------------------------
// res [T][hc][h] += out [T][h] * 2 sigmoid(inject [T][hc] / hc) (ReferenceModel::HcCombine,
// src/model/reference.cpp:189-202); the stored residual is then rounded as a 16-bit buffer would
// hold it (round: 0 none, 1 bf16, 2 fp16; src/kernels/core.hip:4132-4135) and y = GroupedNorm of the
// stored values: each stream normalized on its own under its slice of the [hc h] gamma
// (reference.cpp:151-160). out == NULL skips the combine. y may alias nothing else.
void orc_hc_combine_norm(float* res, const float* out, const float* inject, const float* w, float* y,
                         std::size_t tokens, std::size_t hc, std::size_t h, float eps, int round, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t)
      for (std::size_t s = 0; s < hc; ++s) {
        float* dst = res + (t * hc + s) * h;
        if (out != nullptr) {
          const float a = 2.0F * SigmoidF(inject[t * hc + s] / static_cast<float>(hc));
          for (std::size_t i = 0; i < h; ++i) dst[i] += out[t * h + i] * a;
        }
        if (round == 1) orc_round_bf16(dst, h);
        if (round == 2) orc_round_fp16(dst, h);
        float* yr = y + (t * hc + s) * h;
        for (std::size_t i = 0; i < h; ++i) yr[i] = dst[i];
        RmsNormRow(yr, h, w + s * h, eps);
      }
  });
}

// inject [T][irows] = iw [irows][hc h] . xn [T][hc h], double accumulation (MatVec(m.inject, 0, xn,
// inject), reference.cpp:185-187 through src/model/cpu_ops.cpp:108-118).
void orc_hc_inject(const float* xn, const float* iw, float* inject, std::size_t tokens, std::size_t cols,
                   std::size_t irows, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t)
      for (std::size_t r = 0; r < irows; ++r) {
        double acc = 0.0;
        for (std::size_t i = 0; i < cols; ++i) acc += static_cast<double>(iw[r * cols + i]) * xn[t * cols + i];
        inject[t * irows + r] = static_cast<float>(acc);
      }
  });
}

// mixed [T][h] = (sum over s of xn[t][s][i] * sigmoid(gate[t][s][i])) / hc (reference.cpp:179-188).
void orc_hc_mix(const float* xn, const float* gate, float* mixed, std::size_t tokens, std::size_t hc, std::size_t h,
                int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t) {
      float* m = mixed + t * h;
      for (std::size_t i = 0; i < h; ++i) m[i] = 0.0F;
      for (std::size_t s = 0; s < hc; ++s) {
        const std::size_t base = (t * hc + s) * h;
        for (std::size_t i = 0; i < h; ++i) m[i] += xn[base + i] * SigmoidF(gate[base + i]);
      }
      for (std::size_t i = 0; i < h; ++i) m[i] /= static_cast<float>(hc);
    }
  });
}

// out [T][h] = sum over slots, in order, of mw[t k + s] * yp[pos[t k + s]], then + sigmoid(sg[t]) * sx[t]
// (ReferenceModel::Moe, reference.cpp:558-578; rows of yp are the experts' down projections).
void orc_moe_combine(const float* yp, const std::uint32_t* pos, const float* mw, const float* sx, const float* sg,
                     float* out, std::size_t tokens, std::size_t k, std::size_t h, int threads) {
  ForRows(tokens, threads, [=](std::size_t b, std::size_t e) {
    for (std::size_t t = b; t < e; ++t) {
      float* o = out + t * h;
      for (std::size_t i = 0; i < h; ++i) o[i] = 0.0F;
      for (std::size_t s = 0; s < k; ++s) {
        const float weight = mw[t * k + s];
        const float* down = yp + static_cast<std::size_t>(pos[t * k + s]) * h;
        for (std::size_t j = 0; j < h; ++j) o[j] += weight * down[j];
      }
      if (sx == nullptr) continue;  // routed experts only
      const float g = SigmoidF(sg[t]);
      for (std::size_t j = 0; j < h; ++j) o[j] += g * sx[t * h + j];
    }
  });
}

// Gated DeltaNet conv step for `tokens` tokens in sequence (Qwen35Reference::Linear,
// src/model/qwen35.cpp:180-198): per channel acc = w[kern-1] * x; acc += w[k] * state[k] (k < kern-1),
// SiLU, the state shifts by the token, then the first l2_channels channels are L2-normalized per head
// of d channels (cpu::L2Norm with the eps passed). state [kern-1][channels] is updated in place.
void orc_conv_l2norm(const float* in, float* state, const float* w, float* out, std::size_t tokens,
                     std::size_t channels, std::size_t kern, std::size_t l2_channels, std::size_t d, float eps) {
  for (std::size_t t = 0; t < tokens; ++t) {
    const float* x = in + t * channels;
    float* o = out + t * channels;
    for (std::size_t ch = 0; ch < channels; ++ch) {
      float acc = w[ch * kern + kern - 1] * x[ch];
      for (std::size_t k = 0; k + 1 < kern; ++k) acc += w[ch * kern + k] * state[k * channels + ch];
      o[ch] = SiluF(acc);
    }
    if (kern > 1) {
      std::copy(state + channels, state + (kern - 1) * channels, state);
      std::copy(x, x + channels, state + (kern - 2) * channels);
    }
    for (std::size_t h = 0; h * d < l2_channels; ++h) L2NormRow(o + h * d, d, eps);
  }
}

}  // extern "C"
