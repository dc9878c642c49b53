// The lean row-norm kernels with three and five octets per thread: rows of 3 g or 5 g octets (H = 1536, 2560, 3072,
// 5120, ...), which the power-of-two layouts of norm.cu would pad. A translation unit of its own so that these
// instantiations compile beside norm.cu's; kernels and launchers are in norm_lean.cuh.
#include "norm_lean.cuh"

namespace halo_b200 {
namespace {

template <typename XT, typename YT, bool ADD>
cudaError_t LaunchOddT(const NormArgs& a, const Shape& sh, unsigned grid, cudaStream_t s) {
  // the (in, out) pairs the lean kernels are built for (the same set as in norm.cu)
  constexpr bool kLeanTypes = (std::is_same_v<XT, float> && !std::is_same_v<YT, f16>) ||
                              (std::is_same_v<XT, bf16> && !std::is_same_v<YT, f16>) ||
                              (std::is_same_v<XT, f16> && std::is_same_v<YT, f16>);
  if constexpr (kLeanTypes) {
    if (sh.k == 3) return LaunchLean<XT, YT, 3, ADD>(a, sh, grid, s);
    if constexpr (sizeof(XT) == 2) {
      if (sh.k == 5) return LaunchLean<XT, YT, 5, ADD>(a, sh, grid, s);
    }
  }
  return cudaErrorInvalidValue;
}

template <typename XT>
cudaError_t LaunchOddY(const NormArgs& a, const Shape& sh, unsigned grid, cudaStream_t s) {
  switch (a.y_dtype) {
    case kF32: return a.delta ? LaunchOddT<XT, float, true>(a, sh, grid, s) : LaunchOddT<XT, float, false>(a, sh, grid, s);
    case kF16: return a.delta ? LaunchOddT<XT, f16, true>(a, sh, grid, s) : LaunchOddT<XT, f16, false>(a, sh, grid, s);
    case kBF16: return a.delta ? LaunchOddT<XT, bf16, true>(a, sh, grid, s) : LaunchOddT<XT, bf16, false>(a, sh, grid, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t LaunchNormLeanOdd(const NormArgs& a, unsigned lg, int k, unsigned rows_per_cta, unsigned grid, cudaStream_t s) {
  Shape sh;
  sh.lg = lg, sh.k = k, sh.r = 1, sh.rows_per_cta = rows_per_cta, sh.full = true;
  switch (a.x_dtype) {
    case kF32: return LaunchOddY<float>(a, sh, grid, s);
    case kF16: return LaunchOddY<f16>(a, sh, grid, s);
    case kBF16: return LaunchOddY<bf16>(a, sh, grid, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace halo_b200
