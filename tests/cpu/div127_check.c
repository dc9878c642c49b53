/* Checks, on the host, the division-free quotient the CUDA Q8 encoders use for amax / 127:
 *   q0 = x * z, z = RN(1 / 127);  r = fma(-q0, 127, x);  q = fma(r, z, q0)
 * against the IEEE division x / 127.0f, over a range of float bit patterns [lo, hi).
 * fmaf() is the C library's correctly rounded fused multiply-add, the operation the device's
 * fma.rn.f32 performs. Prints the number of mismatches and the first one.
 *
 *   div127_check <lo hex> <hi hex> [stride]
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  const uint64_t lo = strtoull(argv[1], NULL, 16), hi = strtoull(argv[2], NULL, 16);
  const uint64_t stride = argc > 3 ? strtoull(argv[3], NULL, 10) : 1;
  const float z = 1.0f / 127.0f;
  uint64_t bad = 0, first = 0, n = 0;
  for (uint64_t b = lo; b < hi; b += stride, ++n) {
    const uint32_t u = (uint32_t)b;
    float x;
    memcpy(&x, &u, 4);
    const float q0 = x * z;
    const float r = fmaf(-q0, 127.0f, x);
    const float q = fmaf(r, z, q0);
    const float want = x / 127.0f;
    if (memcmp(&q, &want, 4) != 0) {
      if (!bad) first = b;
      ++bad;
    }
  }
  printf("%llu %llu %llx\n", (unsigned long long)n, (unsigned long long)bad, (unsigned long long)first);
  return 0;
}
