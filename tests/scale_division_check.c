/* Checks that the division-free scale of the FP8 group quantizer equals the IEEE quotient.
 *
 * The quantizer computes scale = max(amax / qmax, 1e-12) (reference statement:
 * benchmarks/bench.py:2339-2344) as q0 = amax * r, e = fma(-q0, qmax, amax),
 * q = fma(e, r, q0) with r = RN(1 / qmax). This program compares max(q, 1e-12) with
 * max(amax / qmax, 1e-12) for positive finite floats: all of them with stride 1, or every
 * stride-th bit pattern plus every value a bf16 or fp16 input can take.
 *
 * usage: scale_division_check <qmax> <stride>      prints "mismatches=<n> checked=<n>"
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float from_bits(uint32_t b) {
  float f;
  memcpy(&f, &b, 4);
  return f;
}

static int differs(float a, float qmax, float r) {
  const float ref = fmaxf(a / qmax, 1e-12f);
  const float q0 = a * r;
  const float e = fmaf(-q0, qmax, a);
  const float q = fmaxf(fmaf(e, r, q0), 1e-12f);
  return memcmp(&ref, &q, 4) != 0;
}

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  const float qmax = (float)atof(argv[1]);
  const uint32_t stride = (uint32_t)atoi(argv[2]);
  const float r = 1.0f / qmax;
  unsigned long long bad = 0, n = 0;
  for (uint64_t b = 0; b < 0x7f800000u; b += stride, ++n) bad += differs(from_bits((uint32_t)b), qmax, r);
  /* every bf16 value: the upper 16 bits of a float */
  for (uint32_t h = 0; h < 0x7f80u; ++h, ++n) bad += differs(from_bits(h << 16), qmax, r);
  /* every fp16 value, converted exactly */
  for (uint32_t h = 0; h < 0x7c00u; ++h, ++n) {
    const uint32_t ex = h >> 10, man = h & 0x3ffu;
    const float v = ex ? ldexpf((float)(man | 0x400u), (int)ex - 25) : ldexpf((float)man, -24);
    bad += differs(v, qmax, r);
  }
  printf("mismatches=%llu checked=%llu\n", bad, n);
  return bad != 0;
}
