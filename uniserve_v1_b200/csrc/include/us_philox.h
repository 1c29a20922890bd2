// Philox4x32-10 addressed by (seed, position, stage, draw); the same function
// compiles for the host and the device, so the scheduler, the CPU reference
// and the kernels produce identical draws.
//
//   key     = the two halves of splitmix64(seed)
//   counter = [position low, position high, stage, draw]
//
// Reference behaviour: crates/engine/src/batch/philox.rs:18-35 (reference
// project path): a draw is a function of (seed, position) only.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define US_HD __host__ __device__ __forceinline__
#else
#define US_HD inline
#endif

US_HD uint64_t us_splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

US_HD void us_mulhilo32(uint32_t a, uint32_t b, uint32_t* hi, uint32_t* lo) {
  const uint64_t p = (uint64_t)a * (uint64_t)b;
  *hi = (uint32_t)(p >> 32);
  *lo = (uint32_t)p;
}

US_HD void us_philox4x32_10(uint64_t seed, uint64_t position, uint32_t stage, uint32_t draw,
                            uint32_t out[4]) {
  const uint64_t k = us_splitmix64(seed);
  uint32_t k0 = (uint32_t)k, k1 = (uint32_t)(k >> 32);
  uint32_t c0 = (uint32_t)position, c1 = (uint32_t)(position >> 32), c2 = stage, c3 = draw;
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    us_mulhilo32(0xD2511F53u, c0, &hi0, &lo0);
    us_mulhilo32(0xCD9E8D57u, c2, &hi1, &lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n1 = lo1;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    const uint32_t n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// One uniform in [0, 1): the top 24 bits of word 0.
US_HD float us_philox_uniform(uint64_t seed, uint64_t position, uint32_t stage, uint32_t draw) {
  uint32_t w[4];
  us_philox4x32_10(seed, position, stage, draw, w);
  return (float)(w[0] >> 8) * (1.0f / 16777216.0f);
}

// Two standard normals (Box-Muller) from words 0..1 of one counter.
US_HD void us_philox_normal2(uint64_t seed, uint64_t position, uint32_t stage, uint32_t draw,
                             float* n0, float* n1) {
  uint32_t w[4];
  us_philox4x32_10(seed, position, stage, draw, w);
  const float u0 = ((float)(w[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
  const float u1 = ((float)(w[1] >> 8) + 0.5f) * (1.0f / 16777216.0f);
#if defined(__CUDA_ARCH__)
  const float r = sqrtf(-2.f * logf(u0));
  float s, c;
  sincosf(6.283185307179586f * u1, &s, &c);
#else
  const float r = __builtin_sqrtf(-2.f * __builtin_logf(u0));
  const float s = __builtin_sinf(6.283185307179586f * u1);
  const float c = __builtin_cosf(6.283185307179586f * u1);
#endif
  *n0 = r * c;
  *n1 = r * s;
}
