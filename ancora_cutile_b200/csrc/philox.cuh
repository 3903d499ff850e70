// Philox4x32-10 (Random123 constants) and the two float32 -> bf16 roundings every producer of
// bf16 bits in this library uses.  The stochastic rounding is the bit rule of
// ancora/kernels/fused.py:159-161, (bits + dither16) >> 16, with NaN mapped to 0x7FFF.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ uint32_t bf16_rne(float x) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
}

__device__ __forceinline__ uint32_t bf16_sr(float x, uint32_t dither16) {
  const uint32_t u = __float_as_uint(x);
  return (x != x) ? 0x7FFFu : ((u + dither16) >> 16);
}
