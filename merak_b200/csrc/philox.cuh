// Counter-based random numbers (Philox4x32-10) for dropout: the mask of element e of call c at
// step offset o is a pure function of (seed, o + c, e), so the backward pass regenerates it
// instead of reading a stored mask.
#pragma once
#include <stdint.h>

namespace mrk {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ __forceinline__ void philox4x32_10(unsigned long long seed, unsigned long long stream,
                                              unsigned long long counter, uint32_t (&out)[4]) {
  uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), (uint32_t)stream, (uint32_t)(stream >> 32)};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = c[i];
}

// 8 uniforms in [0,1) for elements e .. e+7 (e must be a multiple of 8).
__device__ __forceinline__ void philox_uniform8(unsigned long long seed, unsigned long long stream,
                                                unsigned long long e, float (&r)[8]) {
  uint32_t a[4], b[4];
  philox4x32_10(seed, stream, e >> 2, a);
  philox4x32_10(seed, stream, (e >> 2) + 1, b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r[i] = (float)(a[i] >> 8) * (1.0f / 16777216.0f);
    r[4 + i] = (float)(b[i] >> 8) * (1.0f / 16777216.0f);
  }
}

}  // namespace mrk
