// Dropout on the attention probabilities, evaluated inside the flash kernels.
//
// The keep decision of element (batch, head, query q, key k) is a stateless hash, so the forward
// kernel (a thread owns a query row) and the backward kernel (a thread owns a key row) regenerate the
// same mask without storing it:
//     row key  = mix(mix(base ^ bh * C1) + q * C2)             base = mix of (seed, offset + call id)
//     keep     = mix(row key ^ k * C3) >= p * 2^32
// with mix the 32-bit finaliser of MurmurHash3.  Replaces the dropout of the eager
// matmul -> softmax -> dropout -> matmul attention the reference's models run
// (examples/models/gpt2/config.py:28).
#pragma once
#include <cstdint>

namespace mrk {

__host__ __device__ __forceinline__ uint32_t attn_mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}
__host__ __device__ __forceinline__ uint32_t attn_drop_base(unsigned long long seed, unsigned long long stream) {
  return attn_mix32((uint32_t)seed ^ attn_mix32((uint32_t)(seed >> 32) + 0x9E3779B9u) ^
                    attn_mix32((uint32_t)stream * 0x9E3779B1u + (uint32_t)(stream >> 32)));
}
__host__ __device__ __forceinline__ uint32_t attn_drop_rowkey(uint32_t base, uint32_t bh, uint32_t q) {
  return attn_mix32(attn_mix32(base ^ (bh * 0x85EBCA6Bu)) + q * 0xC2B2AE35u);
}
__host__ __device__ __forceinline__ bool attn_drop_keep(uint32_t rowkey, uint32_t k, uint32_t thresh) {
  return attn_mix32(rowkey ^ (k * 0x9E3779B1u)) >= thresh;
}
// p * 2^32, saturated
__host__ __device__ __forceinline__ uint32_t attn_drop_thresh(float p) {
  const double t = (double)p * 4294967296.0;
  return t >= 4294967295.0 ? 0xFFFFFFFFu : (uint32_t)t;
}

}  // namespace mrk
