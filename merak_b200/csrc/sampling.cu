// Next-token sampling for text generation: temperature, top-k and top-p (nucleus) filtering, softmax
// and the draw, one launch for the whole batch (one thread block per row of logits).
//
// Replaces the chain of ATen kernels the reference runs per generated token (topk, sort, softmax,
// cumsum, scatter, multinomial: Merak/inference/text_generation_inference.py:35-69,221-235).
//
//   1. radix select (four 8-bit passes over the order-preserving integer image of the floats) finds
//      the k-th largest logit of the row;
//   2. the logits above it and as many ties as needed are gathered into shared memory (k <= 1024) and
//      sorted in descending order with a bitonic network;
//   3. softmax over the kept candidates at the given temperature, nucleus cut (the shortest prefix
//      whose probability mass exceeds top_p, always at least one token), renormalisation;
//   4. the token is drawn by inverting the cumulative distribution at a uniform number, taken from
//      `uniforms[row]` when given (tests) or from Philox(seed, row) otherwise.  `greedy` returns the
//      arg-max instead.
#include <cuda_bf16.h>
#include <math.h>

#include "elementwise.h"
#include "host_common.h"
#include "philox.cuh"

namespace mrk {

constexpr int kSampleThreads = 256;
constexpr int kSampleMaxK = 1024;

__device__ __forceinline__ uint32_t float_key(float f) {      // larger float <-> larger key
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_topk_topp_kernel(const T* __restrict__ logits, long long row_stride, int V, int top_k, float top_p,
                        float inv_temperature, int greedy, const float* __restrict__ uniforms,
                        unsigned long long seed, unsigned long long step, long long* __restrict__ out_token,
                        float* __restrict__ out_prob) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_remaining;
  __shared__ float cand_val[kSampleMaxK];
  __shared__ int cand_idx[kSampleMaxK];
  __shared__ int s_count, s_tie_room;
  __shared__ float red[kSampleThreads / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* x = logits + (long long)row * row_stride;
  const int k = top_k < 1 ? 1 : (top_k > kSampleMaxK ? kSampleMaxK : (top_k > V ? V : top_k));

  // ---- 1. k-th largest key by radix select ----
  if (tid == 0) { s_prefix = 0u; s_remaining = (uint32_t)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    hist[tid] = 0u;                                       // kSampleThreads == 256 bins
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < V; i += kSampleThreads) {
      const uint32_t key = float_key(load_logit<T>(x, i));
      if ((key & mask) == (prefix & mask)) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t need = s_remaining;
      int b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_prefix = prefix | ((uint32_t)b << shift);
      s_remaining = need;                                 // how many keys equal to the final threshold are kept
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;
  // ---- 2. gather: everything above the threshold, then ties up to k ----
  if (tid == 0) { s_count = 0; s_tie_room = (int)s_remaining; }
  __syncthreads();
  for (int i = tid; i < V; i += kSampleThreads) {
    const float v = load_logit<T>(x, i);
    const uint32_t key = float_key(v);
    bool take = key > kth;
    if (!take && key == kth) take = atomicSub(&s_tie_room, 1) > 0;
    if (take) {
      const int slot = atomicAdd(&s_count, 1);
      if (slot < kSampleMaxK) { cand_val[slot] = v; cand_idx[slot] = i; }
    }
  }
  __syncthreads();
  const int n = min(s_count, k);
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  for (int i = n + tid; i < n2; i += kSampleThreads) { cand_val[i] = -INFINITY; cand_idx[i] = 0x7fffffff; }
  __syncthreads();
  // bitonic sort, descending by value (ascending index among equal values: deterministic)
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < n2; i += kSampleThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const bool desc = (i & size) == 0;
          const float a = cand_val[i], b = cand_val[j];
          const int ia = cand_idx[i], ib = cand_idx[j];
          const bool a_first = a > b || (a == b && ia < ib);
          if (desc ? !a_first : a_first) {
            cand_val[i] = b; cand_val[j] = a;
            cand_idx[i] = ib; cand_idx[j] = ia;
          }
        }
      }
      __syncthreads();
    }
  }
  if (greedy) {
    if (tid == 0) {
      out_token[row] = cand_idx[0];
      if (out_prob) out_prob[row] = 1.f;
    }
    return;
  }
  // ---- 3. softmax over the candidates, nucleus cut ----
  const float vmax = cand_val[0];
  float part = 0.f;
  for (int i = tid; i < n; i += kSampleThreads) {
    const float e = __expf((cand_val[i] - vmax) * inv_temperature);
    cand_val[i] = e;
    part += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((tid & 31) == 0) red[tid >> 5] = part;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int w = 0; w < kSampleThreads / 32; ++w) total += red[w];
    // shortest prefix whose mass exceeds top_p (sequential: at most 1024 terms)
    int keep = n;
    if (top_p > 0.f && top_p < 1.f) {
      float cum = 0.f;
      for (int i = 0; i < n; ++i) {
        cum += cand_val[i] / total;
        if (cum > top_p) { keep = i + 1; break; }
      }
    }
    float kept = 0.f;
    for (int i = 0; i < keep; ++i) kept += cand_val[i];
    // ---- 4. draw ----
    float u;
    if (uniforms) {
      u = uniforms[row];
    } else {
      uint32_t r4[4];
      philox4x32_10(seed, step, (unsigned long long)row, r4);
      u = (float)(r4[0] >> 8) * (1.0f / 16777216.0f);
    }
    const float target = u * kept;
    float cum = 0.f;
    int pick = keep - 1;
    for (int i = 0; i < keep; ++i) {
      cum += cand_val[i];
      if (target < cum) { pick = i; break; }
    }
    out_token[row] = cand_idx[pick];
    if (out_prob) out_prob[row] = cand_val[pick] / kept;
  }
}

}  // namespace mrk

using namespace mrk;

// logits [rows, V] (fp32 or bf16, row pitch `row_stride` elements); out_token int64 [rows]; out_prob
// optional fp32 [rows] (probability of the drawn token after filtering).  1 <= top_k <= 1024.
MRK_API int mrk_sample_topk_topp(const void* logits, int is_bf16, long long rows, int V, long long row_stride,
                                 int top_k, float top_p, float temperature, int greedy, const float* uniforms,
                                 unsigned long long seed, unsigned long long step, long long* out_token,
                                 float* out_prob, void* stream) {
  MRK_REQUIRE(rows > 0 && V > 0 && logits && out_token, "sample: bad arguments");
  MRK_REQUIRE(top_k >= 1 && top_k <= kSampleMaxK, "sample: top_k %d outside [1, %d]", top_k, kSampleMaxK);
  MRK_REQUIRE(greedy || temperature > 0.f, "sample: temperature must be positive");
  cudaStream_t s = (cudaStream_t)stream;
  const float inv_t = greedy ? 1.f : 1.f / temperature;
  if (is_bf16)
    sample_topk_topp_kernel<__nv_bfloat16><<<(unsigned)rows, kSampleThreads, 0, s>>>(
        (const __nv_bfloat16*)logits, row_stride, V, top_k, top_p, inv_t, greedy, uniforms, seed, step, out_token,
        out_prob);
  else
    sample_topk_topp_kernel<float><<<(unsigned)rows, kSampleThreads, 0, s>>>(
        (const float*)logits, row_stride, V, top_k, top_p, inv_t, greedy, uniforms, seed, step, out_token, out_prob);
  MRK_CHECK_LAUNCH();
  return 0;
}
