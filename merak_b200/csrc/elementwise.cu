// Memory-bound kernels around the GEMMs: softmax cross-entropy (plain and vocab-parallel),
// fused AdamW on flat buffers, embedding gather / scatter-add, rotary embedding, SwiGLU,
// bias-gradient column sums, dropout, casts and squared-norm reductions.  Every kernel moves
// 16 bytes per thread per access and is sized as a multiple of the SM count.
//
// Reference call sites these replace: vocab-parallel cross entropy
// (Merak/core/mpu/cross_entropy.py:26-118), torch.optim.AdamW + fp32 master copy-back
// (Merak/core/zero/stage1.py:734-740), grad-norm / clipping (Merak/core/pipeline/utils.py:38-111),
// VocabParallelEmbedding (Merak/core/mpu/layers.py:145-165), HF rotary embedding and SwiGLU
// python ops (Merak/core/sequence_parallel/modeling/llama.py:227-228).
#include "elementwise.h"
#include "host_common.h"
#include "philox.cuh"
#include "sm100_ptx.cuh"
#include "activations.cuh"

namespace mrk {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

static inline unsigned grid_for(long long work_items, int threads, int waves = 8) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * waves;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

// -------------------------------------------------------------------------------------------------
// Cross entropy.  One CTA per row.  Pass 1 (online max / sum-exp, target logit) reads the row once;
// when gradients are requested the row is read again (L2-resident) and dlogits written.
//   stats[row] = {max, sumexp, target_logit} in natural units, for the local vocabulary slice
//   [vocab_start, vocab_start + V).
// -------------------------------------------------------------------------------------------------
constexpr int kCeThreads = 256;

template <bool kF32>
__device__ __forceinline__ void load_logits8(const void* base, long long idx, float (&f)[8]) {
  if (kF32) {
    const float4 a = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx)[0];
    const float4 b = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = unpack_bf16x2(w[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

template <bool kF32>
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const void* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ stats,
                long long M, int V, long long ld, int vocab_start, int ignore_index) {
  __shared__ float red_m[kCeThreads / 32], red_s[kCeThreads / 32];
  const long long row = blockIdx.x;
  if (row >= M) return;
  const long long base = row * ld;
  float m = -INFINITY, s = 0.f;
  const int nvec = V / 8;
  for (int vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
    float f[8];
    load_logits8<kF32>(logits, base + (long long)vi * 8, f);
    float bm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) bm = fmaxf(bm, f[i]);
    const float nm = fmaxf(m, bm);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += __expf(f[i] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += kCeThreads) {   // ragged tail
    const float x = kF32 ? reinterpret_cast<const float*>(logits)[base + c]
                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[base + c]);
    const float nm = fmaxf(m, x);
    s = s * __expf(m - nm) + __expf(x - nm);
    m = nm;
  }
  // combine (max, sum) pairs across the block
  const float wm = warp_max(m);
  s = warp_sum(s * (m == -INFINITY ? 0.f : __expf(m - wm)));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { red_m[warp] = wm; red_s[warp] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = red_m[0];
    for (int w = 1; w < kCeThreads / 32; ++w) bm = fmaxf(bm, red_m[w]);
    float bs = 0.f;
    for (int w = 0; w < kCeThreads / 32; ++w) bs += red_s[w] * (red_m[w] == -INFINITY ? 0.f : __expf(red_m[w] - bm));
    const long long lab = labels[row];
    float tgt = 0.f;
    const long long local = lab - vocab_start;
    if (lab != ignore_index && local >= 0 && local < V)
      tgt = kF32 ? reinterpret_cast<const float*>(logits)[base + local]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[base + local]);
    stats[row * 3 + 0] = bm;
    stats[row * 3 + 1] = bs;
    stats[row * 3 + 2] = tgt;
  }
}

// loss[row] = lse - target (0 for ignored rows); dlogits = (softmax - onehot) * grad_scale[0] (0 for ignored).
// `lse` holds the global log-sum-exp per row (after the tensor-parallel exchange when vocab is sharded).
template <bool kF32>
__global__ void __launch_bounds__(kCeThreads)
ce_grad_kernel(const void* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ lse,
               const float* __restrict__ grad_scale, void* __restrict__ dlogits, long long M, int V, long long ld,
               long long ldd, int vocab_start, int ignore_index) {
  const long long row = blockIdx.x;
  if (row >= M) return;
  const long long lab = labels[row];
  const bool ignored = lab == ignore_index;
  const float l = lse[row];
  const float gs = ignored ? 0.f : grad_scale[0];
  const long long local = lab - vocab_start;
  const long long base = row * ld, dbase = row * ldd;
  const int nvec = V / 8;
  for (int vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
    float f[8];
    load_logits8<kF32>(logits, base + (long long)vi * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float g = __expf(f[i] - l);
      if ((long long)vi * 8 + i == local) g -= 1.f;
      f[i] = g * gs;
    }
    if (kF32) {
      float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(dlogits) + dbase + (long long)vi * 8);
      d[0] = make_float4(f[0], f[1], f[2], f[3]);
      d[1] = make_float4(f[4], f[5], f[6], f[7]);
    } else {
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dlogits) + dbase + (long long)vi * 8) =
          make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += kCeThreads) {
    const float x = kF32 ? reinterpret_cast<const float*>(logits)[base + c]
                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[base + c]);
    float g = __expf(x - l);
    if (c == local) g -= 1.f;
    g *= gs;
    if (kF32) reinterpret_cast<float*>(dlogits)[dbase + c] = g;
    else reinterpret_cast<__nv_bfloat16*>(dlogits)[dbase + c] = __float2bfloat16(g);
  }
}

// Reduces per-row stats into: lse[row], loss_sum (atomic), valid_count (atomic).  `tp_parts` partial
// stats blocks laid out [part][row][3] are merged first (1 for the single-GPU case).
__global__ void ce_finalize_kernel(const float* __restrict__ stats, int tp_parts, long long part_stride,
                                   const long long* __restrict__ labels, float* __restrict__ lse,
                                   float* __restrict__ loss_rows, float* __restrict__ loss_sum,
                                   float* __restrict__ valid_count, long long M, int ignore_index) {
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float loss = 0.f, valid = 0.f;
  if (row < M) {
    float m = -INFINITY;
    for (int t = 0; t < tp_parts; ++t) m = fmaxf(m, stats[t * part_stride + row * 3]);
    float s = 0.f, tgt = 0.f;
    for (int t = 0; t < tp_parts; ++t) {
      const float pm = stats[t * part_stride + row * 3];
      s += stats[t * part_stride + row * 3 + 1] * (pm == -INFINITY ? 0.f : __expf(pm - m));
      tgt += stats[t * part_stride + row * 3 + 2];
    }
    const float l = m + __logf(s);
    lse[row] = l;
    if (labels[row] != ignore_index) { loss = l - tgt; valid = 1.f; }
    if (loss_rows) loss_rows[row] = loss;
  }
  loss = warp_sum(loss);
  valid = warp_sum(valid);
  if ((threadIdx.x & 31) == 0) {
    if (loss != 0.f) atomicAdd(loss_sum, loss);
    if (valid != 0.f) atomicAdd(valid_count, valid);
  }
}

// -------------------------------------------------------------------------------------------------
// Fused AdamW on flat buffers.  grad may be bf16 or fp32; master/m/v are fp32; an optional bf16
// (or fp32) model copy is refreshed in the same pass.  Scalars that change every step (lr, bias
// corrections, the gradient scale produced by clipping / loss scaling, and the skip flag raised by
// an overflow) are read from device memory so the launch is CUDA-graph replayable.
//   hp = {lr, beta1, beta2, eps, weight_decay, bias_correction1, bias_correction2}
// -------------------------------------------------------------------------------------------------
template <bool kGradF32, bool kOutF32>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, const void* __restrict__ grad,
             void* __restrict__ model_out, const float* __restrict__ hp, const float* __restrict__ grad_scale,
             const int* __restrict__ skip, long long n) {
  if (skip != nullptr && *skip != 0) return;
  const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4], bc1 = hp[5], bc2 = hp[6];
  const float gs = grad_scale ? grad_scale[0] : 1.f;
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float g[4];
    if (kGradF32) {
      const float4 t = reinterpret_cast<const float4*>(grad)[i];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(grad)[i];
      const float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    }
    float4 p4 = reinterpret_cast<float4*>(master)[i], m4 = reinterpret_cast<float4*>(m)[i], v4 = reinterpret_cast<float4*>(v)[i];
    float pp[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = g[k] * gs;
      mm[k] = b1 * mm[k] + (1.f - b1) * gk;
      vv[k] = b2 * vv[k] + (1.f - b2) * gk * gk;
      const float mh = mm[k] / bc1, vh = vv[k] / bc2;
      pp[k] = pp[k] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (model_out) {
      if (kOutF32) reinterpret_cast<float4*>(model_out)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      else reinterpret_cast<uint2*>(model_out)[i] = make_uint2(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]));
    }
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = nvec * 4 + threadIdx.x;
    const float gk = (kGradF32 ? reinterpret_cast<const float*>(grad)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i])) * gs;
    const float mk = b1 * m[i] + (1.f - b1) * gk, vk = b2 * v[i] + (1.f - b2) * gk * gk;
    const float pk = master[i] * (1.f - lr * wd) - lr * (mk / bc1) / (sqrtf(vk / bc2) + eps);
    m[i] = mk; v[i] = vk; master[i] = pk;
    if (model_out) {
      if (kOutF32) reinterpret_cast<float*>(model_out)[i] = pk;
      else reinterpret_cast<__nv_bfloat16*>(model_out)[i] = __float2bfloat16(pk);
    }
  }
}

// sum of squares of a flat buffer, accumulated into out[0]; out[1] counts non-finite values.
template <bool kF32>
__global__ void __launch_bounds__(256) sumsq_kernel(const void* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[8], redbad[8];
  float acc = 0.f, bad = 0.f;
  const long long nvec = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    load_logits8<kF32>(x, i * 8, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) { acc += f[k] * f[k]; if (!isfinite(f[k])) bad += 1.f; }
  }
  if (blockIdx.x == 0) {
    for (long long i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float f = kF32 ? reinterpret_cast<const float*>(x)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
      acc += f * f;
      if (!isfinite(f)) bad += 1.f;
    }
  }
  acc = warp_sum(acc); bad = warp_sum(bad);
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = acc; redbad[threadIdx.x >> 5] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f, b = 0.f;
    for (int w = 0; w < 8; ++w) { t += red[w]; b += redbad[w]; }
    atomicAdd(out, t);
    if (b != 0.f) atomicAdd(out + 1, b);
  }
}

// clip coefficient from an accumulated squared norm:  scale_out = base_scale * min(1, max_norm / (sqrt(sumsq)*base_scale + 1e-6));
// skip_out = 1 when the norm is not finite.  norm_out receives the (unscaled-by-clip) gradient norm.
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float base_scale, float max_norm,
                                 float* __restrict__ scale_out, int* __restrict__ skip_out, float* __restrict__ norm_out) {
  const float norm = sqrtf(sumsq[0]) * base_scale;
  const bool bad = !isfinite(norm) || sumsq[1] != 0.f;
  float coef = 1.f;
  if (max_norm > 0.f && norm > max_norm) coef = max_norm / (norm + 1e-6f);
  scale_out[0] = bad ? 0.f : base_scale * coef;
  if (skip_out) skip_out[0] = bad ? 1 : 0;
  if (norm_out) norm_out[0] = norm;
}

// -------------------------------------------------------------------------------------------------
// Embedding: out[t, :] = sum_k table_k[idx_k[t], :]  (word + position + token-type), rows outside
// [vocab_start, vocab_start+rows) contribute zero (vocab-parallel).  Backward scatter-adds into
// fp32 gradient tables.
// -------------------------------------------------------------------------------------------------
struct EmbedTables {
  const __nv_bfloat16* table[3];
  const long long* idx[3];
  int rows[3];
  int start[3];
  int count;
};

__global__ void __launch_bounds__(128)
embedding_fwd_kernel(EmbedTables t, __nv_bfloat16* __restrict__ out, long long T, int H) {
  const int nvec = H / 8;
  for (long long tok = blockIdx.x; tok < T; tok += gridDim.x) {
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < t.count; ++k) {
        const long long id = t.idx[k][tok] - t.start[k];
        if (id < 0 || id >= t.rows[k]) continue;
        const uint4 u = *reinterpret_cast<const uint4*>(t.table[k] + id * H + vi * 8);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack_bf16x2(w[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
      *reinterpret_cast<uint4*>(out + tok * H + vi * 8) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
}

template <bool kGradF32>
__global__ void __launch_bounds__(128)
embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ idx, void* __restrict__ dtable,
                     long long T, int H, int rows, int start) {
  for (long long tok = blockIdx.x; tok < T; tok += gridDim.x) {
    const long long id = idx[tok] - start;
    if (id < 0 || id >= rows) continue;
    for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
      const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + tok * H + c));
      if (kGradF32) {
        float* d = reinterpret_cast<float*>(dtable) + id * H + c;
        atomicAdd(d, g.x);
        atomicAdd(d + 1, g.y);
      } else {
        atomicAdd(reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(dtable) + id * H + c),
                  __floats2bfloat162_rn(g.x, g.y));
      }
    }
  }
}

// -------------------------------------------------------------------------------------------------
// Rotary position embedding on [B, L, H, D] (rotate-half convention), in place or out of place.
// `inverse` applies the transposed rotation (backward pass).  cos/sin are fp32 [L_max, D/2].
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, const float* __restrict__ cosb,
            const float* __restrict__ sinb, const long long* __restrict__ pos, long long B, int L, int H, int D,
            long long sb, long long ss, long long sh, long long ysb, long long yss, long long ysh, int inverse) {
  const int half = D / 2;
  const long long total = B * L * H * (long long)(half / 2);   // two rotation pairs per thread
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int pj = (int)(i % (half / 2)) * 2;
    long long r = i / (half / 2);
    const int h = (int)(r % H); r /= H;
    const int l = (int)(r % L);
    const long long b = r / L;
    const long long p = pos ? pos[b * L + l] : l;
    const __nv_bfloat16* src = x + b * sb + l * ss + h * sh;
    __nv_bfloat16* dst = y + b * ysb + l * yss + h * ysh;
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + pj));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + half + pj));
    const float2 c = *reinterpret_cast<const float2*>(cosb + p * half + pj);
    float2 s = *reinterpret_cast<const float2*>(sinb + p * half + pj);
    if (inverse) { s.x = -s.x; s.y = -s.y; }
    *reinterpret_cast<__nv_bfloat162*>(dst + pj) = __floats2bfloat162_rn(lo.x * c.x - hi.x * s.x, lo.y * c.y - hi.y * s.y);
    *reinterpret_cast<__nv_bfloat162*>(dst + half + pj) = __floats2bfloat162_rn(hi.x * c.x + lo.x * s.x, hi.y * c.y + lo.y * s.y);
  }
}

// 16-byte variant: a thread rotates 8 (low, high) pairs; needs D % 16 == 0 and 16-byte aligned rows.
__global__ void __launch_bounds__(256)
rope_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, const float* __restrict__ cosb,
                const float* __restrict__ sinb, const long long* __restrict__ pos, long long B, int L, int H, int D,
                long long sb, long long ss, long long sh, long long ysb, long long yss, long long ysh, int inverse) {
  const int half = D / 2;
  const int groups = half / 8;
  const long long total = B * L * H * (long long)groups;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int pj = (int)(i % groups) * 8;
    long long r = i / groups;
    const int h = (int)(r % H); r /= H;
    const int l = (int)(r % L);
    const long long b = r / L;
    const long long p = pos ? pos[b * L + l] : l;
    const __nv_bfloat16* src = x + b * sb + l * ss + h * sh;
    __nv_bfloat16* dst = y + b * ysb + l * yss + h * ysh;
    const uint4 lo4 = *reinterpret_cast<const uint4*>(src + pj);
    const uint4 hi4 = *reinterpret_cast<const uint4*>(src + half + pj);
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cosb + p * half + pj));
    const float4 c1 = __ldg(reinterpret_cast<const float4*>(cosb + p * half + pj) + 1);
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sinb + p * half + pj));
    const float4 s1 = __ldg(reinterpret_cast<const float4*>(sinb + p * half + pj) + 1);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    if (inverse) {
#pragma unroll
      for (int k = 0; k < 8; ++k) sn[k] = -sn[k];
    }
    const uint32_t lw[4] = {lo4.x, lo4.y, lo4.z, lo4.w}, hw[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 lo = unpack_bf16x2(lw[k]), hi = unpack_bf16x2(hw[k]);
      ol[k] = pack_bf16x2(lo.x * c[2 * k] - hi.x * sn[2 * k], lo.y * c[2 * k + 1] - hi.y * sn[2 * k + 1]);
      oh[k] = pack_bf16x2(hi.x * c[2 * k] + lo.x * sn[2 * k], hi.y * c[2 * k + 1] + lo.y * sn[2 * k + 1]);
    }
    *reinterpret_cast<uint4*>(dst + pj) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
    *reinterpret_cast<uint4*>(dst + half + pj) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
}

// -------------------------------------------------------------------------------------------------
// SwiGLU on a fused [M, 2F] gate|up tensor:  out = silu(gate) * up ;  backward writes [M, 2F].
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long M, int F, long long ld) {
  const int nvec = F / 8;
  const long long total = M * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / nvec;
    const int c = (int)(i % nvec) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + row * ld + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + row * ld + F + c);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = unpack_bf16x2(gw[k]), u = unpack_bf16x2(uw[k]);
      o[k] = pack_bf16x2(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + row * F + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                  __nv_bfloat16* __restrict__ dgu, long long M, int F, long long ld) {
  const int nvec = F / 8;
  const long long total = M * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / nvec;
    const int c = (int)(i % nvec) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + row * ld + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + row * ld + F + c);
    const uint4 d4 = *reinterpret_cast<const uint4*>(dout + row * F + c);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w}, dw[4] = {d4.x, d4.y, d4.z, d4.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = unpack_bf16x2(gw[k]), u = unpack_bf16x2(uw[k]), d = unpack_bf16x2(dw[k]);
      const float sx = 1.f / (1.f + __expf(-g.x)), sy = 1.f / (1.f + __expf(-g.y));
      og[k] = pack_bf16x2(d.x * u.x * sx * (1.f + g.x * (1.f - sx)), d.y * u.y * sy * (1.f + g.y * (1.f - sy)));
      ou[k] = pack_bf16x2(d.x * g.x * sx, d.y * g.y * sy);
    }
    *reinterpret_cast<uint4*>(dgu + row * ld + c) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dgu + row * ld + F + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// -------------------------------------------------------------------------------------------------
// Column sums of a [M, N] bf16 matrix into fp32 (bias gradients): out[n] (+)= sum_m x[m, n].
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, long long M, int N, long long ld, int rows_per_block) {
  // block = 32 column-pairs x 8 row lanes
  const int cp = blockIdx.x * 32 + (threadIdx.x & 31);     // column pair index
  const int rl = threadIdx.x >> 5;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  float a = 0.f, b = 0.f;
  if (cp * 2 < N) {
    for (long long r = r0 + rl; r < r1; r += 8) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + r * ld + cp * 2));
      a += f.x; b += f.y;
    }
  }
  __shared__ float sa[8][33], sb2[8][33];
  sa[rl][threadIdx.x & 31] = a; sb2[rl][threadIdx.x & 31] = b;
  __syncthreads();
  if (rl == 0 && cp * 2 < N) {
    for (int k = 1; k < 8; ++k) { a += sa[k][threadIdx.x & 31]; b += sb2[k][threadIdx.x & 31]; }
    atomicAdd(out + cp * 2, a);
    if (cp * 2 + 1 < N) atomicAdd(out + cp * 2 + 1, b);
  }
}

// Same reduction with 16-byte loads: thread = 8 columns, block = 256 columns x 8 row lanes.
__global__ void __launch_bounds__(256)
colsum_vec_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, long long M, int N, long long ld,
                  int rows_per_block) {
  const int cg = blockIdx.x * 32 + (threadIdx.x & 31);     // group of 8 columns
  const int rl = threadIdx.x >> 5;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  const bool live = cg * 8 < N;
  if (live) {
    const __nv_bfloat16* base = x + cg * 8;
    long long r = r0 + rl;
    for (; r + 24 < r1; r += 32) {
      uint4 u[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) u[q] = __ldg(reinterpret_cast<const uint4*>(base + (r + 8 * q) * ld));
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t w[4] = {u[q].x, u[q].y, u[q].z, u[q].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
      }
    }
    for (; r < r1; r += 8) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(base + r * ld));
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
    }
  }
  __shared__ float red[8][32][9];
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rl][threadIdx.x & 31][k] = acc[k];
  __syncthreads();
  // 256 threads finish the 256 columns of the block: thread t sums column t over the 8 row lanes
  const int col = threadIdx.x;
  float t = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) t += red[k][col >> 3][col & 7];
  const int gcol = blockIdx.x * 256 + col;
  if (gcol < N) atomicAdd(out + gcol, t);
}

// -------------------------------------------------------------------------------------------------
// Activation between the two GEMMs of an MLP, outside the GEMMs.  Evaluating erf-GELU in the GEMM
// epilogue made the eight epilogue warps the bottleneck of a K = 1024 GEMM (0.218 ms with the
// activation and the saved pre-activation against 0.116 ms with the bias only, 16384 x 4096 x 1024);
// as a pass of its own it runs at memory speed.  The backward pass multiplies the incoming gradient
// by act'(h) and, while the values are in registers, adds their column sums (the bias gradient of the
// first GEMM) into `colsum_out`: the layout is the column-sum kernel's.
// -------------------------------------------------------------------------------------------------
template <int kAct>
__global__ void __launch_bounds__(256)
act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      o[k] = pack_bf16x2(apply_act<kAct>(f.x), apply_act<kAct>(f.y));
    }
    reinterpret_cast<uint4*>(y)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int kAct>
__global__ void __launch_bounds__(256)
act_bwd_colsum_kernel(const __nv_bfloat16* __restrict__ d, const __nv_bfloat16* __restrict__ h,
                      __nv_bfloat16* __restrict__ out, float* __restrict__ colsum_out, long long M, int N, long long ld,
                      int rows_per_block) {
  const int cg = blockIdx.x * 32 + (threadIdx.x & 31);     // group of 8 columns
  const int rl = threadIdx.x >> 5;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (cg * 8 < N) {
    for (long long r = r0 + rl; r < r1; r += 16) {
      // two rows in flight per thread
      const long long ra = r, rb = r + 8;
      const bool has_b = rb < r1;
      const uint4 da = __ldg(reinterpret_cast<const uint4*>(d + ra * ld + cg * 8));
      const uint4 ha = __ldg(reinterpret_cast<const uint4*>(h + ra * ld + cg * 8));
      uint4 db = make_uint4(0, 0, 0, 0), hb = make_uint4(0, 0, 0, 0);
      if (has_b) {
        db = __ldg(reinterpret_cast<const uint4*>(d + rb * ld + cg * 8));
        hb = __ldg(reinterpret_cast<const uint4*>(h + rb * ld + cg * 8));
      }
      const uint32_t dwa[4] = {da.x, da.y, da.z, da.w}, hwa[4] = {ha.x, ha.y, ha.z, ha.w};
      const uint32_t dwb[4] = {db.x, db.y, db.z, db.w}, hwb[4] = {hb.x, hb.y, hb.z, hb.w};
      uint32_t oa[4], ob[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 g = unpack_bf16x2(dwa[e]), z = unpack_bf16x2(hwa[e]);
        const float v0 = g.x * apply_act_grad<kAct>(z.x), v1 = g.y * apply_act_grad<kAct>(z.y);
        oa[e] = pack_bf16x2(v0, v1);
        const float2 q = unpack_bf16x2(oa[e]);        // the sum is over the rounded values the next GEMM reads
        acc[2 * e] += q.x; acc[2 * e + 1] += q.y;
      }
      *reinterpret_cast<uint4*>(out + ra * ld + cg * 8) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
      if (has_b) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 g = unpack_bf16x2(dwb[e]), z = unpack_bf16x2(hwb[e]);
          const float v0 = g.x * apply_act_grad<kAct>(z.x), v1 = g.y * apply_act_grad<kAct>(z.y);
          ob[e] = pack_bf16x2(v0, v1);
          const float2 q = unpack_bf16x2(ob[e]);
          acc[2 * e] += q.x; acc[2 * e + 1] += q.y;
        }
        *reinterpret_cast<uint4*>(out + rb * ld + cg * 8) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
      }
    }
  }
  if (colsum_out == nullptr) return;
  __shared__ float red[8][32][9];
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rl][threadIdx.x & 31][k] = acc[k];
  __syncthreads();
  const int col = threadIdx.x;
  float t = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) t += red[k][col >> 3][col & 7];
  const int gcol = blockIdx.x * 256 + col;
  if (gcol < N) atomicAdd(colsum_out + gcol, t);
}

// -------------------------------------------------------------------------------------------------
// Dropout (forward, and backward with the regenerated mask), scaled casts.
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dropout_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n, float p,
               const unsigned long long* __restrict__ rng, unsigned long long call_id) {
  const unsigned long long seed = rng[0], offset = rng[1];
  const float ks = 1.f / (1.f - p);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n / 8; i += (long long)gridDim.x * blockDim.x) {
    float r[8];
    philox_uniform8(seed, offset + call_id, (unsigned long long)i * 8, r);
    const uint4 u = reinterpret_cast<const uint4*>(x)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      o[k] = pack_bf16x2(r[2 * k] < p ? 0.f : f.x * ks, r[2 * k + 1] < p ? 0.f : f.y * ks);
    }
    reinterpret_cast<uint4*>(y)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <bool kInF32, bool kOutF32>
__global__ void __launch_bounds__(256)
scaled_cast_kernel(const void* __restrict__ x, void* __restrict__ y, long long n, const float* __restrict__ scale_ptr,
                   float scale, int accumulate) {
  const float s = scale * (scale_ptr ? scale_ptr[0] : 1.f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = kInF32 ? reinterpret_cast<const float*>(x)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    v *= s;
    if (kOutF32) {
      float* d = reinterpret_cast<float*>(y) + i;
      *d = accumulate ? *d + v : v;
    } else {
      __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(y) + i;
      *d = __float2bfloat16(accumulate ? __bfloat162float(*d) + v : v);
    }
  }
}

}  // namespace mrk

using namespace mrk;

MRK_API int mrk_ce_stats(const void* logits, const long long* labels, float* stats, long long M, int V, long long ld,
                         int vocab_start, int ignore_index, int logits_f32, void* stream) {
  MRK_REQUIRE(M > 0 && V > 0, "cross entropy: empty input");
  MRK_REQUIRE(ld % 8 == 0, "cross entropy: row pitch must be a multiple of 8 elements");
  cudaStream_t s = (cudaStream_t)stream;
  if (logits_f32) ce_stats_kernel<true><<<(unsigned)M, kCeThreads, 0, s>>>(logits, labels, stats, M, V, ld, vocab_start, ignore_index);
  else ce_stats_kernel<false><<<(unsigned)M, kCeThreads, 0, s>>>(logits, labels, stats, M, V, ld, vocab_start, ignore_index);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_ce_finalize(const float* stats, int tp_parts, long long part_stride, const long long* labels, float* lse,
                            float* loss_rows, float* loss_sum, float* valid_count, long long M, int ignore_index,
                            void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  ce_finalize_kernel<<<(unsigned)((M + 255) / 256), 256, 0, s>>>(stats, tp_parts, part_stride, labels, lse, loss_rows,
                                                                  loss_sum, valid_count, M, ignore_index);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_ce_grad(const void* logits, const long long* labels, const float* lse, const float* grad_scale,
                        void* dlogits, long long M, int V, long long ld, long long ldd, int vocab_start,
                        int ignore_index, int logits_f32, void* stream) {
  MRK_REQUIRE(ld % 8 == 0 && ldd % 8 == 0, "cross entropy: row pitch must be a multiple of 8 elements");
  cudaStream_t s = (cudaStream_t)stream;
  if (logits_f32) ce_grad_kernel<true><<<(unsigned)M, kCeThreads, 0, s>>>(logits, labels, lse, grad_scale, dlogits, M, V, ld, ldd, vocab_start, ignore_index);
  else ce_grad_kernel<false><<<(unsigned)M, kCeThreads, 0, s>>>(logits, labels, lse, grad_scale, dlogits, M, V, ld, ldd, vocab_start, ignore_index);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_adamw(float* master, float* m, float* v, const void* grad, void* model_out, const float* hp,
                      const float* grad_scale, const int* skip, long long n, int grad_f32, int out_f32, void* stream) {
  MRK_REQUIRE(n > 0, "adamw: empty buffer");
  MRK_REQUIRE(((uintptr_t)master & 15) == 0 && ((uintptr_t)m & 15) == 0 && ((uintptr_t)v & 15) == 0 &&
              ((uintptr_t)grad & (grad_f32 ? 15 : 7)) == 0 && ((uintptr_t)model_out & (out_f32 ? 15 : 7)) == 0,
              "adamw: buffers must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = grid_for(n / 4 + 1, 256, 8);
  if (grad_f32 && out_f32) adamw_kernel<true, true><<<grid, 256, 0, s>>>(master, m, v, grad, model_out, hp, grad_scale, skip, n);
  else if (grad_f32) adamw_kernel<true, false><<<grid, 256, 0, s>>>(master, m, v, grad, model_out, hp, grad_scale, skip, n);
  else if (out_f32) adamw_kernel<false, true><<<grid, 256, 0, s>>>(master, m, v, grad, model_out, hp, grad_scale, skip, n);
  else adamw_kernel<false, false><<<grid, 256, 0, s>>>(master, m, v, grad, model_out, hp, grad_scale, skip, n);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_sumsq(const void* x, long long n, float* out2, int is_f32, void* stream) {
  MRK_REQUIRE(((uintptr_t)x & 15) == 0, "sumsq: buffer must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = grid_for(n / 8 + 1, 256, 4);
  if (is_f32) sumsq_kernel<true><<<grid, 256, 0, s>>>(x, n, out2);
  else sumsq_kernel<false><<<grid, 256, 0, s>>>(x, n, out2);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_clip_coef(const float* sumsq2, float base_scale, float max_norm, float* scale_out, int* skip_out,
                          float* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sumsq2, base_scale, max_norm, scale_out, skip_out, norm_out);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_embedding_fwd(const void* const* tables, const long long* const* idx, const int* rows, const int* starts,
                              int count, void* out, long long T, int H, void* stream) {
  MRK_REQUIRE(count >= 1 && count <= 3 && H % 8 == 0, "embedding: bad arguments");
  EmbedTables t;
  t.count = count;
  for (int k = 0; k < 3; ++k) {
    t.table[k] = k < count ? (const __nv_bfloat16*)tables[k] : nullptr;
    t.idx[k] = k < count ? idx[k] : nullptr;
    t.rows[k] = k < count ? rows[k] : 0;
    t.start[k] = k < count ? starts[k] : 0;
  }
  const long long cap = (long long)sm_count() * 16;
  embedding_fwd_kernel<<<(unsigned)(T < cap ? T : cap), 128, 0, (cudaStream_t)stream>>>(t, (__nv_bfloat16*)out, T, H);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_embedding_bwd(const void* dout, const long long* idx, void* dtable, long long T, int H, int rows,
                              int start, int grad_f32, void* stream) {
  MRK_REQUIRE(H % 2 == 0, "embedding: hidden size must be even");
  const long long cap = (long long)sm_count() * 16;
  const unsigned grid = (unsigned)(T < cap ? T : cap);
  if (grad_f32) embedding_bwd_kernel<true><<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dout, idx, dtable, T, H, rows, start);
  else embedding_bwd_kernel<false><<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dout, idx, dtable, T, H, rows, start);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_rope(const void* x, void* y, const float* cosb, const float* sinb, const long long* pos, long long B,
                     int L, int H, int D, long long sb, long long ss, long long sh, long long ysb, long long yss,
                     long long ysh, int inverse, void* stream) {
  MRK_REQUIRE(D % 4 == 0, "rope: head dim must be a multiple of 4");
  const bool vec = D % 16 == 0 && ((sb | ss | sh | ysb | yss | ysh) % 8) == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0 &&
                   (((uintptr_t)cosb | (uintptr_t)sinb) & 15) == 0;
  if (vec) {
    const long long total8 = B * L * H * (long long)(D / 16);
    rope_vec_kernel<<<grid_for(total8, 256, 8), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)y, cosb, sinb, pos, B, L, H, D, sb, ss, sh, ysb, yss, ysh, inverse);
    MRK_CHECK_LAUNCH();
    return 0;
  }
  const long long total = B * L * H * (long long)(D / 4);
  rope_kernel<<<grid_for(total, 256, 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, cosb, sinb, pos, B, L, H, D, sb, ss, sh, ysb, yss, ysh, inverse);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_swiglu_fwd(const void* gu, void* out, long long M, int F, long long ld, void* stream) {
  MRK_REQUIRE(F % 8 == 0 && ld % 8 == 0, "swiglu: sizes must be multiples of 8");
  swiglu_fwd_kernel<<<grid_for(M * (F / 8), 256, 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, M, F, ld);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long M, int F, long long ld, void* stream) {
  MRK_REQUIRE(F % 8 == 0 && ld % 8 == 0, "swiglu: sizes must be multiples of 8");
  swiglu_bwd_kernel<<<grid_for(M * (F / 8), 256, 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, M, F, ld);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_act_fwd(const void* x, void* y, long long n, int act, void* stream) {
  MRK_REQUIRE(n % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0, "act_fwd: needs 16-byte vectors");
  const long long nvec = n / 8;
  const dim3 grid = grid_for(nvec, 256, 8);
  cudaStream_t s = (cudaStream_t)stream;
  const __nv_bfloat16* xi = (const __nv_bfloat16*)x;
  __nv_bfloat16* yo = (__nv_bfloat16*)y;
  switch (act) {
    case MRK_ACT_GELU_ERF: act_fwd_kernel<MRK_ACT_GELU_ERF><<<grid, 256, 0, s>>>(xi, yo, nvec); break;
    case MRK_ACT_GELU_TANH: act_fwd_kernel<MRK_ACT_GELU_TANH><<<grid, 256, 0, s>>>(xi, yo, nvec); break;
    case MRK_ACT_RELU: act_fwd_kernel<MRK_ACT_RELU><<<grid, 256, 0, s>>>(xi, yo, nvec); break;
    case MRK_ACT_SILU: act_fwd_kernel<MRK_ACT_SILU><<<grid, 256, 0, s>>>(xi, yo, nvec); break;
    default: MRK_REQUIRE(false, "act_fwd: unknown activation %d", act);
  }
  MRK_CHECK_LAUNCH();
  return 0;
}

// out[M,N] = d[M,N] * act'(h[M,N]) (all bf16 with row pitch `ld`; `out` may alias `d`); the column sums of
// `out` are ADDED into colsum_out[N] (fp32) when it is given.
MRK_API int mrk_act_bwd(const void* d, const void* h, void* out, float* colsum_out, long long M, int N, long long ld,
                        int act, void* stream) {
  MRK_REQUIRE(N % 8 == 0 && ld % 8 == 0 && ((uintptr_t)d & 15) == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)out & 15) == 0,
              "act_bwd: needs 16-byte vectors");
  const int col_blocks = (N / 8 + 31) / 32;
  int row_blocks = (int)((long long)sm_count() * 8 / col_blocks);
  if (row_blocks < 1) row_blocks = 1;
  long long rpb = (M + row_blocks - 1) / row_blocks;
  rpb = (rpb + 15) / 16 * 16;
  row_blocks = (int)((M + rpb - 1) / rpb);
  dim3 grid(col_blocks, row_blocks);
  cudaStream_t s = (cudaStream_t)stream;
  const __nv_bfloat16 *di = (const __nv_bfloat16*)d, *hi = (const __nv_bfloat16*)h;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
  switch (act) {
    case MRK_ACT_GELU_ERF: act_bwd_colsum_kernel<MRK_ACT_GELU_ERF><<<grid, 256, 0, s>>>(di, hi, oo, colsum_out, M, N, ld, (int)rpb); break;
    case MRK_ACT_GELU_TANH: act_bwd_colsum_kernel<MRK_ACT_GELU_TANH><<<grid, 256, 0, s>>>(di, hi, oo, colsum_out, M, N, ld, (int)rpb); break;
    case MRK_ACT_RELU: act_bwd_colsum_kernel<MRK_ACT_RELU><<<grid, 256, 0, s>>>(di, hi, oo, colsum_out, M, N, ld, (int)rpb); break;
    case MRK_ACT_SILU: act_bwd_colsum_kernel<MRK_ACT_SILU><<<grid, 256, 0, s>>>(di, hi, oo, colsum_out, M, N, ld, (int)rpb); break;
    default: MRK_REQUIRE(false, "act_bwd: unknown activation %d", act);
  }
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_colsum(const void* x, float* out, long long M, int N, long long ld, void* stream) {
  MRK_REQUIRE(N % 2 == 0 && ld % 2 == 0, "colsum: N must be even");
  if (ld % 8 == 0 && ld >= (N + 7) / 8 * 8 && ((uintptr_t)x & 15) == 0) {
    // (a ragged last group of columns is read up to the row pitch and only its valid columns are added)
    // 16-byte loads: a block covers 256 columns x its row range, 8 row lanes, 4 rows in flight per thread
    const int col_blocks = (N / 8 + 31) / 32;
    int row_blocks = (int)((long long)sm_count() * 8 / col_blocks);
    if (row_blocks < 1) row_blocks = 1;
    long long rpb = (M + row_blocks - 1) / row_blocks;
    rpb = (rpb + 31) / 32 * 32;
    row_blocks = (int)((M + rpb - 1) / rpb);
    dim3 grid(col_blocks, row_blocks);
    colsum_vec_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, out, M, N, ld, (int)rpb);
    MRK_CHECK_LAUNCH();
    return 0;
  }
  const int col_blocks = (N / 2 + 31) / 32;
  int row_blocks = (int)((long long)sm_count() * 4 / col_blocks);
  if (row_blocks < 1) row_blocks = 1;
  long long rpb = (M + row_blocks - 1) / row_blocks;
  rpb = (rpb + 7) / 8 * 8;
  row_blocks = (int)((M + rpb - 1) / rpb);
  dim3 grid(col_blocks, row_blocks);
  colsum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, out, M, N, ld, (int)rpb);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_dropout(const void* x, void* y, long long n, float p, const void* rng, unsigned long long call_id, void* stream) {
  MRK_REQUIRE(n % 8 == 0, "dropout: element count must be a multiple of 8");
  dropout_kernel<<<grid_for(n / 8, 256, 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, p, (const unsigned long long*)rng, call_id);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_scaled_cast(const void* x, void* y, long long n, const float* scale_ptr, float scale, int in_f32,
                            int out_f32, int accumulate, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = grid_for(n, 256, 8);
  if (in_f32 && out_f32) scaled_cast_kernel<true, true><<<grid, 256, 0, s>>>(x, y, n, scale_ptr, scale, accumulate);
  else if (in_f32) scaled_cast_kernel<true, false><<<grid, 256, 0, s>>>(x, y, n, scale_ptr, scale, accumulate);
  else if (out_f32) scaled_cast_kernel<false, true><<<grid, 256, 0, s>>>(x, y, n, scale_ptr, scale, accumulate);
  else scaled_cast_kernel<false, false><<<grid, 256, 0, s>>>(x, y, n, scale_ptr, scale, accumulate);
  MRK_CHECK_LAUNCH();
  return 0;
}
