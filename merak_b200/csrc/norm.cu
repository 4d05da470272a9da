// Fused (dropout +) residual-add + LayerNorm / RMSNorm, forward and backward.
//
//   z = dropout(x, p) + residual            (both optional)
//   y = (z - mean) * rstd * gamma + beta    (LayerNorm)     or     z * rstd * gamma   (RMSNorm)
//
// One pass over HBM per direction: the row lives in registers between the statistics and the
// normalisation; the dropout mask is regenerated from a counter-based generator in the backward
// pass instead of being stored.  Replaces torch.nn.LayerNorm / LlamaRMSNorm and the separate
// dropout + residual kernels of the reference's blocks
// (Merak/core/tensor_parallel/transformer_blocks.py:34-42).
#include "elementwise.h"
#include "host_common.h"
#include "philox.cuh"
#include "sm100_ptx.cuh"

namespace mrk {


template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) t += red[w];
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                            pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
// gamma/beta may be bf16 or fp32
__device__ __forceinline__ void load8p(const void* p, int idx, bool f32, float (&f)[8]) {
  if (f32) load8f(reinterpret_cast<const float*>(p) + idx, f);
  else load8(reinterpret_cast<const __nv_bfloat16*>(p) + idx, f);
}

struct NormFwdParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* residual;   // optional
  const void* gamma;
  const void* beta;                // optional (nullptr for RMSNorm)
  __nv_bfloat16* y;
  __nv_bfloat16* z;                // optional: pre-norm sum (needed when residual/dropout is used)
  float* mean;                     // optional (LayerNorm)
  float* rstd;
  const unsigned long long* rng;   // [seed, offset] on device; nullptr = no dropout
  unsigned long long call_id;
  float p_drop;
  float eps;
  long long M;
  int H;
  int rms;
  int params_f32;
};

constexpr int kNormSlots = 32;     // accumulator rows of the weight / bias gradient partial sums

__device__ __forceinline__ void red_add_f4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int THREADS, int kMaxVecPerThread>
__global__ void __launch_bounds__(THREADS) norm_fwd_kernel(const NormFwdParams p) {
  __shared__ float red[THREADS / 32];
  const int nvec = p.H / 8;
  const bool drop = p.rng != nullptr && p.p_drop > 0.f;
  const float keep_scale = drop ? 1.f / (1.f - p.p_drop) : 1.f;
  unsigned long long seed = 0, offset = 0;
  if (drop) { seed = p.rng[0]; offset = p.rng[1]; }
  for (long long row = blockIdx.x; row < p.M; row += gridDim.x) {
    float v[kMaxVecPerThread][8];
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < kMaxVecPerThread; ++it) {
      const int vi = threadIdx.x + it * THREADS;
      if (vi < nvec) {
        load8(p.x + row * p.H + vi * 8, v[it]);
        if (drop) {
          const unsigned long long e = (unsigned long long)row * p.H + (unsigned long long)vi * 8;
          float r[8];
          philox_uniform8(seed, offset + p.call_id, e, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[it][i] = r[i] < p.p_drop ? 0.f : v[it][i] * keep_scale;
        }
        if (p.residual) {
          float r[8];
          load8(p.residual + row * p.H + vi * 8, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[it][i] += r[i];
        }
        if (p.z) {
          store8(p.z + row * p.H + vi * 8, v[it]);
          // statistics are taken on the rounded values the backward pass will read
#pragma unroll
          for (int i = 0; i < 8; ++i) v[it][i] = __bfloat162float(__float2bfloat16(v[it][i]));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += p.rms ? v[it][i] * v[it][i] : v[it][i];
      }
    }
    float mean = 0.f, rstd;
    if (p.rms) {
      const float ms = block_sum<THREADS>(sum, red) / p.H;
      rstd = rsqrtf(ms + p.eps);
    } else {
      mean = block_sum<THREADS>(sum, red) / p.H;
      float sq = 0.f;
#pragma unroll
      for (int it = 0; it < kMaxVecPerThread; ++it) {
        const int vi = threadIdx.x + it * THREADS;
        if (vi < nvec) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { const float d = v[it][i] - mean; sq += d * d; }
        }
      }
      const float var = block_sum<THREADS>(sq, red) / p.H;
      rstd = rsqrtf(var + p.eps);
    }
    if (threadIdx.x == 0) {
      if (p.mean) p.mean[row] = mean;
      if (p.rstd) p.rstd[row] = rstd;
    }
#pragma unroll
    for (int it = 0; it < kMaxVecPerThread; ++it) {
      const int vi = threadIdx.x + it * THREADS;
      if (vi < nvec) {
        float g[8], o[8];
        load8p(p.gamma, vi * 8, p.params_f32, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[it][i] - mean) * rstd * g[i];
        if (p.beta) {
          float bb[8];
          load8p(p.beta, vi * 8, p.params_f32, bb);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += bb[i];
        }
        store8(p.y + row * p.H + vi * 8, o);
      }
    }
  }
}

struct NormBwdParams {
  const __nv_bfloat16* dy;
  const __nv_bfloat16* z;          // input of the norm (x + residual after dropout)
  const __nv_bfloat16* dz_extra;   // optional gradient arriving on the residual stream
  const void* gamma;
  const float* mean;               // nullptr for RMSNorm
  const float* rstd;
  __nv_bfloat16* dres;             // gradient wrt z (residual branch); may alias dx when no dropout
  __nv_bfloat16* dx;               // optional: gradient wrt x (through dropout)
  float* dgamma;                   // fp32 [H]: written by the reduction over `partial`
  float* dbeta;                    // optional
  float* partial;                  // workspace [gridDim.x][2][H]: per-block partial sums
  const unsigned long long* rng;
  unsigned long long call_id;
  float p_drop;
  long long M;
  int H;
  int rms;
  int params_f32;
};

template <int THREADS, int kMaxVecPerThread>
__global__ void __launch_bounds__(THREADS, (THREADS == 128 && kMaxVecPerThread == 1) ? 8 : 1)
norm_bwd_kernel(const NormBwdParams p) {
  __shared__ float red[THREADS / 32];
  const int nvec = p.H / 8;
  const bool drop = p.rng != nullptr && p.p_drop > 0.f && p.dx != nullptr;
  const float keep_scale = drop ? 1.f / (1.f - p.p_drop) : 1.f;
  unsigned long long seed = 0, offset = 0;
  if (drop) { seed = p.rng[0]; offset = p.rng[1]; }
  float dg[kMaxVecPerThread][8], db[kMaxVecPerThread][8];
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it)
#pragma unroll
    for (int i = 0; i < 8; ++i) { dg[it][i] = 0.f; db[it][i] = 0.f; }

  // The loads of the next row are issued before the reductions of the current one, so a block keeps
  // two rows in flight instead of stalling on DRAM between its block-wide sums.
  uint4 raw_dy[kMaxVecPerThread], raw_z[kMaxVecPerThread];
  auto fetch = [&](long long row) {
#pragma unroll
    for (int it = 0; it < kMaxVecPerThread; ++it) {
      const int vi = threadIdx.x + it * THREADS;
      if (vi < nvec && row < p.M) {
        raw_dy[it] = __ldg(reinterpret_cast<const uint4*>(p.dy + row * p.H + vi * 8));
        raw_z[it] = __ldg(reinterpret_cast<const uint4*>(p.z + row * p.H + vi * 8));
      }
    }
  };
  auto unpack8 = [](const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = unpack_bf16x2(w[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  };
  fetch(blockIdx.x);
  for (long long row = blockIdx.x; row < p.M; row += gridDim.x) {
    const float mean = p.mean ? p.mean[row] : 0.f;
    const float rstd = p.rstd[row];
    float xh[kMaxVecPerThread][8], dxh[kMaxVecPerThread][8];
    float s1 = 0.f, s2 = 0.f;
    float dyv_all[kMaxVecPerThread][8];
#pragma unroll
    for (int it = 0; it < kMaxVecPerThread; ++it) {
      const int vi = threadIdx.x + it * THREADS;
      if (vi < nvec) { unpack8(raw_dy[it], dyv_all[it]); unpack8(raw_z[it], xh[it]); }
    }
    fetch(row + gridDim.x);
#pragma unroll
    for (int it = 0; it < kMaxVecPerThread; ++it) {
      const int vi = threadIdx.x + it * THREADS;
      if (vi < nvec) {
        float g[8];
        float (&dyv)[8] = dyv_all[it];
        load8p(p.gamma, vi * 8, p.params_f32, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[it][i] = (xh[it][i] - mean) * rstd;
          dxh[it][i] = dyv[i] * g[i];
          dg[it][i] += dyv[i] * xh[it][i];
          db[it][i] += dyv[i];
          s1 += dxh[it][i];
          s2 += dxh[it][i] * xh[it][i];
        }
      }
    }
    if (p.rms) s1 = 0.f; else s1 = block_sum<THREADS>(s1, red) / p.H;
    s2 = block_sum<THREADS>(s2, red) / p.H;
#pragma unroll
    for (int it = 0; it < kMaxVecPerThread; ++it) {
      const int vi = threadIdx.x + it * THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (dxh[it][i] - s1 - xh[it][i] * s2);
        if (p.dz_extra) {
          float e[8];
          load8(p.dz_extra + row * p.H + vi * 8, e);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += e[i];
        }
        if (p.dres) store8(p.dres + row * p.H + vi * 8, o);
        if (p.dx && p.dx != p.dres) {
          if (drop) {
            const unsigned long long e = (unsigned long long)row * p.H + (unsigned long long)vi * 8;
            float r[8];
            philox_uniform8(seed, offset + p.call_id, e, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = r[i] < p.p_drop ? 0.f : o[i] * keep_scale;
          }
          store8(p.dx + row * p.H + vi * 8, o);
        }
      }
    }
  }
  // every thread owns distinct columns: add this block's partial sums into one of kNormSlots
  // accumulator rows (zero before the launch); a second kernel sums the rows and clears them again
  float* pg = p.partial + (long long)(blockIdx.x % kNormSlots) * 2 * p.H;
#pragma unroll
  for (int it = 0; it < kMaxVecPerThread; ++it) {
    const int vi = threadIdx.x + it * THREADS;
    if (vi < nvec) {
      red_add_f4(pg + vi * 8, dg[it][0], dg[it][1], dg[it][2], dg[it][3]);
      red_add_f4(pg + vi * 8 + 4, dg[it][4], dg[it][5], dg[it][6], dg[it][7]);
      red_add_f4(pg + p.H + vi * 8, db[it][0], db[it][1], db[it][2], db[it][3]);
      red_add_f4(pg + p.H + vi * 8 + 4, db[it][4], db[it][5], db[it][6], db[it][7]);
    }
  }
}

// -------------------------------------------------------------------------------------------------
// One warp per row, for hidden sizes up to 1024 that are multiples of 256.  A lane holds V = H / 256
// vectors of 8 values; sums are warp shuffles, so no warp ever waits for another one (the block-wide
// kernels above spend most of a row at their barriers: 0.59 and 0.27 of the copy bandwidth at
// H = 1024).  Same arithmetic and the same dropout counters as the block-wide kernels.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

template <int V>
__global__ void __launch_bounds__(128) norm_fwd_warp_kernel(const NormFwdParams p) {
  const int lane = threadIdx.x & 31;
  const long long warp_id = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const long long n_warps = (long long)gridDim.x * 4;
  const bool drop = p.rng != nullptr && p.p_drop > 0.f;
  const float keep_scale = drop ? 1.f / (1.f - p.p_drop) : 1.f;
  unsigned long long seed = 0, offset = 0;
  if (drop) { seed = p.rng[0]; offset = p.rng[1]; }
  const float inv_h = 1.f / (float)p.H;
  // gamma / beta of this lane's columns stay in registers for all rows
  float g[V][8], bb[V][8];
#pragma unroll
  for (int it = 0; it < V; ++it) {
    load8p(p.gamma, (lane + 32 * it) * 8, p.params_f32, g[it]);
    if (p.beta) load8p(p.beta, (lane + 32 * it) * 8, p.params_f32, bb[it]);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) bb[it][i] = 0.f;
    }
  }
  for (long long row = warp_id; row < p.M; row += n_warps) {
    uint4 rx[V], rr[V];
#pragma unroll
    for (int it = 0; it < V; ++it) {
      rx[it] = __ldg(reinterpret_cast<const uint4*>(p.x + row * p.H + (lane + 32 * it) * 8));
      if (p.residual) rr[it] = __ldg(reinterpret_cast<const uint4*>(p.residual + row * p.H + (lane + 32 * it) * 8));
    }
    float v[V][8];
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < V; ++it) {
      const int vi = lane + 32 * it;
      const uint32_t w[4] = {rx[it].x, rx[it].y, rx[it].z, rx[it].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 t = unpack_bf16x2(w[i]); v[it][2 * i] = t.x; v[it][2 * i + 1] = t.y; }
      if (drop) {
        const unsigned long long e = (unsigned long long)row * p.H + (unsigned long long)vi * 8;
        float r[8];
        philox_uniform8(seed, offset + p.call_id, e, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[it][i] = r[i] < p.p_drop ? 0.f : v[it][i] * keep_scale;
      }
      if (p.residual) {
        const uint32_t q[4] = {rr[it].x, rr[it].y, rr[it].z, rr[it].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 t = unpack_bf16x2(q[i]); v[it][2 * i] += t.x; v[it][2 * i + 1] += t.y; }
      }
      if (p.z) {
        store8(p.z + row * p.H + vi * 8, v[it]);
        // statistics are taken on the rounded values the backward pass will read
#pragma unroll
        for (int i = 0; i < 8; ++i) v[it][i] = __bfloat162float(__float2bfloat16(v[it][i]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += p.rms ? v[it][i] * v[it][i] : v[it][i];
    }
    float mean = 0.f, rstd;
    if (p.rms) {
      rstd = rsqrtf(warp_sum(sum) * inv_h + p.eps);
    } else {
      mean = warp_sum(sum) * inv_h;
      float sq = 0.f;
#pragma unroll
      for (int it = 0; it < V; ++it)
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float d = v[it][i] - mean; sq += d * d; }
      rstd = rsqrtf(warp_sum(sq) * inv_h + p.eps);
    }
    if (lane == 0) {
      if (p.mean) p.mean[row] = mean;
      if (p.rstd) p.rstd[row] = rstd;
    }
#pragma unroll
    for (int it = 0; it < V; ++it) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = fmaf((v[it][i] - mean) * rstd, g[it][i], bb[it][i]);
      store8(p.y + row * p.H + (lane + 32 * it) * 8, o);
    }
  }
}

template <int V>
__global__ void __launch_bounds__(128) norm_bwd_warp_kernel(const NormBwdParams p) {
  __shared__ float red[4][2][V * 256 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp_id = (long long)blockIdx.x * 4 + warp;
  const long long n_warps = (long long)gridDim.x * 4;
  const bool drop = p.rng != nullptr && p.p_drop > 0.f && p.dx != nullptr;
  const float keep_scale = drop ? 1.f / (1.f - p.p_drop) : 1.f;
  unsigned long long seed = 0, offset = 0;
  if (drop) { seed = p.rng[0]; offset = p.rng[1]; }
  const float inv_h = 1.f / (float)p.H;
  float g[V][8], dg[V][8], db[V][8];
#pragma unroll
  for (int it = 0; it < V; ++it) {
    load8p(p.gamma, (lane + 32 * it) * 8, p.params_f32, g[it]);
#pragma unroll
    for (int i = 0; i < 8; ++i) { dg[it][i] = 0.f; db[it][i] = 0.f; }
  }
  for (long long row = warp_id; row < p.M; row += n_warps) {
    uint4 rdy[V], rz[V], rex[V];
#pragma unroll
    for (int it = 0; it < V; ++it) {
      const long long off = row * p.H + (lane + 32 * it) * 8;
      rdy[it] = __ldg(reinterpret_cast<const uint4*>(p.dy + off));
      rz[it] = __ldg(reinterpret_cast<const uint4*>(p.z + off));
      if (p.dz_extra) rex[it] = __ldg(reinterpret_cast<const uint4*>(p.dz_extra + off));
    }
    const float mean = p.mean ? p.mean[row] : 0.f;
    const float rstd = p.rstd[row];
    float xh[V][8], dxh[V][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < V; ++it) {
      const uint32_t wd[4] = {rdy[it].x, rdy[it].y, rdy[it].z, rdy[it].w};
      const uint32_t wz[4] = {rz[it].x, rz[it].y, rz[it].z, rz[it].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 d = unpack_bf16x2(wd[i]), z = unpack_bf16x2(wz[i]);
        const float dyv[2] = {d.x, d.y}, zv[2] = {z.x, z.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int k = 2 * i + e;
          xh[it][k] = (zv[e] - mean) * rstd;
          dxh[it][k] = dyv[e] * g[it][k];
          dg[it][k] += dyv[e] * xh[it][k];
          db[it][k] += dyv[e];
          s1 += dxh[it][k];
          s2 += dxh[it][k] * xh[it][k];
        }
      }
    }
    s1 = p.rms ? 0.f : warp_sum(s1) * inv_h;
    s2 = warp_sum(s2) * inv_h;
#pragma unroll
    for (int it = 0; it < V; ++it) {
      const int vi = lane + 32 * it;
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rstd * (dxh[it][i] - s1 - xh[it][i] * s2);
      if (p.dz_extra) {
        const uint32_t we[4] = {rex[it].x, rex[it].y, rex[it].z, rex[it].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 t = unpack_bf16x2(we[i]); o[2 * i] += t.x; o[2 * i + 1] += t.y; }
      }
      if (p.dres) store8(p.dres + row * p.H + vi * 8, o);
      if (p.dx && p.dx != p.dres) {
        if (drop) {
          const unsigned long long e = (unsigned long long)row * p.H + (unsigned long long)vi * 8;
          float r[8];
          philox_uniform8(seed, offset + p.call_id, e, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = r[i] < p.p_drop ? 0.f : o[i] * keep_scale;
        }
        store8(p.dx + row * p.H + vi * 8, o);
      }
    }
  }
  // the four warps of the block add up their partial sums in shared memory, then the block adds
  // them into one of kNormSlots accumulator rows (see norm_bwd_kernel)
#pragma unroll
  for (int it = 0; it < V; ++it)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      red[warp][0][(lane + 32 * it) * 8 + i] = dg[it][i];
      red[warp][1][(lane + 32 * it) * 8 + i] = db[it][i];
    }
  __syncthreads();
  float* pg = p.partial + (long long)(blockIdx.x % kNormSlots) * 2 * p.H;
  for (int c = threadIdx.x * 4; c < 2 * p.H; c += 128 * 4) {
    const int which = c / p.H, col = c % p.H;       // H is a multiple of 256: a group of 4 never straddles
    float t[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      t[k] = red[0][which][col + k] + red[1][which][col + k] + red[2][which][col + k] + red[3][which][col + k];
    red_add_f4(pg + which * p.H + col, t[0], t[1], t[2], t[3]);
  }
}

__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(float* __restrict__ partial, int blocks, int H, float* __restrict__ dgamma,
                       float* __restrict__ dbeta) {
  // grid.y = 0: gamma, 1: beta; 8 row-lanes x 32 columns per block
  const int col = blockIdx.x * 32 + (threadIdx.x & 31);
  const int rl = threadIdx.x >> 5;
  const int which = blockIdx.y;
  float* out = which == 0 ? dgamma : dbeta;     // may be null (RMSNorm has no bias): the rows are still cleared
  float acc = 0.f;
  if (col < H)
    for (int b = rl; b < blocks; b += 8) {
      float* slot = partial + ((long long)b * 2 + which) * H + col;
      acc += *slot;
      *slot = 0.f;            // leave the accumulator rows clean for the next call
    }
  __shared__ float sm[8][33];
  sm[rl][threadIdx.x & 31] = acc;
  __syncthreads();
  if (rl == 0 && col < H && out != nullptr) {
    for (int k = 1; k < 8; ++k) acc += sm[k][threadIdx.x & 31];
    out[col] = acc;
  }
}

}  // namespace mrk

using namespace mrk;

// Grid of the warp-per-row kernels: every block resident at once (blocks of 128 threads, no dynamic
// shared memory), or fewer when there is less work.  The occupancy query runs once per kernel.
template <auto kernel>
static unsigned resident_grid(long long want) {
  static int per_sm = 0;          // one instance per kernel
  if (per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 128, 0) != cudaSuccess || n < 1) n = 1;
    per_sm = n;
  }
  const long long cap = (long long)sm_count() * per_sm;
  return (unsigned)(want < cap ? want : cap);
}

template <int T, int V>
static void launch_norm_fwd(const NormFwdParams& p, unsigned grid, cudaStream_t s) {
  norm_fwd_kernel<T, V><<<grid, T, 0, s>>>(p);
}
template <int T, int V>
static void launch_norm_bwd(const NormBwdParams& p, unsigned grid, cudaStream_t s) {
  norm_bwd_kernel<T, V><<<grid, T, 0, s>>>(p);
}

MRK_API int mrk_norm_fwd(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                         void* z, float* mean, float* rstd, const void* rng, unsigned long long call_id,
                         float p_drop, float eps, long long M, int H, int rms, int params_f32, void* stream) {
  MRK_REQUIRE(H % 8 == 0 && H <= 8192, "norm: hidden size %d unsupported", H);
  MRK_REQUIRE(M > 0, "norm: empty input");
  NormFwdParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, gamma, beta, (__nv_bfloat16*)y,
                  (__nv_bfloat16*)z, mean, rstd, (const unsigned long long*)rng, call_id, p_drop, eps, M, H, rms,
                  params_f32};
  cudaStream_t s = (cudaStream_t)stream;
  if (H <= 1024 && H % 256 == 0) {
    // one warp per row; as many blocks of four warps as are resident at once
    const long long want = (M + 3) / 4;
    switch (H / 256) {
      case 1: norm_fwd_warp_kernel<1><<<resident_grid<norm_fwd_warp_kernel<1>>(want), 128, 0, s>>>(p); break;
      case 2: norm_fwd_warp_kernel<2><<<resident_grid<norm_fwd_warp_kernel<2>>(want), 128, 0, s>>>(p); break;
      case 3: norm_fwd_warp_kernel<3><<<resident_grid<norm_fwd_warp_kernel<3>>(want), 128, 0, s>>>(p); break;
      default: norm_fwd_warp_kernel<4><<<resident_grid<norm_fwd_warp_kernel<4>>(want), 128, 0, s>>>(p); break;
    }
    MRK_CHECK_LAUNCH();
    return 0;
  }
  const long long cap = (long long)sm_count() * 32;
  const unsigned grid = (unsigned)(M < cap ? M : cap);
  if (H <= 1024) launch_norm_fwd<128, 1>(p, grid, s);
  else if (H <= 2048) launch_norm_fwd<128, 2>(p, grid, s);
  else if (H <= 4096) launch_norm_fwd<256, 2>(p, grid, s);
  else launch_norm_fwd<256, 4>(p, grid, s);
  MRK_CHECK_LAUNCH();
  return 0;
}

// The kernel that walks the rows (both entry points use the same one, so their results are identical).
static void launch_norm_bwd_main(const NormBwdParams& p, cudaStream_t s) {
  const long long M = p.M;
  const int H = p.H;
  const long long cap = (long long)sm_count() * 8;
  const unsigned grid = (unsigned)(M < cap ? M : cap);
  if (H <= 1024 && H % 256 == 0) {
    const long long want = (M + 3) / 4;
    switch (H / 256) {
      case 1: norm_bwd_warp_kernel<1><<<resident_grid<norm_bwd_warp_kernel<1>>(want), 128, 0, s>>>(p); break;
      case 2: norm_bwd_warp_kernel<2><<<resident_grid<norm_bwd_warp_kernel<2>>(want), 128, 0, s>>>(p); break;
      case 3: norm_bwd_warp_kernel<3><<<resident_grid<norm_bwd_warp_kernel<3>>(want), 128, 0, s>>>(p); break;
      default: norm_bwd_warp_kernel<4><<<resident_grid<norm_bwd_warp_kernel<4>>(want), 128, 0, s>>>(p); break;
    }
  } else if (H <= 1024) launch_norm_bwd<128, 1>(p, grid, s);
  else if (H <= 2048) launch_norm_bwd<128, 2>(p, grid, s);
  else if (H <= 4096) launch_norm_bwd<256, 2>(p, grid, s);
  else launch_norm_bwd<256, 4>(p, grid, s);
}

// Number of workspace rows (each 2*H floats) mrk_norm_bwd may use.
// The workspace must be zero before the first call; every call leaves it zero again.
MRK_API int mrk_norm_bwd_workspace_rows() { return kNormSlots; }

MRK_API int mrk_norm_bwd(const void* dy, const void* z, const void* dz_extra, const void* gamma, const float* mean,
                         const float* rstd, void* dres, void* dx, float* dgamma, float* dbeta, float* workspace,
                         const void* rng, unsigned long long call_id, float p_drop, long long M, int H, int rms,
                         int params_f32, void* stream) {
  MRK_REQUIRE(H % 8 == 0 && H <= 8192, "norm: hidden size %d unsupported", H);
  MRK_REQUIRE(M > 0 && workspace != nullptr, "norm: empty input or missing workspace");
  NormBwdParams p{(const __nv_bfloat16*)dy, (const __nv_bfloat16*)z, (const __nv_bfloat16*)dz_extra, gamma, mean,
                  rstd, (__nv_bfloat16*)dres, (__nv_bfloat16*)dx, dgamma, dbeta, workspace,
                  (const unsigned long long*)rng, call_id, p_drop, M, H, rms, params_f32};
  cudaStream_t s = (cudaStream_t)stream;
  launch_norm_bwd_main(p, s);
  MRK_CHECK_LAUNCH();
  dim3 rgrid((H + 31) / 32, 2);
  norm_bwd_reduce_kernel<<<rgrid, 256, 0, s>>>(workspace, kNormSlots, H, dgamma, dbeta);
  MRK_CHECK_LAUNCH();
  return 0;
}

// -------------------------------------------------------------------------------------------------
// Allocation-free variant of the norm backward (declared in norm_noalloc.h).
//
// mrk_norm_bwd needs scratch for the per-block partial sums of the weight / bias gradients and
// expects the caller to hand it in.  Code that runs where device memory can no longer be
// requested (inside a region that forbids cudaMalloc, in a process whose memory is fully
// pre-partitioned, behind an allocator that must not be re-entered) cannot do that, so this entry
// point keeps the scratch in a fixed array that lives in the library image itself.
// -------------------------------------------------------------------------------------------------
namespace mrk {
constexpr int kNoAllocMaxH = 2048;        // largest hidden size served
// kNormSlots * 2 * 2048 floats = 512 KiB, resident on every GPU that loads this library, until exit.
// Device arrays start out zero, and every call leaves the accumulator rows zero again.
static __device__ __align__(256) float g_norm_noalloc_scratch[kNormSlots * 2 * kNoAllocMaxH];

// Device address of the array above, per device.  The symbol's name is only a host-side handle;
// the address a kernel can use has to be asked for, with the device in question current.
static float* g_norm_noalloc_ptr[64] = {nullptr};

static int norm_noalloc_scratch(float** out) {
  int dev = 0;
  MRK_CUDA_OK(cudaGetDevice(&dev));
  MRK_REQUIRE(dev >= 0 && dev < 64, "norm (no-alloc): device index %d out of range", dev);
  if (g_norm_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    MRK_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_norm_noalloc_scratch));
    MRK_REQUIRE(p != nullptr, "norm (no-alloc): scratch symbol has no device address");
    g_norm_noalloc_ptr[dev] = p;
  }
  *out = g_norm_noalloc_ptr[dev];
  return 0;
}
}  // namespace mrk

MRK_API int mrk_norm_bwd_noalloc(const void* dy, const void* z, const void* dz_extra, const void* gamma,
                                 const float* mean, const float* rstd, void* dres, void* dx, float* dgamma,
                                 float* dbeta, long long M, int H, int rms, int params_f32, void* stream) {
  MRK_REQUIRE(H % 8 == 0 && H > 0, "norm (no-alloc): hidden size %d must be a positive multiple of 8", H);
  MRK_REQUIRE(H <= kNoAllocMaxH,
              "norm (no-alloc): hidden size %d exceeds the built-in scratch (max %d); use mrk_norm_bwd with a "
              "caller-provided workspace", H, kNoAllocMaxH);
  MRK_REQUIRE(M > 0 && dy && z && gamma && rstd && dgamma, "norm (no-alloc): missing argument");
  float* scratch = nullptr;
  int rc = norm_noalloc_scratch(&scratch);
  if (rc) return rc;
  NormBwdParams p{(const __nv_bfloat16*)dy, (const __nv_bfloat16*)z, (const __nv_bfloat16*)dz_extra, gamma, mean,
                  rstd, (__nv_bfloat16*)dres, (__nv_bfloat16*)dx, dgamma, dbeta, scratch,
                  nullptr, 0ull, 0.f, M, H, rms, params_f32};
  cudaStream_t s = (cudaStream_t)stream;
  // Blocks add their partial sums into the kNormSlots accumulator rows; the reduction kernel sums
  // the rows and clears them, so a completed call leaves the array zero.  A call whose second
  // launch failed would leave partial sums behind, so the rows are also cleared up front (a
  // memset on the caller's stream; it allocates nothing).
  MRK_CUDA_OK(cudaMemsetAsync(scratch, 0, sizeof(float) * kNormSlots * 2 * kNoAllocMaxH, s));
  launch_norm_bwd_main(p, s);
  MRK_CHECK_LAUNCH();
  dim3 rgrid((H + 31) / 32, 2);
  norm_bwd_reduce_kernel<<<rgrid, 256, 0, s>>>(scratch, kNormSlots, H, dgamma, dbeta);
  MRK_CHECK_LAUNCH();
  return 0;
}
