// Fused compute + collective kernels over peer-mapped (symmetric) memory, and the host side of
// that data plane (allocation, CUDA IPC handle exchange helpers).
//
// Data-parallel optimizer step, two kernels per step instead of all-reduce + clip + AdamW +
// (ZeRO-1) all-gather:
//
//   dp_reduce_scatter_kernel   every rank sums ITS shard of the flat fp32 gradient buffer straight
//                              out of all ranks' buffers (peer loads), keeps the reduced shard and
//                              its masked squared norm, and posts the norm to every rank.
//   dp_adamw_allgather_kernel  global clip coefficient from the posted norms, AdamW on the shard
//                              (fp32 master + moments live only on the owner), and the refreshed
//                              bf16 parameters are stored into every rank's model buffer.
//
// This replaces Merak/core/merak_engine.py:552-621 (bucketed all-reduce), Merak/core/zero/
// stage1.py:476-757 (reduce-scatter, step, all-gather) and Merak/core/amp/fp16_optimizer.py:118-185.
#include <math.h>
#include <string.h>

#include "fused_comm.h"
#include "host_common.h"
#include "symm.cuh"

namespace mrk {

constexpr int kDpThreads = 512;

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid in warp 0
}

// flags: one byte per 64-element granule of the flat buffer (absolute index / 64):
//   bit 0  weight decay applies            bit 1  excluded from the gradient norm on this rank
constexpr unsigned kFlagDecay = 1u, kFlagNoNorm = 2u;

template <int N>
__global__ void __launch_bounds__(kDpThreads)
dp_reduce_scatter_kernel(PeerPtrs grads, PeerPtrs ctrls, int n_rt, int rank, long long lo, long long cnt,
                         const unsigned char* __restrict__ flags, uint32_t epoch, int sync, long long budget,
                         unsigned* status) {
  const int n = N > 0 ? N : n_rt;
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(ctrls.p[rank]);
  __shared__ float red[kDpThreads / 32];
  __shared__ int s_last;
  bool ok = true;
  if (sync) {   // every rank's backward pass has finished writing its gradient buffer
    if (blockIdx.x == 0) symm_signal(ctrls, n, rank, 0, epoch);
    ok = symm_wait(mine, n, 0, epoch, budget, status);
  }
  float acc = 0.f, bad = 0.f;
  if (ok) {
    float* dst = reinterpret_cast<float*>(grads.p[rank]) + lo;
    const long long nvec = cnt >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      float4 part[N > 0 ? N : kSymmMaxRanks];
#pragma unroll
      for (int k = 0; k < (N > 0 ? N : kSymmMaxRanks); ++k) {
        if (k < n) part[k] = ld_relaxed_sys_f4(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[k]) + lo) + i);
      }
      float4 s = part[0];
#pragma unroll
      for (int k = 1; k < (N > 0 ? N : kSymmMaxRanks); ++k) {
        if (k < n) { s.x += part[k].x; s.y += part[k].y; s.z += part[k].z; s.w += part[k].w; }
      }
      reinterpret_cast<float4*>(dst)[i] = s;
      const unsigned f = flags ? flags[(lo + (i << 2)) >> 6] : 0u;
      if (!(f & kFlagNoNorm)) {
        acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
        bad += (isfinite(s.x) ? 0.f : 1.f) + (isfinite(s.y) ? 0.f : 1.f) + (isfinite(s.z) ? 0.f : 1.f) +
               (isfinite(s.w) ? 0.f : 1.f);
      }
    }
  }
  const float tot = block_sum(acc, red);
  const float totbad = block_sum(bad, red);
  if (threadIdx.x == 0) {
    atomicAdd(&mine->local_acc[0], tot);
    // a block whose bounded wait ran out skipped its part of the shard: count it as a bad value so
    // that whichever block finishes last posts a non-zero "bad" and every rank skips the update
    atomicAdd(&mine->local_acc[1], ok ? totbad : totbad + 1.f);
    __threadfence();
    s_last = atomicAdd(&mine->done[0], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {   // the last block posts this rank's partial norm to every rank
    __threadfence();
    if ((int)threadIdx.x < n) {
      const float a = *reinterpret_cast<volatile float*>(&mine->local_acc[0]);
      const float b = ok ? *reinterpret_cast<volatile float*>(&mine->local_acc[1]) : INFINITY;
      SymmCtrl* peer = reinterpret_cast<SymmCtrl*>(ctrls.p[threadIdx.x]);
      volatile float* slot = peer->slots[rank];
      slot[0] = a;
      slot[1] = b;
      __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      mine->local_acc[0] = 0.f;
      mine->local_acc[1] = 0.f;
      mine->done[0] = 0u;
    }
    if (sync) symm_signal(ctrls, n, rank, 1, epoch);
  }
}

template <int N>
__global__ void __launch_bounds__(kDpThreads)
dp_adamw_allgather_kernel(PeerPtrs models, PeerPtrs ctrls, int n_rt, int rank, long long lo, long long cnt,
                          const float* __restrict__ grad_shard, float* __restrict__ master, float* __restrict__ m,
                          float* __restrict__ v, const unsigned char* __restrict__ flags,
                          const float* __restrict__ hp, float grad_scale, float max_norm,
                          const float* __restrict__ sumsq_src, float* __restrict__ norm_out, int* __restrict__ skip_out,
                          uint32_t epoch, int sync, int wait_partials, long long budget, unsigned* status) {
  const int n = N > 0 ? N : n_rt;
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(ctrls.p[rank]);
  __shared__ int s_last;
  bool ok = true;
  if (sync && wait_partials) ok = symm_wait(mine, n, 1, epoch, budget, status);
  float ss = 0.f, bad = 0.f;
  if (sumsq_src) {
    ss = sumsq_src[0];
    bad = sumsq_src[1];
  } else {
    for (int k = 0; k < n; ++k) {
      ss += *reinterpret_cast<volatile float*>(&mine->slots[k][0]);
      bad += *reinterpret_cast<volatile float*>(&mine->slots[k][1]);
    }
  }
  const float norm = sqrtf(ss) * grad_scale;
  const bool skip = !ok || !isfinite(norm) || bad != 0.f;
  float gs = grad_scale;
  if (max_norm > 0.f && norm > max_norm) gs *= max_norm / (norm + 1e-6f);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (norm_out) *norm_out = norm;
    if (skip_out) *skip_out = skip ? 1 : 0;
  }
  if (!skip) {
    const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4];
    const float rbc1 = 1.f / hp[5], rbc2 = 1.f / hp[6];
    const long long nvec = cnt >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      const float4 g0 = reinterpret_cast<const float4*>(grad_shard)[2 * i], g1 = reinterpret_cast<const float4*>(grad_shard)[2 * i + 1];
      float4 p0 = reinterpret_cast<float4*>(master)[2 * i], p1 = reinterpret_cast<float4*>(master)[2 * i + 1];
      float4 m0 = reinterpret_cast<float4*>(m)[2 * i], m1 = reinterpret_cast<float4*>(m)[2 * i + 1];
      float4 v0 = reinterpret_cast<float4*>(v)[2 * i], v1 = reinterpret_cast<float4*>(v)[2 * i + 1];
      float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
      float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      const unsigned f = flags ? flags[(lo + (i << 3)) >> 6] : kFlagDecay;
      const float decay = 1.f - lr * ((f & kFlagDecay) ? wd : 0.f);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float gk = g[k] * gs;
        mm[k] = b1 * mm[k] + (1.f - b1) * gk;
        vv[k] = b2 * vv[k] + (1.f - b2) * gk * gk;
        pp[k] = pp[k] * decay - lr * (mm[k] * rbc1) / (sqrtf(vv[k] * rbc2) + eps);
      }
      reinterpret_cast<float4*>(master)[2 * i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(pp[4], pp[5], pp[6], pp[7]);
      reinterpret_cast<float4*>(m)[2 * i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
      reinterpret_cast<float4*>(v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
      const uint4 w = make_uint4(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]), pack_bf16x2(pp[4], pp[5]),
                                 pack_bf16x2(pp[6], pp[7]));
      // all-gather: the owner stores the refreshed bf16 parameters into every rank's model buffer
#pragma unroll
      for (int k = 0; k < (N > 0 ? N : kSymmMaxRanks); ++k) {
        if (k < n) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(models.p[k]) + lo)[i] = w;
      }
    }
  }
  if (sync) {   // every rank's stores have landed before anybody's next forward pass reads parameters
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&mine->done[1], 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last) {
      if (threadIdx.x == 0) mine->done[1] = 0u;
      __threadfence_system();
      symm_signal(ctrls, n, rank, 2, epoch);
      symm_wait(mine, n, 2, epoch, budget, status);
    }
  }
}

// Waits for the posted partial norms and sums them into out[0..1] (used when the norm still has to
// be all-reduced over the tensor- and pipeline-parallel groups before the update).
__global__ void dp_norm_gather_kernel(PeerPtrs ctrls, int n, int rank, float* out, uint32_t epoch, int sync,
                                      long long budget, unsigned* status) {
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(ctrls.p[rank]);
  bool ok = true;
  if (sync) ok = symm_wait(mine, n, 1, epoch, budget, status);
  if (threadIdx.x == 0) {
    float ss = 0.f, bad = ok ? 0.f : INFINITY;
    for (int k = 0; k < n; ++k) {
      ss += *reinterpret_cast<volatile float*>(&mine->slots[k][0]);
      bad += *reinterpret_cast<volatile float*>(&mine->slots[k][1]);
    }
    out[0] = ss;
    out[1] = bad;
  }
}

// Stand-alone barrier over the group (signal + bounded wait on barrier slot `which`).
__global__ void symm_barrier_kernel(PeerPtrs ctrls, int n, int rank, int which, uint32_t epoch, int signal,
                                    long long budget, unsigned* status) {
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(ctrls.p[rank]);
  __threadfence_system();
  if (signal) symm_signal(ctrls, n, rank, which, epoch);
  symm_wait(mine, n, which, epoch, budget, status);
}

static inline long long budget_cycles(int budget_ms) {
  return (long long)(budget_ms > 0 ? budget_ms : 2000) * 2000000ll;   // ~2 GHz SM clock
}

static int fill_peers(PeerPtrs* out, void* const* ptrs, int n) {
  for (int k = 0; k < kSymmMaxRanks; ++k) out->p[k] = k < n ? ptrs[k] : nullptr;
  return 0;
}

}  // namespace mrk

using namespace mrk;

// ---- symmetric memory: allocation and CUDA IPC ---------------------------------------------------
MRK_API int mrk_symm_alloc(unsigned long long bytes, void** out) {
  MRK_REQUIRE(out != nullptr && bytes > 0, "symm_alloc: bad arguments");
  void* p = nullptr;
  MRK_CUDA_OK(cudaMalloc(&p, bytes));
  MRK_CUDA_OK(cudaMemset(p, 0, bytes));
  MRK_CUDA_OK(cudaDeviceSynchronize());
  *out = p;
  return 0;
}

MRK_API int mrk_symm_free(void* p) {
  if (p) MRK_CUDA_OK(cudaFree(p));
  return 0;
}

MRK_API int mrk_symm_ctrl_bytes() { return (int)((sizeof(SymmCtrl) + 255) / 256 * 256); }

MRK_API int mrk_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

MRK_API int mrk_ipc_get_handle(void* p, unsigned char* out) {
  cudaIpcMemHandle_t h;
  MRK_CUDA_OK(cudaIpcGetMemHandle(&h, p));
  memcpy(out, &h, sizeof(h));
  return 0;
}

MRK_API int mrk_ipc_open(const unsigned char* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  MRK_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}

MRK_API int mrk_ipc_close(void* p) {
  if (p) MRK_CUDA_OK(cudaIpcCloseMemHandle(p));
  return 0;
}

// ---- launches --------------------------------------------------------------------------------------
static unsigned dp_grid(long long items) {
  long long blocks = (items + kDpThreads - 1) / kDpThreads;
  const long long cap = (long long)sm_count() * 2;   // everything resident: blocks poll flags
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

MRK_API int mrk_dp_reduce_scatter(void* const* grad_ptrs, void* const* ctrl_ptrs, int n, int rank, long long lo,
                                  long long cnt, const unsigned char* flags, unsigned epoch, int sync, int budget_ms,
                                  void* stream) {
  MRK_REQUIRE(n >= 1 && n <= kSymmMaxRanks && rank >= 0 && rank < n, "dp_reduce_scatter: bad group (%d ranks)", n);
  MRK_REQUIRE(cnt >= 0 && (cnt % 8) == 0 && (lo % 8) == 0, "dp_reduce_scatter: shard must be a multiple of 8 elements");
  PeerPtrs g, c;
  fill_peers(&g, grad_ptrs, n);
  fill_peers(&c, ctrl_ptrs, n);
  unsigned* status = status_word_device();
  MRK_REQUIRE(status != nullptr, "dp_reduce_scatter: status word unavailable");
  const unsigned grid = dp_grid(cnt / 4);
  const long long b = budget_cycles(budget_ms);
  cudaStream_t s = (cudaStream_t)stream;
#define MRK_RS(NN) dp_reduce_scatter_kernel<NN><<<grid, kDpThreads, 0, s>>>(g, c, n, rank, lo, cnt, flags, epoch, sync, b, status)
  switch (n) {
    case 1: MRK_RS(1); break;
    case 2: MRK_RS(2); break;
    case 4: MRK_RS(4); break;
    case 8: MRK_RS(8); break;
    default: MRK_RS(0); break;
  }
#undef MRK_RS
  MRK_CHECK_LAUNCH();
  return 0;
}

// One device-to-device copy on `stream` (a copy-engine transfer; `dst` may be peer-mapped memory).
// The overlapped data-parallel reduction pushes finished pieces of the gradient buffer to their
// owner's staging buffer with it while the backward pass keeps every SM: the copy engines move the
// bytes over NVLink, no thread block is spent and none can get in the way of a persistent GEMM grid.
MRK_API int mrk_memcpy_d2d_async(void* dst, const void* src, unsigned long long bytes, void* stream) {
  MRK_REQUIRE(dst != nullptr && src != nullptr && bytes > 0, "memcpy_d2d_async: bad arguments");
  MRK_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return 0;
}

MRK_API int mrk_dp_adamw_allgather(void* const* model_ptrs, void* const* ctrl_ptrs, int n, int rank, long long lo,
                                   long long cnt, const float* grad_shard, float* master, float* m, float* v,
                                   const unsigned char* flags, const float* hp, float grad_scale, float max_norm,
                                   const float* sumsq_src, float* norm_out, int* skip_out, unsigned epoch, int sync,
                                   int wait_partials, int budget_ms, void* stream) {
  MRK_REQUIRE(n >= 1 && n <= kSymmMaxRanks && rank >= 0 && rank < n, "dp_adamw_allgather: bad group (%d ranks)", n);
  MRK_REQUIRE(cnt > 0 && (cnt % 8) == 0 && (lo % 8) == 0, "dp_adamw_allgather: shard must be a multiple of 8 elements");
  MRK_REQUIRE((((uintptr_t)grad_shard | (uintptr_t)master | (uintptr_t)m | (uintptr_t)v) & 15) == 0,
              "dp_adamw_allgather: buffers must be 16-byte aligned");
  PeerPtrs mo, c;
  fill_peers(&mo, model_ptrs, n);
  fill_peers(&c, ctrl_ptrs, n);
  unsigned* status = status_word_device();
  MRK_REQUIRE(status != nullptr, "dp_adamw_allgather: status word unavailable");
  const unsigned grid = dp_grid(cnt / 8);
  const long long b = budget_cycles(budget_ms);
  cudaStream_t s = (cudaStream_t)stream;
#define MRK_AG(NN)                                                                                           \
  dp_adamw_allgather_kernel<NN><<<grid, kDpThreads, 0, s>>>(mo, c, n, rank, lo, cnt, grad_shard, master, m, v, \
                                                            flags, hp, grad_scale, max_norm, sumsq_src,      \
                                                            norm_out, skip_out, epoch, sync, wait_partials, b, status)
  switch (n) {
    case 1: MRK_AG(1); break;
    case 2: MRK_AG(2); break;
    case 4: MRK_AG(4); break;
    case 8: MRK_AG(8); break;
    default: MRK_AG(0); break;
  }
#undef MRK_AG
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_dp_norm_gather(void* const* ctrl_ptrs, int n, int rank, float* out2, unsigned epoch, int sync,
                               int budget_ms, void* stream) {
  MRK_REQUIRE(n >= 1 && n <= kSymmMaxRanks && rank >= 0 && rank < n, "dp_norm_gather: bad group (%d ranks)", n);
  PeerPtrs c;
  fill_peers(&c, ctrl_ptrs, n);
  unsigned* status = status_word_device();
  MRK_REQUIRE(status != nullptr, "dp_norm_gather: status word unavailable");
  dp_norm_gather_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, n, rank, out2, epoch, sync, budget_cycles(budget_ms), status);
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_symm_barrier(void* const* ctrl_ptrs, int n, int rank, int which, unsigned epoch, int signal,
                             int budget_ms, void* stream) {
  MRK_REQUIRE(n >= 1 && n <= kSymmMaxRanks && rank >= 0 && rank < n && which >= 0 && which < kSymmBarriers,
              "symm_barrier: bad arguments");
  PeerPtrs c;
  fill_peers(&c, ctrl_ptrs, n);
  unsigned* status = status_word_device();
  MRK_REQUIRE(status != nullptr, "symm_barrier: status word unavailable");
  symm_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, n, rank, which, epoch, signal, budget_cycles(budget_ms), status);
  MRK_CHECK_LAUNCH();
  return 0;
}

// ---- tensor parallelism: GEMM -> reduce-scatter / all-reduce, pull side ---------------------------
namespace mrk {

// Every rank's GEMM has written its partial product [M, N] (bf16) into its peer-mapped buffer.  This
// rank owns the rows of its sequence segments: it pulls those rows of every rank's partial
// (coalesced 16-byte peer loads), sums them in fp32 and stores bf16.  Local row r is global row
// ((r / seg_rows) * n + rank) * seg_rows + r % seg_rows.
template <int N_RANKS>
__global__ void __launch_bounds__(kDpThreads)
tp_reduce_pull_kernel(PeerPtrs parts, PeerPtrs ctrls, int n_rt, int rank, __nv_bfloat16* __restrict__ out,
                      long long rows_local, int N, int seg_rows, const __nv_bfloat16* __restrict__ bias,
                      uint32_t epoch, int sync, long long budget, unsigned* status) {
  const int n = N_RANKS > 0 ? N_RANKS : n_rt;
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(ctrls.p[rank]);
  bool ok = true;
  if (sync) {
    if (blockIdx.x == 0) symm_signal(ctrls, n, rank, 5, epoch);
    ok = symm_wait(mine, n, 5, epoch, budget, status);
  }
  if (!ok) return;
  const int vec_per_row = N >> 3;
  const long long nvec = rows_local * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int cv = (int)(i - r * vec_per_row);
    const long long b = r / seg_rows;
    const long long grow = (b * n + rank) * seg_rows + (r - b * seg_rows);
    uint4 part[N_RANKS > 0 ? N_RANKS : kSymmMaxRanks];
#pragma unroll
    for (int k = 0; k < (N_RANKS > 0 ? N_RANKS : kSymmMaxRanks); ++k)
      if (k < n) part[k] = ld_relaxed_sys_u4(reinterpret_cast<const uint4*>(
                     reinterpret_cast<const __nv_bfloat16*>(parts.p[k]) + grow * N) + cv);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (bias != nullptr) {
      const uint4 bb = __ldg(reinterpret_cast<const uint4*>(bias) + cv);
      const uint32_t w[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] = f.x; acc[2 * e + 1] = f.y; }
    }
#pragma unroll
    for (int k = 0; k < (N_RANKS > 0 ? N_RANKS : kSymmMaxRanks); ++k) {
      if (k < n) {
        const uint32_t w[4] = {part[k].x, part[k].y, part[k].z, part[k].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
      }
    }
    reinterpret_cast<uint4*>(out + r * N)[cv] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                           pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// All-reduce = the pull above into a peer-mapped "reduced" buffer, then every rank pulls the other
// ranks' reduced rows: out[row] for all M rows.
__global__ void __launch_bounds__(kDpThreads)
tp_gather_rows_kernel(PeerPtrs reds, PeerPtrs ctrls, int n, int rank, __nv_bfloat16* __restrict__ out, long long M,
                      int N, int seg_rows, uint32_t epoch, int sync, long long budget, unsigned* status) {
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(ctrls.p[rank]);
  bool ok = true;
  if (sync) {
    if (blockIdx.x == 0) symm_signal(ctrls, n, rank, 6, epoch);
    ok = symm_wait(mine, n, 6, epoch, budget, status);
  }
  if (!ok) return;
  const int vec_per_row = N >> 3;
  const long long nvec = M * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int cv = (int)(i - r * vec_per_row);
    const long long s = r / seg_rows;
    const int owner = (int)(s % n);
    const long long local = (s / n) * seg_rows + (r - s * seg_rows);
    reinterpret_cast<uint4*>(out + r * N)[cv] = ld_relaxed_sys_u4(
        reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(reds.p[owner]) + local * N) + cv);
  }
}

}  // namespace mrk

MRK_API int mrk_tp_reduce_pull(void* const* part_ptrs, void* const* ctrl_ptrs, int n, int rank, void* out,
                               long long rows_local, int N, int seg_rows, const void* bias, unsigned epoch, int sync,
                               int budget_ms, void* stream) {
  MRK_REQUIRE(n >= 2 && n <= kSymmMaxRanks && rank >= 0 && rank < n, "tp_reduce_pull: bad group");
  MRK_REQUIRE(N % 8 == 0 && rows_local > 0 && seg_rows > 0 && rows_local % seg_rows == 0, "tp_reduce_pull: bad shape");
  PeerPtrs a, c;
  fill_peers(&a, part_ptrs, n);
  fill_peers(&c, ctrl_ptrs, n);
  unsigned* status = status_word_device();
  MRK_REQUIRE(status != nullptr, "tp_reduce_pull: status word unavailable");
  const unsigned grid = dp_grid(rows_local * (N / 8));
  const long long b = budget_cycles(budget_ms);
  cudaStream_t s = (cudaStream_t)stream;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* bi = reinterpret_cast<const __nv_bfloat16*>(bias);
#define MRK_PULL(NN) tp_reduce_pull_kernel<NN><<<grid, kDpThreads, 0, s>>>(a, c, n, rank, o, rows_local, N, seg_rows, bi, epoch, sync, b, status)
  switch (n) {
    case 2: MRK_PULL(2); break;
    case 4: MRK_PULL(4); break;
    case 8: MRK_PULL(8); break;
    default: MRK_PULL(0); break;
  }
#undef MRK_PULL
  MRK_CHECK_LAUNCH();
  return 0;
}

MRK_API int mrk_tp_gather_rows(void* const* red_ptrs, void* const* ctrl_ptrs, int n, int rank, void* out, long long M,
                               int N, int seg_rows, unsigned epoch, int sync, int budget_ms, void* stream) {
  MRK_REQUIRE(n >= 2 && n <= kSymmMaxRanks && rank >= 0 && rank < n, "tp_gather_rows: bad group");
  MRK_REQUIRE(N % 8 == 0 && M > 0 && seg_rows > 0, "tp_gather_rows: bad shape");
  PeerPtrs a, c;
  fill_peers(&a, red_ptrs, n);
  fill_peers(&c, ctrl_ptrs, n);
  unsigned* status = status_word_device();
  MRK_REQUIRE(status != nullptr, "tp_gather_rows: status word unavailable");
  tp_gather_rows_kernel<<<dp_grid(M * (N / 8)), kDpThreads, 0, (cudaStream_t)stream>>>(
      a, c, n, rank, reinterpret_cast<__nv_bfloat16*>(out), M, N, seg_rows, epoch, sync, budget_cycles(budget_ms), status);
  MRK_CHECK_LAUNCH();
  return 0;
}
