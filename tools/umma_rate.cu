// Cycles per tcgen05.mma on B200 as a function of how often the issuing thread commits.
//
// One CTA (cta_group::1, 128 x 256 x 16) or one CTA pair (cta_group::2, 256 x 256 x 16) per SM issues
// bf16 UMMAs back to back from shared memory that holds random values; no TMA, no epilogue.  After
// every `per` k-blocks of four UMMAs the thread issues `commits` tcgen05.commit instructions to
// mbarriers nobody waits on, which is what a GEMM main loop does to hand a ring stage back to its
// producer.  Every wait in here is bounded.
//
// Build and run (one B200):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -I merak_b200/csrc -o /tmp/umma_rate tools/umma_rate.cu && /tmp/umma_rate
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "sm100_ptx.cuh"
using namespace mrk;

__device__ unsigned g_status;

template <int CG>
__global__ void __launch_bounds__(128, 1) umma_rate_kernel(long long* out, int iters, int commits, int per) {
  constexpr int N = 256, STAGES = 4;
  constexpr int kA = 128 * 64 * 2, kB = (N / CG) * 64 * 2, kStage = kA + kB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t done_bar, sink[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < STAGES * kStage / 4; i += blockDim.x) {
    uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    const uint32_t lo = 0x3F00u | (h & 0x80FFu), hi = 0x3F00u | ((h >> 16) & 0x80FFu);   // bf16 values in (-2, 2)
    reinterpret_cast<uint32_t*>(smem)[i] = lo | (hi << 16);
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&done_bar), 1);
    mbar_init(smem_u32(&sink[0]), 1);
    mbar_init(smem_u32(&sink[1]), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    if (CG == 2) { tmem_alloc_pair(smem_u32(&tmem_slot), 512); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const bool leader = CG == 1 || cluster_ctarank() == 0;
  if (warp == 1 && lane == 0 && leader) {
    const uint32_t idesc = make_idesc_bf16(CG == 2 ? 256 : 128, N, 0, 0);
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      const uint32_t sa = smem_u32(smem + (it % STAGES) * kStage), sb = sa + kA;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (CG == 2) umma_bf16_ss_pair(tmem_base, desc_kmajor(sa, k), desc_kmajor(sb, k), idesc, (it | k) ? 1u : 0u);
        else umma_bf16_ss(tmem_base, desc_kmajor(sa, k), desc_kmajor(sb, k), idesc, (it | k) ? 1u : 0u);
      }
      if ((it % per) == per - 1)
        for (int c = 0; c < commits; ++c) {
          if (CG == 2) umma_commit_pair(c == 0 ? smem_u32(&sink[0]) : map_to_cta(smem_u32(&sink[1]), 1));
          else umma_commit(smem_u32(&sink[c]));
        }
    }
    if (CG == 2) umma_commit_pair(smem_u32(&done_bar)); else umma_commit(smem_u32(&done_bar));
    mbar_wait(smem_u32(&done_bar), 0, &abort_flag, &g_status);
    if (blockIdx.x == 0) out[0] = clock64() - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync_all();
  if (warp == 0) {
    tc_fence_after();
    if (CG == 2) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
  }
}

template <int CG>
static void run(const char* name, int iters, int commits, int per) {
  long long* out;
  cudaMalloc(&out, 8);
  cudaMemset(out, 0, 8);
  const int smem = 4 * (128 * 64 * 2 + (256 / CG) * 64 * 2) + 1024;
  cudaFuncSetAttribute(umma_rate_kernel<CG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms / CG * CG);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  for (int rep = 0; rep < 2; ++rep) {
    cudaError_t e = cudaLaunchKernelEx(&cfg, umma_rate_kernel<CG>, out, iters, commits, per);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("%s: %s\n", name, cudaGetErrorString(e)); return; }
  }
  long long h = 0;
  cudaMemcpy(&h, out, 8, cudaMemcpyDeviceToHost);
  const double cyc = (double)h / (iters * 4.0);
  printf("| %s | %d per %d k-block(s) | %.1f | %.0f |\n", name, commits, per, cyc, 2.0 * 128 * 256 * 16 / cyc);
  cudaFree(out);
}

int main() {
  printf("| UMMA | commits | cycles per UMMA | FLOP / clock / SM |\n|---|---|---|---|\n");
  const int iters = 4000;
  for (int commits : {0, 1, 2})
    for (int per : {1, 2}) {
      if (commits == 0 && per == 2) continue;
      run<1>("cta_group::1 128x256x16", iters, commits, per);
      run<2>("cta_group::2 256x256x16", iters, commits, per);
    }
  unsigned st = 0;
  cudaMemcpyFromSymbol(&st, g_status, 4);
  printf("status word %u\n", st);
  return st != 0;
}
