// Device-side primitives of the symmetric-memory data plane: every rank of a group maps every
// other rank's buffers (CUDA IPC over NVLink / NVSwitch) and a small zero-initialised control
// block per rank that carries barrier flags and per-source result slots.
//
// Flags are monotonic epochs: rank s signals barrier `which` by storing `epoch` (release, system
// scope) into flags[which][s] of each peer's control block; a rank waits by polling its OWN control
// block (local memory) until every source has reached the epoch.  Every wait is bounded: when the
// budget runs out the kernel raises kStatusFlagTimeout in the device status word, skips its work
// and returns, so the context stays usable and the host can read what happened.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace mrk {

constexpr int kSymmMaxRanks = 16;
constexpr int kSymmBarriers = 16;

struct SymmCtrl {
  uint32_t flags[kSymmBarriers][kSymmMaxRanks];  // last epoch signalled, per barrier and source rank
  float slots[kSymmMaxRanks][4];                 // per-source partial results (written by the source)
  float local_acc[4];                            // this rank's block-level accumulators
  uint32_t done[kSymmBarriers];                  // this rank's block-completion counters
};

struct PeerPtrs {
  void* p[kSymmMaxRanks];
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Threads 0..n-1 of the calling block each signal one peer.  The caller makes earlier writes of
// the whole grid visible first (__threadfence_system + a block-completion counter) where needed.
__device__ __forceinline__ void symm_signal(const PeerPtrs& ctrls, int n, int rank, int which, uint32_t epoch) {
  if ((int)threadIdx.x < n) {
    SymmCtrl* peer = reinterpret_cast<SymmCtrl*>(ctrls.p[threadIdx.x]);
    st_release_sys_u32(&peer->flags[which][rank], epoch);
  }
}

// Threads 0..n-1 of the calling block each wait for one source; returns (to every thread of the
// block) whether all sources arrived within `budget` SM cycles.  Contains __syncthreads.
__device__ __forceinline__ bool symm_wait(SymmCtrl* mine, int n, int which, uint32_t epoch, long long budget,
                                          unsigned* status) {
  int ok = 1;
  if ((int)threadIdx.x < n) {
    const uint32_t* f = &mine->flags[which][threadIdx.x];
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys_u32(f) - epoch) < 0) {
      if (clock64() - t0 > budget) {
        raise_status(status, kStatusFlagTimeout);
        ok = 0;
        break;
      }
      __nanosleep(100);
    }
  }
  return __syncthreads_and(ok) != 0;
}

}  // namespace mrk
