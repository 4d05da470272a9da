// Expert-parallel token exchange by direct peer stores (all-to-all of rows without a library
// collective): every rank writes the rows destined for rank d straight into d's receive buffer at
// the row offset reserved for this source, then signals; a rank's kernel returns once every source
// has signalled, so the expert GEMMs that follow in the stream see all their rows.
//
// The reference has no mixture-of-experts path; this is the dispatch/combine step of
// merak_b200/parallel/expert.py for peer-mapped expert-parallel groups.
#include "fused_comm.h"
#include "host_common.h"
#include "symm.cuh"

namespace mrk {

constexpr int kA2AThreads = 512;

struct A2ASplits {
  long long send_begin[kSymmMaxRanks + 1];   // rows [send_begin[d], send_begin[d+1]) of `send` go to rank d
  long long dst_row[kSymmMaxRanks];          // first row of this source's block in rank d's receive buffer
};

__global__ void __launch_bounds__(kA2AThreads)
moe_alltoall_push_kernel(PeerPtrs recv, PeerPtrs ctrls, int n, int rank, const uint4* __restrict__ send,
                         A2ASplits sp, int vec_per_row, uint32_t epoch, int sync, long long budget, unsigned* status) {
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(ctrls.p[rank]);
  __shared__ int s_last;
  // entry: every rank is done reading the receive buffer this call overwrites
  bool ok = true;
  if (sync) {
    if (blockIdx.x == 0) symm_signal(ctrls, n, rank, 7, epoch);
    ok = symm_wait(mine, n, 7, epoch, budget, status);
  }
  if (ok) {
    const long long total_vec = sp.send_begin[n] * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec;
         i += (long long)gridDim.x * blockDim.x) {
      const long long row = i / vec_per_row;
      const int cv = (int)(i - row * vec_per_row);
      int d = 0;
#pragma unroll 1
      while (d + 1 < n && row >= sp.send_begin[d + 1]) ++d;
      uint4* dst = reinterpret_cast<uint4*>(recv.p[d]) + (sp.dst_row[d] + (row - sp.send_begin[d])) * vec_per_row + cv;
      *dst = __ldg(send + i);
    }
  }
  if (sync) {   // exit: all rows of all sources have landed here
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&mine->done[2], 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last) {
      if (threadIdx.x == 0) mine->done[2] = 0u;
      __threadfence_system();
      symm_signal(ctrls, n, rank, 8, epoch);
      symm_wait(mine, n, 8, epoch, budget, status);
    }
  }
}

}  // namespace mrk

using namespace mrk;

// send: [rows, H] bf16 (H % 8 == 0), rows grouped by destination rank; send_begin[n+1] and
// dst_row[n] are host arrays.  recv_ptrs[d] is rank d's receive buffer (peer-mapped).
MRK_API int mrk_moe_alltoall_push(void* const* recv_ptrs, void* const* ctrl_ptrs, int n, int rank, const void* send,
                                  const long long* send_begin, const long long* dst_row, int H, int elem_bytes,
                                  unsigned epoch, int sync, int budget_ms, void* stream) {
  MRK_REQUIRE(n >= 1 && n <= kSymmMaxRanks && rank >= 0 && rank < n, "moe_alltoall_push: bad group");
  MRK_REQUIRE((H * elem_bytes) % 16 == 0 && ((uintptr_t)send & 15) == 0, "moe_alltoall_push: rows must be 16-byte multiples");
  PeerPtrs r, c;
  A2ASplits sp;
  for (int k = 0; k < kSymmMaxRanks; ++k) {
    r.p[k] = k < n ? recv_ptrs[k] : nullptr;
    c.p[k] = k < n ? ctrl_ptrs[k] : nullptr;
    sp.dst_row[k] = k < n ? dst_row[k] : 0;
  }
  for (int k = 0; k <= kSymmMaxRanks; ++k) sp.send_begin[k] = send_begin[k <= n ? k : n];
  unsigned* status = status_word_device();
  MRK_REQUIRE(status != nullptr, "moe_alltoall_push: status word unavailable");
  const int vec_per_row = H * elem_bytes / 16;
  const long long total = sp.send_begin[n] * vec_per_row;
  long long blocks = (total + kA2AThreads - 1) / kA2AThreads;
  const long long cap = (long long)sm_count() * 2;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  moe_alltoall_push_kernel<<<(unsigned)blocks, kA2AThreads, 0, (cudaStream_t)stream>>>(
      r, c, n, rank, reinterpret_cast<const uint4*>(send), sp, vec_per_row, epoch, sync,
      (long long)(budget_ms > 0 ? budget_ms : 2000) * 2000000ll, status);
  MRK_CHECK_LAUNCH();
  return 0;
}
