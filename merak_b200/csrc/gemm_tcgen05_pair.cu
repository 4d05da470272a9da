// CTA-pair bf16 GEMM: the same computation as gemm_tcgen05.cu, executed by clusters of two CTAs.
//
// One cta_group::2 UMMA multiplies a 256 x 256 x 16 block: each CTA of the pair supplies its own
// 128 rows of A and HALF of the B tile (128 of the 256 columns), and keeps its 128 accumulator rows
// in its own TMEM.  Per SM and k-block that is 16 KB of A + 16 KB of B for the same 128x256x64
// of math that costs the single-CTA kernel 48 KB, i.e. one third less L2->SM traffic, which is
// what bounds the single-CTA kernel.  No multicast is used: every CTA loads exactly the bytes it
// keeps.
//
//   warp 0   TMA producer (both CTAs; completion bytes are credited to the even CTA's barrier)
//   warp 1   TMEM allocation (both CTAs); UMMA issue + commits (even CTA only)
//   warps 2..9  epilogue of this CTA's 128 rows (two warps per TMEM lane quadrant, half the columns each).
//               bf16 outputs are staged in shared memory (128-byte swizzled boxes) and written with TMA
//               stores: full 128-byte lines instead of 16-byte pieces scattered over 32 rows per
//               instruction, which is what made the epilogue the bottleneck of short-K problems.
#include "gemm_common.cuh"
#include "host_common.h"

namespace mrk {

constexpr int kPairBlockM = 256;      // rows per cluster tile (128 per CTA)
constexpr int kPairBlockN = 256;
constexpr int kPairBlockK = 64;       // one k-block: the 64-element swizzle atom
constexpr int kPairThreads = 320;     // TMA warp, UMMA warp, 8 epilogue warps
// A ring stage holds kPairGroup consecutive k-blocks and has ONE full and ONE empty barrier: the UMMA
// thread waits once and commits once per eight UMMAs.  Measured on B200 with 256x256x16 UMMAs back to
// back: no commit 128 cycles per UMMA, one commit per four UMMAs 138-166 (the more code around the
// commit, the worse), one per eight 128.
constexpr int kPairGroup = 2;
constexpr int kPairStages = 3;
constexpr int kPairABytes = 128 * kPairBlockK * 2;            // this CTA's rows of A, one k-block
constexpr int kPairBBytes = (kPairBlockN / 2) * kPairBlockK * 2;  // this CTA's half of B, one k-block
constexpr int kPairSubBytes = kPairABytes + kPairBBytes;      // 32 KB per k-block
constexpr int kPairStageBytes = kPairGroup * kPairSubBytes;   // 64 KB
// epilogue staging: one 128-row x 64-column bf16 box (TMA-store source) per column half
constexpr int kPairStagingBytes = 2 * 16384;
constexpr int kPairSmemTotal = kPairStages * kPairStageBytes + kPairStagingBytes + 1024 + 1024;

// mode 1, store thread: the partial product of sub-tile `u` is complete in this rank's buffer.
__device__ __forceinline__ void rs_publish(const GemmParams& p, int owner, int u) {
  const GemmComm& c = p.comm;
  // the caller has waited for its bulk stores to complete; the release store orders them before the flag
  st_release_sys_u32(c.tile_flags[owner] + (size_t)c.rank * c.units_total + u, c.epoch);
}

// ---- mode 1: reduce phase ---------------------------------------------------------------------------
// After its tiles, every CTA sums the sub-tiles this rank owns.  Peer loads take microseconds, so the
// remote partial products are not read with register loads but streamed into the (now idle) operand
// ring with bulk asynchronous copies, several pieces deep: the otherwise idle TMA thread is the
// producer (waits for a piece's flags, issues one 256-byte row copy per row and remote rank, completion
// on an mbarrier); the 256 epilogue threads are the consumer (remote rows from shared memory + the local
// partial from global memory + bias -> bf16 rows of the result).  A piece is `rows` rows of one
// 128-column sub-tile, sized so that the copies of all remote ranks fit one slot of the ring.
struct RsPlan {
  int rows;          // rows per piece: 128 (n = 2), 64 (n <= 4), 32 (n <= 8)
  int pieces_per_unit;
  int slot_bytes;    // (n - 1) * rows * 256
  int slots;
  int sub_per_row, owned_units;
};

__device__ __forceinline__ RsPlan rs_plan(const GemmParams& p, int ring_bytes) {
  RsPlan q;
  const int n = p.comm.n;
  q.rows = n <= 2 ? 128 : (n <= 4 ? 64 : 32);
  q.pieces_per_unit = 128 / q.rows;
  q.slot_bytes = (n - 1) * q.rows * 256;
  q.slots = ring_bytes / q.slot_bytes;
  if (q.slots > 8) q.slots = 8;
  q.sub_per_row = (p.N + 127) / 128;
  q.owned_units = ((p.M / n) / 128) * q.sub_per_row;
  return q;
}

// piece index -> rows and columns.  lrow0: first local row; grow0: the same row in the full matrix.
__device__ __forceinline__ void rs_piece_coords(const GemmParams& p, const RsPlan& q, int piece, long long& lrow0,
                                                long long& grow0, int& col0, int& row_bytes, int& unit_flag) {
  const GemmComm& c = p.comm;
  const int unit = piece / q.pieces_per_unit, part = piece - unit * q.pieces_per_unit;
  const int lb = unit / q.sub_per_row, sn = unit - lb * q.sub_per_row;
  const long long l0 = (long long)lb * 128;
  const long long b = l0 / c.seg_rows;
  const long long g0 = (b * c.n + c.rank) * c.seg_rows + (l0 - b * c.seg_rows);
  const int m_blk = (int)(g0 / kPairBlockM), cta_p = (int)((g0 % kPairBlockM) / 128);
  unit_flag = ((m_blk * p.num_n_blocks + (sn >> 1)) * 2 + cta_p) * 2 + (sn & 1);
  lrow0 = l0 + part * q.rows;
  grow0 = g0 + part * q.rows;
  col0 = sn * 128;
  row_bytes = min(128, p.N - col0) * 2;
}

// producer: one warp.  Lane 0 claims pieces from the queue, waits for their flags and for a free slot;
// the claimed index (or -1 at the end) is handed to the consumers through `slot_piece`; all 32 lanes
// issue the row copies (a single thread issuing 128 copies per piece was the bottleneck of this phase).
// `drain_ring`: the caller is a compute CTA whose operand ring may still be read by UMMAs: continue
// the ring's bookkeeping (`stage` / `phase`) until every stage has been released.
__device__ __forceinline__ void rs_pull_producer(const GemmParams& p, uint8_t* ring, int ring_bytes,
                                                 uint64_t* empty_bar, uint64_t* pull_full, uint64_t* pull_empty,
                                                 volatile int* slot_piece, bool drain_ring, int stage, uint32_t phase,
                                                 volatile int* abort_flag) {
  const GemmComm& c = p.comm;
  const int n = c.n;
  const int lane = threadIdx.x & 31;
  bool ok = true;
  if (drain_ring && lane == 0) {
    for (int i = 0; i < kPairStages && ok; ++i) {
      ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status);
      if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
    }
  }
  const RsPlan q = rs_plan(p, ring_bytes);
  const uint32_t* my_flags = c.tile_flags[c.rank];
  const int total_pieces = q.owned_units * q.pieces_per_unit;
  int slot = 0;
  uint32_t sphase = 0;
  while (true) {
    int piece = -1;
    long long lrow0 = 0, grow0 = 0;
    int col0 = 0, row_bytes = 0, uf = 0;
    if (lane == 0) {
      piece = ok ? (int)atomicAdd(c.rs_queue, 1u) : total_pieces;
      if (piece >= total_pieces) piece = -1;
      if (!mbar_wait(smem_u32(&pull_empty[slot]), sphase ^ 1u, abort_flag, p.status)) piece = -2;   // give up silently
      if (piece >= 0) {
        rs_piece_coords(p, q, piece, lrow0, grow0, col0, row_bytes, uf);
        for (int k = 0; k < n && ok; ++k) {          // every rank's partial product of this sub-tile exists
          const uint32_t* f = my_flags + (size_t)k * c.units_total + uf;
          const long long t0 = clock64();
          while ((int32_t)(ld_acquire_sys_u32(f) - c.epoch) < 0) {
            if (*abort_flag || clock64() - t0 > c.budget) {
              *abort_flag = 1;
              raise_status(p.status, kStatusFlagTimeout);
              ok = false;
              break;
            }
            __nanosleep(64);
          }
        }
        if (!ok) piece = -1;
      }
      if (piece >= -1) {
        slot_piece[slot] = piece;
        if (piece < 0) mbar_arrive(smem_u32(&pull_full[slot]));                 // tells the consumers to stop
        else mbar_arrive_expect_tx(smem_u32(&pull_full[slot]), (uint32_t)((n - 1) * q.rows * row_bytes));
      }
    }
    piece = __shfl_sync(0xffffffffu, piece, 0);
    if (piece < 0) return;
    grow0 = __shfl_sync(0xffffffffu, grow0, 0);
    col0 = __shfl_sync(0xffffffffu, col0, 0);
    row_bytes = __shfl_sync(0xffffffffu, row_bytes, 0);
    const uint32_t fb = smem_u32(&pull_full[slot]);
    uint32_t dst = smem_u32(ring + slot * q.slot_bytes);
    for (int k = 0; k < n; ++k) {
      if (k == c.rank) continue;
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(c.peer[k]) + grow0 * (long long)p.N + col0;
      for (int r = lane; r < q.rows; r += 32)
        bulk_g2s(dst + r * 256, src + (long long)r * p.N, (uint32_t)row_bytes, fb);
      dst += q.rows * 256;
    }
    if (++slot == q.slots) { slot = 0; sphase ^= 1u; }
  }
}

// consumer: the 256 threads of warps 2..9.
__device__ __forceinline__ void rs_pull_consumer(const GemmParams& p, uint8_t* ring, int ring_bytes,
                                                 uint64_t* pull_full, uint64_t* pull_empty, volatile int* slot_piece,
                                                 volatile int* abort_flag) {
  const GemmComm& c = p.comm;
  const int n = c.n;
  const int tid = (int)threadIdx.x - 64;
  const RsPlan q = rs_plan(p, ring_bytes);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(c.rs_out);
  const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(c.rs_bias);
  const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(c.peer[c.rank]);
  int slot = 0;
  uint32_t sphase = 0;
  while (true) {
    bool ok = mbar_wait(smem_u32(&pull_full[slot]), sphase, abort_flag, p.status);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return;
    const int piece = slot_piece[slot];
    if (piece < 0) return;
    long long lrow0, grow0;
    int col0, row_bytes, uf;
    rs_piece_coords(p, q, piece, lrow0, grow0, col0, row_bytes, uf);
    const uint8_t* src = ring + slot * q.slot_bytes;
    const int chunks_per_row = row_bytes >> 4;
    const int total = q.rows * chunks_per_row;
    for (int ch0 = tid; ch0 < total; ch0 += 256 * 4) {
      // four independent 16-byte loads of the local partial product in flight per thread
      uint4 own[4];
#pragma unroll
      for (int bq = 0; bq < 4; ++bq) {
        const int ch = ch0 + bq * 256;
        if (ch < total) {
          const int r = ch / chunks_per_row, cv = ch - r * chunks_per_row;
          own[bq] = *reinterpret_cast<const uint4*>(mine + (grow0 + r) * (long long)p.N + col0 + cv * 8);
        }
      }
#pragma unroll
      for (int bq = 0; bq < 4; ++bq) {
        const int ch = ch0 + bq * 256;
        if (ch >= total) continue;
        const int r = ch / chunks_per_row, cv = ch - r * chunks_per_row;
        float acc[8];
        {
          const uint32_t w[4] = {own[bq].x, own[bq].y, own[bq].z, own[bq].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] = f.x; acc[2 * e + 1] = f.y; }
        }
        if (bias != nullptr) {
          const uint4 bb = __ldg(reinterpret_cast<const uint4*>(bias + col0) + cv);
          const uint32_t w[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
        }
        for (int k = 0; k < n - 1; ++k) {
          const uint4 v = *reinterpret_cast<const uint4*>(src + (k * q.rows + r) * 256 + cv * 16);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
        }
        *reinterpret_cast<uint4*>(out + (lrow0 + r) * (long long)p.N + col0 + cv * 8) =
            make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                       pack_bf16x2(acc[6], acc[7]));
      }
    }
    mbar_arrive(smem_u32(&pull_empty[slot]));        // 256 arrivals free the slot
    if (++slot == q.slots) { slot = 0; sphase ^= 1u; }
  }
}

// A CTA that only reduces (one of the first CTAs of the grid): the whole dynamic shared memory is its ring.
__device__ __forceinline__ void rs_reducer_role(const GemmParams& p, uint8_t* smem, int ring_bytes, uint8_t* bar_area) {
  uint64_t* pull_full = reinterpret_cast<uint64_t*>(bar_area + 256);
  uint64_t* pull_empty = pull_full + 8;
  volatile int* slot_piece = reinterpret_cast<volatile int*>(bar_area + 512);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_area + 640);
  if (!(p.comm.phase & 2)) return;                   // multiply-only launch (single-GPU tests)
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < 8; ++s) {
      mbar_init(smem_u32(&pull_full[s]), 1);
      mbar_init(smem_u32(&pull_empty[s]), 256);
    }
    fence_mbar_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  if (warp == 0)
    rs_pull_producer(p, smem, ring_bytes, nullptr, pull_full, pull_empty, slot_piece, false, 0, 0u, abort_flag);
  else if (warp >= 2)
    rs_pull_consumer(p, smem, ring_bytes, pull_full, pull_empty, slot_piece, abort_flag);
}

__global__ void __launch_bounds__(kPairThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_aux,
                      const __grid_constant__ CUtensorMap tma_auxin, const GemmParams p) {
  constexpr uint32_t kTmemCols = 512;   // two 256-column accumulator buffers
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kPairStages * kPairStageBytes;
  uint8_t* bar_base = staging + kPairStagingBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);       // used in the even CTA only
  uint64_t* empty_bar = full_bar + kPairStages;                     // one per CTA
  uint64_t* tmem_full_bar = empty_bar + kPairStages;                // one per CTA
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;                     // used in the even CTA only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* aux_full = reinterpret_cast<uint64_t*>(bar_base + 128);    // per column half: aux_in block has landed
  uint64_t* pull_full = reinterpret_cast<uint64_t*>(bar_base + 256);   // mode 1, reduce phase (8 slots at most)
  uint64_t* pull_empty = pull_full + 8;
  volatile int* slot_piece = reinterpret_cast<volatile int*>(bar_base + 512);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader
  const bool leader = cta == 0;
  const bool a_mn = (p.flags & MRK_GEMM_A_MN) != 0;
  const bool b_mn = (p.flags & MRK_GEMM_B_MN) != 0;

  // fused all-gather (GemmComm mode 2): the clusters in front of the compute clusters only move the peers'
  // shards of A; both CTAs of such a cluster leave together, so no cluster barrier is left waiting
  const int aux_ctas = p.comm.mode != 0 ? (int)gridDim.x - p.comm.gemm_ctas : 0;   // gather / reduce CTAs come first
  if (p.comm.mode == 2 && (int)blockIdx.x < aux_ctas) {
    comm_gather_role(p, smem, kPairStages * kPairStageBytes + kPairStagingBytes);
    return;
  }
  // fused reduce-scatter (mode 1): the clusters in front of the compute clusters only reduce
  if (p.comm.mode == 1 && (int)blockIdx.x < aux_ctas) {
    rs_reducer_role(p, smem, kPairStages * kPairStageBytes + kPairStagingBytes, bar_base);
    return;
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), 2 * 8);        // one arrival per epilogue warp of both CTAs
    }
    for (int s = 0; s < 8; ++s) {
      mbar_init(smem_u32(&pull_full[s]), 1);
      mbar_init(smem_u32(&pull_empty[s]), 256);
    }
    mbar_init(smem_u32(&aux_full[0]), 1);
    mbar_init(smem_u32(&aux_full[1]), 1);
    fence_mbar_init();
    if (p.tma_aux_in) tma_prefetch_desc(&tma_auxin);
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.tma_store) tma_prefetch_desc(&tma_c);
    if (p.tma_store_aux) tma_prefetch_desc(&tma_aux);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();                  // both CTAs' barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int cluster_id = ((int)blockIdx.x - aux_ctas) >> 1;
  const int num_clusters = (p.comm.mode != 0 ? p.comm.gemm_ctas : (int)gridDim.x) >> 1;
  const bool rs = p.comm.mode == 1;
  // reduce-only launches (single-GPU tests of the reduce phase) skip the multiplication
  const int num_units = (rs && p.comm.phase == 2) ? 0 : p.num_m_blocks * p.num_n_blocks * p.num_splits;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    int rs_stage = 0;
    uint32_t rs_phase = 0;
    bool rs_ok = true;
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters) {
        int m_blk, n_blk;
        tile_coords(unit / p.num_splits, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
        m_blk = comm_perm_m(p, m_blk, kPairBlockM);
        const int m0 = m_blk * kPairBlockM + (int)cta * 128;
        const int n0 = n_blk * kPairBlockN + (int)cta * (kPairBlockN / 2);
        const int kb_begin = (unit % p.num_splits) * p.kb_per_split;
        const int kb_end = min(p.num_k_blocks, kb_begin + p.kb_per_split);
        if (p.comm.mode == 2 && m0 < p.M) {       // this CTA's 128 rows of A must have arrived
          ok = comm_wait_rows(p, m0, 128, abort_flag);
          if (!ok) break;
        }
        for (int kb = kb_begin; kb < kb_end; kb += kPairGroup) {
          const int nsub = min(kPairGroup, kb_end - kb);
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          if (leader) mbar_arrive_expect_tx(fb, (uint32_t)(nsub * 2 * kPairSubBytes));   // bytes of both CTAs
          for (int sub = 0; sub < nsub; ++sub) {
            const uint32_t sa = smem_u32(smem + stage * kPairStageBytes + sub * kPairSubBytes);
            const uint32_t sb = sa + kPairABytes;
            const int k0 = (kb + sub) * kPairBlockK;
            if (!a_mn) {
              tma_load_2d_pair(sa, &tma_a, fb, k0, m0);
            } else {
#pragma unroll
              for (int atom = 0; atom < 2; ++atom)
                tma_load_2d_pair(sa + atom * (kPairBlockK * 128), &tma_a, fb, m0 + atom * 64, k0);
            }
            if (!b_mn) {
              tma_load_2d_pair(sb, &tma_b, fb, k0, n0);
            } else {
#pragma unroll
              for (int atom = 0; atom < 2; ++atom)
                tma_load_2d_pair(sb + atom * (kPairBlockK * 128), &tma_b, fb, n0 + atom * 64, k0);
            }
          }
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
      rs_stage = stage;
      rs_phase = phase;
      rs_ok = ok;
    }
    if (rs && (p.comm.phase & 2)) {               // reduce phase: the whole warp drives the pulls
      __syncwarp();
      rs_ok = __shfl_sync(0xffffffffu, (int)rs_ok, 0) != 0;
      if (rs_ok)
        rs_pull_producer(p, smem, kPairStages * kPairStageBytes, empty_bar, pull_full, pull_empty, slot_piece, true,
                         rs_stage, rs_phase, abort_flag);
    }
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer (leader CTA) -------------------------------
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_bf16(kPairBlockM, kPairBlockN, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1u, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBlockN;
        const int kb_begin = (unit % p.num_splits) * p.kb_per_split;
        const int kb_end = min(p.num_k_blocks, kb_begin + p.kb_per_split);
        for (int kb = kb_begin; kb < kb_end; kb += kPairGroup) {
          const int nsub = min(kPairGroup, kb_end - kb);
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          for (int sub = 0; sub < nsub; ++sub) {
            const uint32_t sa = smem_u32(smem + stage * kPairStageBytes + sub * kPairSubBytes);
            const uint32_t sb = sa + kPairABytes;
#pragma unroll
            for (int k = 0; k < kPairBlockK / 16; ++k) {
              const uint64_t da = a_mn ? desc_mnmajor(sa, k, kPairBlockK) : desc_kmajor(sa, k);
              const uint64_t db = b_mn ? desc_mnmajor(sb, k, kPairBlockK) : desc_kmajor(sb, k);
              umma_bf16_ss_pair(d_tmem, da, db, idesc, (kb != kb_begin || sub != 0 || k != 0) ? 1u : 0u);
            }
          }
          // release this stage in both CTAs once the UMMAs above have read it
          umma_commit_pair_both(smem_u32(&empty_bar[stage]));
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          umma_commit_pair_both(smem_u32(&tmem_full_bar[acc]));
        }
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -------------------------------
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    // two warps share a TMEM lane quadrant: warps 2..5 take the left half of the columns, 6..9 the right
    const int half = (warp - 2) >> 2;
    uint8_t* stage = staging + half * 16384;        // one 128 x 64 bf16 box, reused by the two 64-column passes
    const bool store_thread = (warp == 2 + half * 4) && lane == 0;     // issues this half's TMA stores
    bool box_busy = false;     // a TMA store that reads the box may still be in flight
    uint32_t aux_phase = 0;    // parity of this half's aux_in barrier
    int iter = 0;
    bool ok = true;
    int pending_flag = -1, pending_owner = 0;     // mode 1: sub-tile whose stores are in flight (store thread)
    // before the box is overwritten: its last store must have read it (128 threads of this half)
    auto box_acquire = [&]() __attribute__((always_inline)) {
      if (box_busy) {
        if (store_thread) tma_store_wait_read<0>();
        named_bar_sync(1 + half, 128);
      }
    };
    // after the box is written: one thread hands it to the TMA unit
    auto box_store = [&](const CUtensorMap* map, int col, long long row0) __attribute__((always_inline)) {
      fence_proxy_async_smem();
      named_bar_sync(1 + half, 128);
      if (store_thread) {
        if (row0 < p.M) tma_store_2d(map, smem_u32(stage), col, (int32_t)row0);
        tma_store_commit();
      }
      box_busy = true;
    };
    for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters, ++iter) {
      int m_blk, n_blk;
      tile_coords(unit / p.num_splits, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
      m_blk = comm_perm_m(p, m_blk, kPairBlockM);
      const bool split_k = p.num_splits > 1;
      const bool first_split = (unit % p.num_splits) == 0;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      const long long row0 = (long long)m_blk * kPairBlockM + (long long)cta * 128;
      const long long row = row0 + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * kPairBlockN;
      const int col_half = n_blk * kPairBlockN + half * (kPairBlockN / 2);
      // staged output for this block? (uniform over the four warps of the half)
      const bool staged32 = p.tma_store == 2 && col_half < p.N;     // fp32 output: boxes of 32 columns
      const bool staged = p.tma_store == 1 && !split_k && col_half < p.N &&
                          (col_half + kPairBlockN / 2 <= p.N || (p.aux_mode == MRK_AUX_NONE && p.aux_out == nullptr));
      // aux_in (residual, or the saved pre-activation of a backward GEMM) comes into the box by TMA
      const bool aux_tma = staged && p.tma_aux_in && p.aux_mode != MRK_AUX_NONE &&
                           !(p.tma_store_aux && p.aux_out != nullptr);
      auto aux_fetch = [&](int col) __attribute__((always_inline)) {        // the box is free: start the load of its aux_in block
        if (store_thread) {
          mbar_arrive_expect_tx(smem_u32(&aux_full[half]), 16384u);
          tma_load_2d(smem_u32(stage), &tma_auxin, smem_u32(&aux_full[half]), col, (int32_t)row0);
        }
      };
      if (aux_tma) {      // the first block's load overlaps the wait for the accumulator
        box_acquire();
        aux_fetch(col_half);
      }
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (rs && store_thread && pending_flag >= 0) {
        // fused reduce-scatter: the previous sub-tile's stores have landed; tell the owner of the rows
        tma_store_wait<0>();
        rs_publish(p, pending_owner, pending_flag);
        pending_flag = -1;
      }
      auto release_tmem = [&]() __attribute__((always_inline)) {
        tc_fence_before();
        __syncwarp();            // every lane's TMEM reads are complete: one (possibly remote) arrival per warp
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));   // TMEM is free
      };
      if (staged) {
        const bool two_pass = p.tma_store_aux && p.aux_out != nullptr;
        const int npass = (col_half + 64 < p.N) ? 2 : 1;        // 64-column passes with anything to write
        for (int b = 0; b < npass; ++b) {
          const int col_b = col_half + b * 64;
          const uint32_t t_b = t_row + half * (kPairBlockN / 2) + b * 64;
          if (two_pass) {
            // the pre-activation side output of these columns first, through the same box
            box_acquire();
            epilogue_tile(p, row, row_ok, t_b, col_b, 64, split_k, first_split, stage, row_in_tile, 1);
            box_store(&tma_aux, col_b, row0);
          }
          if (aux_tma) {
            if (b > 0) {
              box_acquire();
              aux_fetch(col_b);
            }
            ok = mbar_wait(smem_u32(&aux_full[half]), aux_phase, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            aux_phase ^= 1u;
            if (!ok) break;
          } else {
            box_acquire();
          }
          epilogue_tile(p, row, row_ok, t_b, col_b, 64, split_k, first_split, stage, row_in_tile,
                        aux_tma ? 8 : (two_pass ? 2 : 0));
          if (b == npass - 1) release_tmem();
          box_store(&tma_c, col_b, row0);
        }
        if (rs && store_thread && row0 < p.M) {
          pending_flag = ((m_blk * p.num_n_blocks + n_blk) * 2 + (int)cta) * 2 + half;
          pending_owner = (int)((row0 / p.comm.seg_rows) % p.comm.n);
        }
      } else if (staged32) {
        // fp32 output through the same box, 32 columns (one 128-byte row per output row) at a time: a plain
        // store, or an element-wise add when the GEMM accumulates into its output or splits K
        const bool add = split_k || (p.flags & MRK_GEMM_ACCUMULATE) != 0;
        const int npass = min(4, (p.N - col_half + 31) / 32);
        for (int b = 0; b < npass; ++b) {
          const int col_b = col_half + b * 32;
          box_acquire();
          epilogue_tile(p, row, row_ok, t_row + half * (kPairBlockN / 2) + b * 32, col_b, 32, split_k, first_split,
                        stage, row_in_tile, 3);
          if (b == npass - 1) release_tmem();
          fence_proxy_async_smem();
          named_bar_sync(1 + half, 128);
          if (store_thread) {
            if (row0 < p.M) {
              if (add) tma_reduce_add_2d(&tma_c, smem_u32(stage), col_b, (int32_t)row0);
              else tma_store_2d(&tma_c, smem_u32(stage), col_b, (int32_t)row0);
            }
            tma_store_commit();
          }
          box_busy = true;
        }
      } else {
        epilogue_tile(p, row, row_ok, t_row + half * (kPairBlockN / 2), col_half, kPairBlockN / 2, split_k,
                      first_split, nullptr, row_in_tile, 0);
        release_tmem();
      }
    }
    if (store_thread) {
      if (rs) {
        tma_store_wait<0>();
        if (pending_flag >= 0) rs_publish(p, pending_owner, pending_flag);
      } else {
        tma_store_wait_read<0>();     // shared memory stays valid until the last store has read it
      }
    }
    // ------------------- mode 1: reduce the sub-tiles this rank owns (all 8 epilogue warps) -------------------
    if (rs && (p.comm.phase & 2) && ok)
      rs_pull_consumer(p, smem, kPairStages * kPairStageBytes, pull_full, pull_empty, slot_piece, abort_flag);
  }

  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();                  // nobody leaves while its partner may still touch it
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& taux,
                     const CUtensorMap& tauxin, GemmParams& p, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  MRK_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MRK_CUDA_OK(cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kPairSmemTotal));
    configured[dev & 63] = true;
  }
  p.num_m_blocks = (p.M + kPairBlockM - 1) / kPairBlockM;
  p.num_n_blocks = (p.N + kPairBlockN - 1) / kPairBlockN;
  p.num_k_blocks = (p.K + kPairBlockK - 1) / kPairBlockK;
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int max_clusters = sm_count() / 2;
  p.num_splits = 1;
  const bool can_split = (p.flags & MRK_GEMM_OUT_F32) && (p.flags & MRK_GEMM_ACCUMULATE) &&
                         p.act == MRK_ACT_NONE && p.aux_mode == MRK_AUX_NONE && p.aux_out == nullptr;
  if (can_split && p.num_k_blocks >= 16) {
    // Weight gradients have few output tiles and a long K: pick the number of K ranges whose units fill
    // whole rounds of the clusters best.  Cost of `s` ranges, in k-blocks: rounds x (k-blocks per unit + a
    // fixed charge per unit for pipeline fill and the extra pass over the output).
    const int max_by_k = p.num_k_blocks / 8;
    long long best_cost = 0;
    for (int sp = 1; sp <= 32 && sp <= max_by_k; ++sp) {
      const int kb = (p.num_k_blocks + sp - 1) / sp;
      const int nsp = (p.num_k_blocks + kb - 1) / kb;
      const long long rounds = ((long long)tiles * nsp + max_clusters - 1) / max_clusters;
      const long long cost = rounds * (kb + 6);
      if (sp == 1 || cost < best_cost) { best_cost = cost; p.num_splits = nsp; }
    }
  }
  p.kb_per_split = (p.num_k_blocks + p.num_splits - 1) / p.num_splits;
  p.num_splits = (p.num_k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  const int units = tiles * p.num_splits;
  int clusters = units < max_clusters ? units : max_clusters;
  int gather_clusters = 0;
  if (p.comm.mode == 2) {
    // compute clusters + gather clusters, all resident at once: the former wait for the latter
    gather_clusters = (p.comm.gemm_ctas + 1) / 2;       // the caller passes the number of gather CTAs here
    MRK_REQUIRE(gather_clusters >= 1 && gather_clusters < max_clusters, "gemm: bad number of gather CTAs");
    const int room = max_clusters - gather_clusters;
    clusters = units < room ? units : room;
    p.comm.gemm_ctas = 2 * clusters;
  }
  if (p.comm.mode != 0 && p.comm.perm)
    p.comm.perm = (p.comm.seg_rows % kPairBlockM == 0 && p.num_m_blocks % p.comm.n == 0 && p.M % kPairBlockM == 0) ? 1 : 0;
  if (p.comm.mode == 1) {
    MRK_REQUIRE(p.tma_store == 1 && p.num_splits == 1, "gemm_rs: the partial product must leave through TMA stores");
    MRK_REQUIRE(p.comm.units_total == p.num_m_blocks * p.num_n_blocks * 4, "gemm_rs: flag array does not match the tiling");
    MRK_REQUIRE(p.comm.rs_queue != nullptr, "gemm_rs: no work queue");
    // compute clusters + reducer clusters, all resident at once (the reducers must run from the start)
    gather_clusters = (p.comm.reduce_ctas + 1) / 2;
    if (gather_clusters >= max_clusters) gather_clusters = max_clusters / 2;
    const int room = max_clusters - gather_clusters;
    clusters = units < room ? units : room;
    if (p.comm.phase == 2) clusters = room;            // reduce-only launch: everybody reduces
    p.comm.gemm_ctas = 2 * clusters;
    MRK_CUDA_OK(cudaMemsetAsync(p.comm.rs_queue, 0, sizeof(uint32_t), stream));
  }

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (clusters + gather_clusters), 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p.num_splits > 1 && p.tma_store == 1) p.tma_store = 0;
  if (!p.tma_store) p.tma_store_aux = 0;
  if (p.tma_store != 1) p.tma_aux_in = 0;
  MRK_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel, ta, tb, tc, taux, tauxin, p));
  count_launch();
  return 0;
}

}  // namespace mrk
