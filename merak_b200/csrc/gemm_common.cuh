// Pieces shared by the single-CTA and the CTA-pair GEMM kernels: parameter block, activation
// functions, tile rasterisation and the accumulator epilogue (TMEM -> registers -> global).
#pragma once
#include "gemm_tcgen05.h"
#include "sm100_ptx.cuh"
#include "activations.cuh"
#include "symm.cuh"

namespace mrk {

// Collective fused into the GEMM (tensor parallelism over peer-mapped memory).
//   mode 2  all-gather -> GEMM: a few CTAs of the grid stream the peers' shards of A into the local
//           gathered matrix (bulk async copies peer -> shared -> local, many in flight) segment by
//           segment and publish a counter per segment; the TMA producers of the compute CTAs wait
//           for the segments their tile covers, starting with this rank's own rows.  Each remote
//           element crosses NVLink once.
//   mode 1  GEMM -> reduce-scatter (CTA-pair kernel): every rank multiplies its slice of the
//           contraction and writes the bf16 partial product of each 128 x 128 sub-tile into its own
//           peer-mapped buffer, then stores the call's epoch into the flag of that sub-tile in the
//           control memory of the rank that owns those rows.  Row blocks are visited with this
//           rank's own segments last, so what the peers need first is produced first.  When a CTA
//           has finished its tiles, its epilogue warps turn to the sub-tiles this rank owns: they
//           wait for the n flags of a sub-tile, pull the n partials (bulk copies over NVLink into
//           shared memory), sum them in fp32, add the bias and write the reduced rows.  A few
//           CTAs of the grid do nothing else from the start, so the sum of this rank's own
//           segment (whose last contribution is this rank's own, by the order above) runs under
//           the multiplication of the remaining tiles; pieces are claimed from a queue, which the
//           compute CTAs join when their tiles are done.  One launch, no barrier over the group.
// Rows of the full [M, *] matrix are grouped in segments of `seg_rows`; segment s belongs to rank
// s % n and is that rank's local segment s / n (batch-first sequence sharding).
constexpr int kGemmMaxPeers = 8;
constexpr int kGatherWorkers = 2;     // issuing threads per gather CTA (lane 0 of warps 0..W-1), each with its own slots
struct GemmComm {
  int mode, n, rank;
  int seg_rows;
  int perm;                    // start the row-block order at this rank's own segments
  int gemm_ctas;               // modes 1, 2: the LAST gemm_ctas CTAs of the grid compute; the ones before them
                               // gather / reduce.  They come first because blocks are handed to SMs in index
                               // order: if something else holds SMs, it is compute CTAs that start late (they
                               // only wait for data), never the CTAs everybody else waits for.
  void* peer[kGemmMaxPeers];   // bf16 shards of A, one per rank
  long long ld_peer;           // row pitch of those (elements)
  void* gathered;              // mode 2: local gathered A, row pitch ld_peer
  uint32_t* seg_flags;         // mode 2: local, one counter per segment
  void* ctrl[kGemmMaxPeers];   // control blocks (entry barrier of mode 2)
  uint32_t epoch;              // barrier epoch of this call
  uint32_t flag_target;        // mode 2: gather CTAs of all calls so far; a segment is complete when its
                               // counter reaches flag_target * kGatherWorkers
  long long budget;            // wait budget in SM cycles
  // mode 1
  uint32_t* tile_flags[kGemmMaxPeers];   // per rank: [n sources][units_total] epochs, peer-mapped
  int units_total;             // sub-tiles of the full output: num_m_blocks * num_n_blocks * 4
  int own_last;                // row-block order ends (instead of starts) with this rank's own segments
  int phase;                   // 3 = multiply and reduce; 1 = multiply only; 2 = reduce only (tests on one GPU)
  int reduce_ctas;             // CTAs behind the compute CTAs that only reduce (resident from the start)
  uint32_t* rs_queue;          // work queue of the reduce phase: next piece to claim (zero at launch)
  void* rs_out;                // [M / n, N] bf16, this rank's reduced rows
  const void* rs_bias;         // optional bf16 [N]
};

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const void* bias;
  const __nv_bfloat16* aux_in;
  long long ld_aux_in;
  __nv_bfloat16* aux_out;
  long long ld_aux_out;
  int act;        // MrkAct
  int aux_mode;   // MrkAuxMode
  int flags;      // MrkGemmFlags
  float alpha;
  unsigned* status;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  int num_splits, kb_per_split;   // split-K: work unit = (tile, split); partial sums meet in fp32 red.add
  int tma_store;                  // C leaves through shared memory + the TMA unit: 1 = bf16 stores (no accumulate), 2 = fp32 stores or adds
  int tma_store_aux;              // ... and the pre-activation side output too (second tensor map)
  int tma_aux_in;                 // aux_in blocks can be brought in with TMA loads (third tensor map)
  GemmComm comm;
};

// Row-block order under a fused collective: position i of the schedule -> row block.  Blocks are
// visited by distance of their owner from this rank (own segments first), so every rank works on a
// different peer's rows at any time.
__device__ __forceinline__ int comm_perm_m(const GemmParams& p, int i, int block_m) {
  const GemmComm& c = p.comm;
  if (c.mode == 0 || !c.perm) return i;
  const int blocks_per_seg = c.seg_rows / block_m;
  const int per_owner = p.num_m_blocks / c.n;
  const int d = i / per_owner, j = i - d * per_owner;
  const int b = j / blocks_per_seg, w = j - b * blocks_per_seg;
  int owner = c.rank + d + (c.own_last ? 1 : 0);
  if (owner >= c.n) owner -= c.n;
  return (b * c.n + owner) * blocks_per_seg + w;
}

// mode 2, TMA producer thread: waits until the segments covering rows [m0, m0 + rows) have arrived.
__device__ __forceinline__ bool comm_wait_rows(const GemmParams& p, int m0, int rows, volatile int* abort_flag) {
  const GemmComm& c = p.comm;
  const int last_row = min(m0 + rows, p.M) - 1;
  const int s0 = m0 / c.seg_rows, s1 = last_row / c.seg_rows;
  for (int s = s0; s <= s1; ++s) {
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys_u32(c.seg_flags + s) - c.flag_target * kGatherWorkers) < 0) {
      if (*abort_flag || clock64() - t0 > c.budget) {
        *abort_flag = 1;
        raise_status(p.status, kStatusFlagTimeout);
        return false;
      }
      __nanosleep(64);
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");   // the copies were generic-proxy stores; TMA reads next
  return true;
}

// mode 2, gather CTAs: stream every rank's shard into the gathered matrix, own segments first.
// One thread per CTA drives a ring of shared-memory slots with bulk async copies (peer or local
// global -> shared, then shared -> local global), so that about 190 KB per CTA are in flight over
// NVLink; plain loads from a few CTAs cannot cover the link latency.
constexpr int kGatherChunk = 32768;

__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void comm_gather_role(const GemmParams& p, uint8_t* smem, int smem_bytes) {
  const GemmComm& c = p.comm;
  const int cta_g = blockIdx.x;                 // the gather CTAs are the first ones of the grid
  const int worker = threadIdx.x >> 5;
  const int g = cta_g * kGatherWorkers + worker, G = (gridDim.x - c.gemm_ctas) * kGatherWorkers;
  SymmCtrl* mine = reinterpret_cast<SymmCtrl*>(c.ctrl[c.rank]);
  PeerPtrs ctrls;
#pragma unroll
  for (int k = 0; k < kGemmMaxPeers; ++k) ctrls.p[k] = c.ctrl[k];
  // every rank has staged its shard (and is done with the previous use of its buffers)
  if (cta_g == 0) symm_signal(ctrls, c.n, c.rank, 4, c.epoch);
  const bool ok = symm_wait(mine, c.n, 4, c.epoch, c.budget, p.status);
  // on a timeout the consumers run out on the segment counters
  if (!ok || worker >= kGatherWorkers || (threadIdx.x & 31) != 0) return;

  const int total_slots = (smem_bytes - 512) / kGatherChunk;
  const int slots = total_slots / kGatherWorkers;
  uint8_t* bar_area = smem + total_slots * kGatherChunk;
  smem += worker * slots * kGatherChunk;            // this worker's ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(bar_area) + worker * 8;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_area + 256) + worker;
  *abort_flag = 0;
  for (int s = 0; s < slots; ++s) mbar_init(smem_u32(&bars[s]), 1);
  fence_mbar_init();

  const int num_seg = p.M / c.seg_rows;
  const int batches = num_seg / c.n;
  const long long seg_bytes = (long long)c.seg_rows * c.ld_peer * 2;
  const int chunks_per_seg = (int)((seg_bytes + kGatherChunk - 1) / kGatherChunk);
  const int mine_per_seg = chunks_per_seg > g ? (chunks_per_seg - g + G - 1) / G : 0;   // chunks g, g+G, ...
  const long long total = (long long)mine_per_seg * num_seg;
  // chunk i of this CTA: segment order position i / mine_per_seg, chunk g + (i % mine_per_seg) * G
  auto locate = [&](long long i, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes, int& seg) {
    const int pos = (int)(i / mine_per_seg), ci = g + (int)(i % mine_per_seg) * G;
    const int d = pos / batches, b = pos - d * batches;
    int owner = c.rank + d;
    if (owner >= c.n) owner -= c.n;
    seg = b * c.n + owner;
    const long long off = (long long)ci * kGatherChunk;
    bytes = (uint32_t)min((long long)kGatherChunk, seg_bytes - off);
    src = reinterpret_cast<const uint8_t*>(c.peer[owner]) + (long long)b * seg_bytes + off;
    dst = reinterpret_cast<uint8_t*>(c.gathered) + (long long)seg * seg_bytes + off;
  };
  long long head = 0, tail = 0;
  bool good = true;
  while (tail < total && good) {
    // At most slots - 2 loads are in flight, so the slot a new load lands in was last read by a store
    // issued at least two stores ago: waiting until no more than one store is still reading shared
    // memory frees it without draining the store queue.
    while (head < total && head - tail < slots - 1) {
      const int slot = (int)(head % slots);
      if (head >= slots)
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      const uint8_t* src; uint8_t* dst; uint32_t bytes; int seg;
      locate(head, src, dst, bytes, seg);
      mbar_arrive_expect_tx(smem_u32(&bars[slot]), bytes);
      bulk_g2s(smem_u32(smem + slot * kGatherChunk), src, bytes, smem_u32(&bars[slot]));
      ++head;
    }
    const int slot = (int)(tail % slots);
    good = mbar_wait(smem_u32(&bars[slot]), (uint32_t)((tail / slots) & 1), abort_flag, p.status);
    if (!good) break;
    const uint8_t* src; uint8_t* dst; uint32_t bytes; int seg;
    locate(tail, src, dst, bytes, seg);
    bulk_s2g(dst, smem_u32(smem + slot * kGatherChunk), bytes);
    ++tail;
    if (tail % mine_per_seg == 0) {      // this CTA's part of the segment is on its way: complete and publish
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence();
      atomicAdd(c.seg_flags + seg, 1u);
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (mine_per_seg == 0 && good)         // more gather CTAs than chunks: still count for every segment
    for (int s = 0; s < num_seg; ++s) atomicAdd(c.seg_flags + s, 1u);
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  // Grouped raster: 8 row-blocks share their B panel in L2 before the next group starts.
  constexpr int kGroup = 8;
  const int per_group = kGroup * num_n;
  const int g = tile / per_group;
  const int first_m = g * kGroup;
  const int gsz = min(num_m - first_m, kGroup);
  const int r = tile - g * per_group;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

// Epilogue of one accumulator tile for one thread: `row` is this thread's output row, `t_row` the
// TMEM address of its lane at the tile's first column, `col_base` the first output column of the
// tile and `ncols` its width.  All 32 lanes of the warp call this together.
// `stage` (optional): shared-memory staging of this warp group's 128 x 128 output block, laid out as
// two 128-row x 64-column boxes in the 128-byte TMA swizzle; when given, the finished bf16 values go
// there (row `r_in_tile`) instead of to global memory and the caller issues the TMA stores.  The
// caller only passes it for tiles where that is legal (bf16 output, no accumulate, no split-K, and
// either a full-width block or no side tensors).
template <int kAct, int kAux>
__device__ __noinline__ void epilogue_tile_t(const GemmParams& p, long long row, bool row_ok, uint32_t t_row,
                                              int col_base, int ncols, bool split_k, bool first_split,
                                              uint8_t* stage, int r_in_tile, int pass) {
  const bool out_f32 = (p.flags & MRK_GEMM_OUT_F32) != 0;
  const bool accumulate = (p.flags & MRK_GEMM_ACCUMULATE) != 0;
  const bool bias_f32 = (p.flags & MRK_GEMM_BIAS_F32) != 0;
  const bool vec_ok = ((p.ldc & 7) == 0) && ((p.ld_aux_in & 7) == 0) && ((p.ld_aux_out & 7) == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.aux_in) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.aux_out) & 15) == 0);
// Two chunks of 32 columns per TMEM round trip: a load that queues behind the tensor core's own
// accumulator traffic takes about a thousand cycles, and one chunk at a time that latency was most
// of the epilogue.
const int nchunks = min(ncols / 32, (p.N - col_base + 31) / 32);     // uniform across the warp
#pragma unroll 1
for (int c2 = 0; c2 < nchunks; c2 += 2) {
  uint32_t r2[2][32];
  tmem_ld32(t_row + c2 * 32, r2[0]);
  tmem_ld32(t_row + min(c2 + 1, nchunks - 1) * 32, r2[1]);      // (an odd tail re-reads its own chunk)
  tmem_wait_ld();
#pragma unroll
for (int h = 0; h < 2; ++h) {
  const int c = c2 + h;
  if (c >= nchunks) continue;
  const int col0 = col_base + c * 32;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r2[h][j]) * p.alpha;
  const bool full = (col0 + 32 <= p.N);
  if (p.bias != nullptr && first_split) {
    const bool bias_vec = full && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
    if (bias_f32) {
      const float* b = reinterpret_cast<const float*>(p.bias) + col0;
      if (bias_vec) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(b) + q);
          v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (full || col0 + j < p.N) v[j] += __ldg(b + j);
      }
    } else {
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
      if (bias_vec) {       // the same 64 bytes for every lane: four broadcast loads instead of 32 scalar ones
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 t = __ldg(reinterpret_cast<const uint4*>(b) + q);
          const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16x2(w[e]);
            v[8 * q + 2 * e] += f.x;
            v[8 * q + 2 * e + 1] += f.y;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (full || col0 + j < p.N) v[j] += __bfloat162float(__ldg(b + j));
      }
    }
  }
  if (stage != nullptr) {
    // shared-memory staged output: side tensors are only present on full-width blocks here.
    // pass 1 stages the pre-activation side output alone, pass 2 the main output without it; pass 0
    // does the main output and writes a side output, if any, directly; pass 3 is pass 0 with an
    // fp32 box of 32 columns (weight gradients).  Pass 8: like pass 0, and the caller has brought the
    // aux_in block into the box with a TMA load (a thread owns a row, so loading it from global memory
    // touches 32 lines per instruction); the result overwrites it in place.
    if (pass == 1) {
      uint8_t* box = stage + (c >> 1) * 16384;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t off = sw128_offset((uint32_t)r_in_tile, (uint32_t)((c & 1) * 4 + q));
        *reinterpret_cast<uint4*>(box + off) =
            make_uint4(pack_bf16x2(v[8 * q + 0], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                       pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
      }
      continue;
    }
    if ((pass == 0 || pass == 3 || pass == 8) && p.aux_out != nullptr && row_ok) {
      uint4* dst = reinterpret_cast<uint4*>(p.aux_out + row * p.ld_aux_out + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        dst[q] = make_uint4(pack_bf16x2(v[8 * q + 0], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                            pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
    }
    if (kAct != MRK_ACT_NONE && kAux != MRK_AUX_DACT) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act<kAct>(v[j]);
    }
    if (kAux != MRK_AUX_NONE && (row_ok || pass == 8)) {
      const uint4* src = reinterpret_cast<const uint4*>(p.aux_in + row * p.ld_aux_in + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 a = pass == 8 ? *reinterpret_cast<const uint4*>(stage + (c >> 1) * 16384 +
                                                                    sw128_offset((uint32_t)r_in_tile, (uint32_t)((c & 1) * 4 + q)))
                                  : __ldg(src + q);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(w[e]);
          if (kAux == MRK_AUX_ADD) {
            v[8 * q + 2 * e] += f.x;
            v[8 * q + 2 * e + 1] += f.y;
          } else {
            v[8 * q + 2 * e] *= apply_act_grad<kAct>(f.x);
            v[8 * q + 2 * e + 1] *= apply_act_grad<kAct>(f.y);
          }
        }
      }
    }
    if (pass == 3) {
      // fp32 box: these 32 columns are one 128-byte row; the caller stores it or adds it into the output
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(stage + sw128_offset((uint32_t)r_in_tile, (uint32_t)q)) =
            make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      continue;
    }
    uint8_t* box = stage + (c >> 1) * 16384;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t off = sw128_offset((uint32_t)r_in_tile, (uint32_t)((c & 1) * 4 + q));
      *reinterpret_cast<uint4*>(box + off) =
          make_uint4(pack_bf16x2(v[8 * q + 0], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                     pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
    }
    continue;
  }
  if (row_ok && split_k) {
    // partial sum of one K range: reduce into the fp32 output
    float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
    if (full && vec_ok) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * q), "f"(v[4 * q]),
                     "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3]) : "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)      // unrolled with a guard: v[] must stay in registers
        if (col0 + j < p.N) atomicAdd(dst + j, v[j]);
    }
  } else if (row_ok) {
    if (full && vec_ok) {
      if (p.aux_out != nullptr) {
        uint4* dst = reinterpret_cast<uint4*>(p.aux_out + row * p.ld_aux_out + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          dst[q] = make_uint4(pack_bf16x2(v[8 * q + 0], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                              pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
      }
      if (kAct != MRK_ACT_NONE && kAux != MRK_AUX_DACT) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = apply_act<kAct>(v[j]);
      }
      if (kAux != MRK_AUX_NONE) {
        const uint4* src = reinterpret_cast<const uint4*>(p.aux_in + row * p.ld_aux_in + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 a = __ldg(src + q);
          const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16x2(w[e]);
            if (kAux == MRK_AUX_ADD) {
              v[8 * q + 2 * e] += f.x;
              v[8 * q + 2 * e + 1] += f.y;
            } else {
              v[8 * q + 2 * e] *= apply_act_grad<kAct>(f.x);
              v[8 * q + 2 * e + 1] *= apply_act_grad<kAct>(f.y);
            }
          }
        }
      }
      if (out_f32) {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + row * p.ldc + col0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          if (accumulate) {
            const float4 old = dst[q];
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          dst[q] = o;
        }
      } else {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (accumulate) {
            const uint4 old = dst[q];
            const uint32_t w[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf16x2(w[e]);
              v[8 * q + 2 * e] += f.x;
              v[8 * q + 2 * e + 1] += f.y;
            }
          }
          dst[q] = make_uint4(pack_bf16x2(v[8 * q + 0], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                              pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
        }
      }
    } else {
      // ragged right edge or unaligned pitches: element-wise (unrolled with a guard, so that v[]
      // is never indexed dynamically and stays in registers on the vector path too)
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        if (col >= p.N) continue;
        float x = v[j];
        if (p.aux_out != nullptr) p.aux_out[row * p.ld_aux_out + col] = __float2bfloat16(x);
        if (kAct != MRK_ACT_NONE && kAux != MRK_AUX_DACT) x = apply_act<kAct>(x);
        if (kAux == MRK_AUX_ADD) {
          x += __bfloat162float(p.aux_in[row * p.ld_aux_in + col]);
        } else if (kAux == MRK_AUX_DACT) {
          x *= apply_act_grad<kAct>(__bfloat162float(p.aux_in[row * p.ld_aux_in + col]));
        }
        if (out_f32) {
          float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col;
          *dst = accumulate ? (*dst + x) : x;
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
          *dst = __float2bfloat16(accumulate ? (__bfloat162float(*dst) + x) : x);
        }
      }
    }
  }
}
}
}

// Picks the epilogue specialised for (activation, aux mode) once per tile, so the per-element code
// has no run-time dispatch.
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, long long row, bool row_ok, uint32_t t_row,
                                              int col_base, int ncols, bool split_k, bool first_split,
                                              uint8_t* stage = nullptr, int r_in_tile = 0, int pass = 0) {
#define MRK_EPI(ACT, AUX) \
  epilogue_tile_t<ACT, AUX>(p, row, row_ok, t_row, col_base, ncols, split_k, first_split, stage, r_in_tile, pass)
#define MRK_EPI_ACT(ACT)                                             \
  do {                                                               \
    if (p.aux_mode == MRK_AUX_ADD) MRK_EPI(ACT, MRK_AUX_ADD);        \
    else if (p.aux_mode == MRK_AUX_DACT) MRK_EPI(ACT, MRK_AUX_DACT); \
    else MRK_EPI(ACT, MRK_AUX_NONE);                                 \
  } while (0)
  switch (p.act) {
    case MRK_ACT_GELU_ERF: MRK_EPI_ACT(MRK_ACT_GELU_ERF); break;
    case MRK_ACT_GELU_TANH: MRK_EPI_ACT(MRK_ACT_GELU_TANH); break;
    case MRK_ACT_RELU: MRK_EPI_ACT(MRK_ACT_RELU); break;
    case MRK_ACT_SILU: MRK_EPI_ACT(MRK_ACT_SILU); break;
    default: MRK_EPI_ACT(MRK_ACT_NONE); break;
  }
#undef MRK_EPI_ACT
#undef MRK_EPI
}

}  // namespace mrk
