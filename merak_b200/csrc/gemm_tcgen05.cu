// bf16 GEMM on 5th-generation tensor cores: C[M,N] = epilogue(alpha * A[M,K] * B[N,K]^T).
//
// Persistent, warp-specialised kernel (one CTA per SM):
//   warp 0      TMA producer: tiled bulk loads of A and B k-blocks into a ring of 128B-swizzled
//               shared-memory stages (no multicast).
//   warp 1      allocates TMEM, then one lane issues tcgen05.mma (128 x BN x 16 per instruction)
//               into one of two TMEM accumulator buffers and commits stage / accumulator barriers.
//   warps 2..9  epilogue (two warps per TMEM lane quadrant, half the columns each): tcgen05.ld the finished accumulator (one row per thread), apply
//               bias / activation / residual / activation-derivative, store bf16 or fp32.
// The two accumulator buffers let the epilogue of tile i overlap the main loop of tile i+1.
//
// Either operand may be K-major ("row r holds the K values of output row r") or MN-major
// (the transposed storage), so the three GEMMs of a linear layer
//   Y = X W^T,   dX = dY W,   dW = dY^T X
// all run from the same row-major tensors without materialising a transpose.
//
// Covers the GEMM call sites of the reference's Column/RowParallelLinear and lm_head
// (Merak/core/mpu/layers.py:252,354) plus the bias/GELU/residual elementwise passes that
// follow them there.
#include <string.h>

#include "gemm_common.cuh"
#include "host_common.h"

namespace mrk {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kNumThreads = 320;       // TMA warp, UMMA warp, 8 epilogue warps

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // +1024 alignment slack
};

template <int BN>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  using L = SmemLayout<BN>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = (2 * BN <= 512) ? (2 * BN < 32 ? 32 : 2 * BN) : 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bar_base = smem + kStages * L::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool a_mn = (p.flags & MRK_GEMM_A_MN) != 0;
  const bool b_mn = (p.flags & MRK_GEMM_B_MN) != 0;

  // fused all-gather: the CTAs in front of the compute CTAs only move the peers' shards of A
  const int aux_ctas = p.comm.mode == 2 ? (int)gridDim.x - p.comm.gemm_ctas : 0;
  if (p.comm.mode == 2 && (int)blockIdx.x < aux_ctas) {
    comm_gather_role(p, smem, L::kTotal - 1024);
    return;
  }
  const int cta_stride = p.comm.mode == 2 ? p.comm.gemm_ctas : (int)gridDim.x;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), 8 * 32);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_units = p.num_m_blocks * p.num_n_blocks * p.num_splits;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = (int)blockIdx.x - aux_ctas; unit < num_units && ok; unit += cta_stride) {
        int m_blk, n_blk;
        tile_coords(unit / p.num_splits, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
        m_blk = comm_perm_m(p, m_blk, kBlockM);
        const int m0 = m_blk * kBlockM, n0 = n_blk * BN;
        const int kb_begin = (unit % p.num_splits) * p.kb_per_split;
        const int kb_end = min(p.num_k_blocks, kb_begin + p.kb_per_split);
        if (p.comm.mode == 2) {
          ok = comm_wait_rows(p, m0, kBlockM, abort_flag);
          if (!ok) break;
        }
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
          mbar_arrive_expect_tx(fb, L::kStageBytes);
          const int k0 = kb * kBlockK;
          if (!a_mn) {
            tma_load_2d(sa, &tma_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int atom = 0; atom < kBlockM / 64; ++atom)
              tma_load_2d(sa + atom * (kBlockK * 128), &tma_a, fb, m0 + atom * 64, k0);
          }
          if (!b_mn) {
            tma_load_2d(sb, &tma_b, fb, k0, n0);
          } else {
#pragma unroll
            for (int atom = 0; atom < BN / 64; ++atom)
              tma_load_2d(sb + atom * (kBlockK * 128), &tma_b, fb, n0 + atom * 64, k0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kBlockM, BN, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int unit = (int)blockIdx.x - aux_ctas; unit < num_units && ok; unit += cta_stride, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1u, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb_begin = (unit % p.num_splits) * p.kb_per_split;
        const int kb_end = min(p.num_k_blocks, kb_begin + p.kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t da = a_mn ? desc_mnmajor(sa, k, kBlockK) : desc_kmajor(sa, k);
            const uint64_t db = b_mn ? desc_mnmajor(sb, k, kBlockK) : desc_kmajor(sb, k);
            umma_bf16_ss(d_tmem, da, db, idesc, (kb != kb_begin || k != 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(smem_u32(&tmem_full_bar[acc]));
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    int iter = 0;
    bool ok = true;
    for (int unit = (int)blockIdx.x - aux_ctas; unit < num_units && ok; unit += cta_stride, ++iter) {
      int m_blk, n_blk;
      tile_coords(unit / p.num_splits, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
      m_blk = comm_perm_m(p, m_blk, kBlockM);
      const bool split_k = p.num_splits > 1;
      const bool first_split = (unit % p.num_splits) == 0;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const long long row = (long long)m_blk * kBlockM + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      // two warps share a TMEM lane quadrant: warps 2..5 take the left half of the columns, 6..9 the right
      const int half = (warp - 2) >> 2;
      epilogue_tile(p, row, row_ok, t_row + half * (BN / 2), n_blk * BN + half * (BN / 2), BN / 2, split_k,
                    first_split);
      tc_fence_before();
      mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  MRK_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MRK_CUDA_OK(cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     L::kTotal));
    configured[dev & 63] = true;
  }
  p.num_m_blocks = (p.M + kBlockM - 1) / kBlockM;
  p.num_n_blocks = (p.N + BN - 1) / BN;
  p.num_k_blocks = (p.K + kBlockK - 1) / kBlockK;
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  // Split-K when the output has too few tiles to fill the SMs (weight gradients: small [N,K]
  // outputs contracted over all tokens).  Only for fp32 accumulate outputs without an activation.
  p.num_splits = 1;
  const bool can_split = (p.flags & MRK_GEMM_OUT_F32) && (p.flags & MRK_GEMM_ACCUMULATE) &&
                         p.act == MRK_ACT_NONE && p.aux_mode == MRK_AUX_NONE && p.aux_out == nullptr;
  if (can_split && tiles * 2 <= sm_count() && p.num_k_blocks >= 16) {
    int want = sm_count() / tiles;
    const int max_by_k = p.num_k_blocks / 8;
    if (want > max_by_k) want = max_by_k;
    if (want > 32) want = 32;
    if (want > 1) p.num_splits = want;
  }
  p.kb_per_split = (p.num_k_blocks + p.num_splits - 1) / p.num_splits;
  p.num_splits = (p.num_k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  const int units = tiles * p.num_splits;
  int grid = units < sm_count() ? units : sm_count();
  if (p.comm.mode == 2) {
    // compute CTAs + gather CTAs, all resident at once (one CTA per SM): the former wait for the latter
    const int gather = p.comm.gemm_ctas;     // the caller passes the number of gather CTAs here
    MRK_REQUIRE(gather >= 1 && gather < sm_count(), "gemm: bad number of gather CTAs");
    const int room = sm_count() - gather;
    p.comm.gemm_ctas = units < room ? units : room;
    grid = p.comm.gemm_ctas + gather;
  }
  if (p.comm.mode != 0 && p.comm.perm)
    p.comm.perm = (p.comm.seg_rows % kBlockM == 0 && p.num_m_blocks % p.comm.n == 0 && p.M % kBlockM == 0) ? 1 : 0;
  gemm_bf16_kernel<BN><<<grid, kNumThreads, L::kTotal, stream>>>(ta, tb, p);
  MRK_CHECK_LAUNCH();
  return 0;
}

int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& taux,
                     const CUtensorMap& tauxin, GemmParams& p, cudaStream_t stream);

}  // namespace mrk

using namespace mrk;

static int gemm_entry(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                      long long ldb, long long ldc, const void* bias, const void* aux_in,
                      long long ld_aux_in, void* aux_out, long long ld_aux_out, int act, int aux_mode,
                      int flags, float alpha, int block_n, const GemmComm* comm, void* stream) {
  MRK_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %dx%dx%d", M, N, K);
  MRK_REQUIRE(A && B && C, "gemm: null operand");
  MRK_REQUIRE(aux_mode == MRK_AUX_NONE || aux_in != nullptr, "gemm: aux_mode set without aux_in");
  const bool a_mn = flags & MRK_GEMM_A_MN, b_mn = flags & MRK_GEMM_B_MN;
  int bn = block_n;
  // block_n: 0 = choose; 64/128/256 = single-CTA kernel with that tile width; 512 = CTA-pair kernel
  // (256 x 256 tile per 2-CTA cluster).  The pair kernel is the default for anything wide enough.
  if (bn == 0 && M > 128 && N > 128) bn = 512;     // (both kernels carry the fused all-gather)
  if (bn == 0) {
    // Heuristic: widest tile that still fills the SMs reasonably; narrow tiles for small N.
    const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
    const bool splittable = (flags & MRK_GEMM_OUT_F32) && (flags & MRK_GEMM_ACCUMULATE) && act == MRK_ACT_NONE &&
                            aux_mode == MRK_AUX_NONE && aux_out == nullptr && K >= 1024;
    bn = (N <= 128 || (tiles256 < sm_count() && !splittable)) ? 128 : 256;
    if (N <= 64) bn = 64;
  }
  MRK_REQUIRE(bn == 64 || bn == 128 || bn == 256 || bn == 512, "gemm: block_n must be 64, 128, 256 or 512");
  const int b_box_rows = bn == 512 ? 128 : bn;
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn) rc = make_tmap_2d(&ta, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kBlockK, kBlockM, 3);
  else       rc = make_tmap_2d(&ta, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, kBlockK, 3);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_2d(&tb, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, kBlockK, (uint32_t)b_box_rows, 3);
  else       rc = make_tmap_2d(&tb, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, kBlockK, 3);
  if (rc) return rc;
  GemmParams p;
  memset(&p.comm, 0, sizeof(p.comm));
  p.tma_store = 0;
  p.tma_store_aux = 0;
  p.tma_aux_in = 0;
  if (comm != nullptr) p.comm = *comm;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = bias;
  p.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in); p.ld_aux_in = ld_aux_in;
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out); p.ld_aux_out = ld_aux_out;
  p.act = act; p.aux_mode = aux_mode; p.flags = flags; p.alpha = alpha;
  p.status = status_word_device();
  MRK_REQUIRE(p.status != nullptr, "gemm: status word unavailable");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 512) {
    // bf16 outputs that a tensor map can describe leave through shared memory + TMA stores
    CUtensorMap tc = ta;
    p.tma_store = 0;
    if (!(flags & (MRK_GEMM_OUT_F32 | MRK_GEMM_ACCUMULATE)) && (ldc % 8) == 0 &&
        (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
      rc = make_tmap_2d(&tc, C, 2, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 128, 3);
      if (rc) return rc;
      p.tma_store = 1;
    }
    if ((flags & MRK_GEMM_OUT_F32) && (ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
      // fp32 outputs (weight gradients): boxes of 128 rows x 32 columns, stored or added by the TMA unit
      rc = make_tmap_2d(&tc, C, 4, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 32, 128, 3);
      if (rc) return rc;
      p.tma_store = 2;
    }
    CUtensorMap taux = ta;
    if (p.tma_store && aux_out != nullptr && (ld_aux_out % 8) == 0 && (reinterpret_cast<uintptr_t>(aux_out) & 15) == 0) {
      rc = make_tmap_2d(&taux, aux_out, 2, (uint64_t)N, (uint64_t)M, (uint64_t)ld_aux_out, 64, 128, 3);
      if (rc) return rc;
      p.tma_store_aux = 1;
    }
    CUtensorMap tauxin = ta;
    p.tma_aux_in = 0;
    if (p.tma_store == 1 && aux_mode != MRK_AUX_NONE && (ld_aux_in % 8) == 0 &&
        (reinterpret_cast<uintptr_t>(aux_in) & 15) == 0) {
      rc = make_tmap_2d(&tauxin, aux_in, 2, (uint64_t)N, (uint64_t)M, (uint64_t)ld_aux_in, 64, 128, 3);
      if (rc) return rc;
      p.tma_aux_in = 1;
    }
    return launch_gemm_pair(ta, tb, tc, taux, tauxin, p, s);
  }
  if (bn == 256) return launch<256>(ta, tb, p, s);
  if (bn == 128) return launch<128>(ta, tb, p, s);
  return launch<64>(ta, tb, p, s);
}

MRK_API int mrk_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, const void* bias, const void* aux_in,
                          long long ld_aux_in, void* aux_out, long long ld_aux_out, int act, int aux_mode,
                          int flags, float alpha, int block_n, void* stream) {
  return gemm_entry(A, B, C, M, N, K, lda, ldb, ldc, bias, aux_in, ld_aux_in, aux_out, ld_aux_out, act, aux_mode,
                    flags, alpha, block_n, nullptr, stream);
}

static int fill_comm(GemmComm* c, int mode, int n, int rank, int seg_rows, void* const* peers, long long ld_peer,
                     void* const* ctrls, unsigned epoch, int budget_ms, int M) {
  MRK_REQUIRE(n >= 2 && n <= kGemmMaxPeers && rank >= 0 && rank < n, "gemm: tensor-parallel group of %d ranks", n);
  MRK_REQUIRE(seg_rows > 0 && M % seg_rows == 0 && (M / seg_rows) % n == 0,
              "gemm: %d rows do not split into segments of %d over %d ranks", M, seg_rows, n);
  memset(c, 0, sizeof(*c));
  c->mode = mode; c->n = n; c->rank = rank; c->seg_rows = seg_rows; c->perm = 1;
  for (int k = 0; k < n; ++k) {
    c->peer[k] = peers[k];
    c->ctrl[k] = ctrls ? ctrls[k] : nullptr;
  }
  c->ld_peer = ld_peer;
  c->epoch = epoch;
  c->budget = (long long)(budget_ms > 0 ? budget_ms : 2000) * 2000000ll;
  return 0;
}

// all-gather -> GEMM.  `gathered` ([M, K] bf16, pitch K, local) is filled from every rank's shard
// ([M/n, K], pitch K, peer-mapped) while C = act(gathered * W^T + bias) is computed.
MRK_API int mrk_gemm_bf16_ag(void* gathered, void* const* peer_shards, const void* B, void* C, int M, int N, int K,
                             long long ldb, long long ldc, const void* bias, void* aux_out, long long ld_aux_out,
                             int act, int flags, float alpha, void* const* ctrls, unsigned* seg_flags,
                             unsigned flag_target, int gather_ctas, int n, int rank, int seg_rows, unsigned epoch,
                             int budget_ms, void* stream) {
  MRK_REQUIRE((K % 8) == 0 && ((uintptr_t)gathered & 15) == 0, "gemm_ag: K must be a multiple of 8");
  MRK_REQUIRE(!(flags & MRK_GEMM_A_MN), "gemm_ag: A must be [M, K]");
  GemmComm c;
  int rc = fill_comm(&c, 2, n, rank, seg_rows, peer_shards, K, ctrls, epoch, budget_ms, M);
  if (rc) return rc;
  c.gathered = gathered;
  c.seg_flags = seg_flags;
  c.flag_target = flag_target;
  c.gemm_ctas = gather_ctas;
  return gemm_entry(gathered, B, C, M, N, K, K, ldb, ldc, bias, nullptr, 0, aux_out, ld_aux_out, act, MRK_AUX_NONE,
                    flags, alpha, 0, &c, stream);
}

// GEMM -> reduce-scatter in one launch (see gemm_common.cuh, mode 1).  `parts[k]` is rank k's
// [M, N] bf16 partial-product buffer (peer-mapped; entry `rank` is written here), `tile_flags[k]`
// rank k's flag array of n * units uint32 (peer-mapped, zero before first use, shared by all calls
// with growing `epoch`), `out` [M / n, N] bf16 receives this rank's rows of the sum (+ bias).
// Requirements: M a multiple of 256 * ... see the checks; the caller falls back to the two-kernel
// path (plain GEMM + pull-and-sum) otherwise.  phase: 3 normally; 1 / 2 split the multiplication
// and the reduction into two launches for single-GPU tests.
MRK_API int mrk_gemm_bf16_rs_units(int M, int N) {
  return ((M + 255) / 256) * ((N + 255) / 256) * 4;
}

MRK_API int mrk_gemm_bf16_rs(const void* A, const void* B, void* const* parts, void* const* tile_flags, void* out,
                             const void* bias, int M, int N, int K, long long lda, long long ldb, int flags, int n,
                             int rank, int seg_rows, unsigned epoch, int phase, int reduce_ctas, unsigned* queue,
                             int budget_ms, void* stream) {
  MRK_REQUIRE(M % 128 == 0 && seg_rows % 128 == 0 && N % 64 == 0 && M > 128 && N > 128,
              "gemm_rs: shape %dx%d (segments of %d rows) is not tileable into 128-row sub-tiles", M, N, seg_rows);
  MRK_REQUIRE(!(flags & (MRK_GEMM_OUT_F32 | MRK_GEMM_ACCUMULATE)), "gemm_rs: bf16 partial products only");
  MRK_REQUIRE(phase >= 1 && phase <= 3 && out != nullptr, "gemm_rs: bad arguments");
  GemmComm c;
  int rc = fill_comm(&c, 1, n, rank, seg_rows, parts, N, nullptr, epoch, budget_ms, M);
  if (rc) return rc;
  for (int k = 0; k < n; ++k) c.tile_flags[k] = reinterpret_cast<uint32_t*>(tile_flags[k]);
  c.units_total = mrk_gemm_bf16_rs_units(M, N);
  c.own_last = 1;
  c.phase = phase;
  c.rs_out = out;
  c.rs_bias = bias;
  c.reduce_ctas = reduce_ctas;
  c.rs_queue = queue;
  return gemm_entry(A, B, parts[rank], M, N, K, lda, ldb, N, nullptr, nullptr, 0, nullptr, 0, MRK_ACT_NONE,
                    MRK_AUX_NONE, flags, 1.0f, 512, &c, stream);
}
