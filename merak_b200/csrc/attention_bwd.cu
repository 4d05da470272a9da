// Flash attention backward on tcgen05.  One CTA owns one 128-key block of one (batch, kv head)
// and walks over the query blocks (and, for grouped-query attention, over the query heads that
// share the kv head).  Five products per (key block, query block):
//
//   S^T  = K Q^T          P^T  = exp2(S^T * scale - lse)
//   dP^T = V dO^T         dS^T = P^T o (dP^T - delta) * scale
//   dV  += P^T dO         dK  += dS^T Q            dQ += dS K     (dQ partials are added into an fp32 buffer)
//
// All five run on the tensor core with TMEM accumulators: S^T, dP^T (consumed by the compute
// warps one key row per thread), dK and dV (resident for the whole CTA), and a dQ partial that is
// added to global memory: head dim 64 stages the [128 q][64] tile in shared memory and hands it to
// the TMA unit as two bulk tensor reductions (whole 128-byte lines per request; a thread holds one
// row, so direct vector reductions touch 32 different lines per warp instruction), head dim 128
// has no shared memory left for that and issues the vector reductions.  P^T and dS^T are written to shared memory once
// and serve as the K-major A operand of dV/dK and as the MN-major A operand of dQ; the Q and dO
// tiles likewise serve as K-major B of the first two products and MN-major B of dK/dV.
//
//   warp 0       TMA producer           warp 1   UMMA issuer
//   warps 2..9   compute: two warpgroups, each handles 64 of the 128 query columns of every row.
//
// Head dim 64 runs as a software pipeline over the query blocks.  A compute thread copies its 64
// S^T and 64 dP^T values into registers and releases those TMEM columns at once, so the tensor core
// computes S^T / dP^T of block i+1 while the CUDA cores work on block i; the P^T / dS^T stores of
// block i wait for the dV / dK / dQ products of block i-1 (which read the same shared memory), and
// the dQ partial of block i-1 (double buffered in TMEM) is drained while those products of block i
// run.  Head dim 128 fills all 512 TMEM columns (the dQ partial reuses the S^T columns), so it keeps
// the plain order: products, element-wise step, products, drain.
#include "attention.h"
#include "host_common.h"
#include "sm100_ptx.cuh"
#include "attention_dropout.cuh"
#include <type_traits>

namespace mrk {

int make_bshd_tmap(CUtensorMap* out, const void* base, int D, int L, int H, int B, long long sb, long long ss,
                   long long sh, int box_rows);

constexpr int kBwdThreads = 320;

struct AttnBwdParams {
  const float* lse;        // [B, H, Lq]
  const float* delta;      // [B, H, Lq]  rowsum(dO o O)
  float* dq_acc;           // [B, Lq, H, D] fp32, zero-initialised
  __nv_bfloat16* dk;       // [B, Lk, Hkv, D] strides below
  __nv_bfloat16* dv;
  long long dk_sb, dk_ss, dk_sh;
  long long dv_sb, dv_ss, dv_sh;
  const float* key_bias;   // optional [B, Lk]
  int B, H, Hkv, Lq, Lk;
  int causal;
  float scale, scale_log2;
  float p_drop;                    // dropout on the probabilities (0 = off): same arguments as the forward call
  const unsigned long long* rng;
  unsigned long long call_id;
  unsigned* status;
};

template <int D>
struct AttnBwdSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kStages = (D == 64) ? 2 : 1;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kTile;
  static constexpr int kStageOff = 2 * kTile;                    // [Q_j | dO_j] per stage
  static constexpr int kPOff = kStageOff + kStages * 2 * kTile;  // P^T   [128 kv][128 q] bf16
  static constexpr int kDSOff = kPOff + 32768;                   // dS^T
  static constexpr int kStatOff = kDSOff + 32768;                // per compute warp: 2 x (lse2[64] | delta[64] | row key[64])
  static constexpr int kBarOff = kStatOff + 8 * 2 * 192 * 4;
  static constexpr int kDQStageOff = kBarOff + 1024;             // D=64: one [32 q][32] fp32 tile per compute warp
  static constexpr int kTotal = kDQStageOff + (D == 64 ? 8 * 4096 : 0) + 1024;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}


template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                const __grid_constant__ CUtensorMap tdq, const __grid_constant__ CUtensorMap tdk,
                const __grid_constant__ CUtensorMap tdv, const AttnBwdParams p) {
  using L = AttnBwdSmem<D>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSCol = 0, kDPCol = 128, kDKCol = 256, kDVCol = 256 + D;
  constexpr uint32_t kDQCol = (D == 64) ? 384 : 0;   // D=64: two buffers of 64 columns; D=128: reuses the S^T columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;                    // 1
  uint64_t* qdo_full = bars + 1;               // kStages
  uint64_t* qdo_empty = qdo_full + kStages;    // kStages
  uint64_t* sp_full = qdo_empty + kStages;     // 1
  uint64_t* pds_full = sp_full + 1;            // 1 (256 arrivals)
  uint64_t* dq_full = pds_full + 1;            // 1
  uint64_t* dq_empty = dq_full + 1;            // 2 (256 arrivals), one per dQ buffer
  uint64_t* dkv_full = dq_empty + 2;           // 1
  uint64_t* sdp_free = dkv_full + 1;           // 1 (256 arrivals): S^T and dP^T are in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sdp_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat = reinterpret_cast<float*>(smem + L::kStatOff);  // [8 warps][2 buffers][lse2[64] | delta * scale[64] | dropout row key[64]]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_blk = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int group = p.H / p.Hkv;
  const int k0 = kv_blk * 128;
  const int shift = p.Lk - p.Lq;   // key k visible to query q iff k <= q + shift (causal)
  const int n_qblocks = (p.Lq + 127) / 128;
  int j_begin = 0;
  if (p.causal) {
    const int first_q = k0 - shift;          // smallest query index that sees key k0
    j_begin = first_q <= 0 ? 0 : first_q / 128;
  }
  const int iters_per_head = max(0, n_qblocks - j_begin);
  const int total_iters = iters_per_head * group;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(kv_full), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&qdo_full[s]), 1);
      mbar_init(smem_u32(&qdo_empty[s]), 1);
    }
    mbar_init(smem_u32(sp_full), 1);
    mbar_init(smem_u32(pds_full), 256);
    mbar_init(smem_u32(dq_full), 1);
    mbar_init(smem_u32(&dq_empty[0]), 256);
    mbar_init(smem_u32(&dq_empty[1]), 256);
    mbar_init(smem_u32(dkv_full), 1);
    mbar_init(smem_u32(sdp_free), 256);
    fence_mbar_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
    tma_prefetch_desc(&tdo);
    tma_prefetch_desc(&tdq);
    tma_prefetch_desc(&tdk);
    tma_prefetch_desc(&tdv);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t k_smem = smem_u32(smem + L::kKOff), v_smem = smem_u32(smem + L::kVOff);
  const uint32_t p_smem = smem_u32(smem + L::kPOff), ds_smem = smem_u32(smem + L::kDSOff);

  if (warp == 0) {
    if (lane == 0 && total_iters > 0) {
      mbar_arrive_expect_tx(smem_u32(kv_full), 2 * L::kTile);
#pragma unroll
      for (int a = 0; a < D / 64; ++a) {
        tma_load_4d(k_smem + a * 16384, &tk, smem_u32(kv_full), a * 64, k0, hkv, b);
        tma_load_4d(v_smem + a * 16384, &tv, smem_u32(kv_full), a * 64, k0, hkv, b);
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int it = 0; it < total_iters; ++it) {
        const int h = hkv * group + it / iters_per_head;
        const int j = j_begin + it % iters_per_head;
        if (!mbar_wait(smem_u32(&qdo_empty[stage]), phase ^ 1u, abort_flag, p.status)) break;
        const uint32_t fb = smem_u32(&qdo_full[stage]);
        const uint32_t qs = smem_u32(smem + L::kStageOff + stage * 2 * L::kTile);
        const uint32_t dos = qs + L::kTile;
        mbar_arrive_expect_tx(fb, 2 * L::kTile);
#pragma unroll
        for (int a = 0; a < D / 64; ++a) {
          tma_load_4d(qs + a * 16384, &tq, fb, a * 64, j * 128, h, b);
          tma_load_4d(dos + a * 16384, &tdo, fb, a * 64, j * 128, h, b);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && total_iters > 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_dkv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t idesc_dq = make_idesc_bf16(128, D, 1, 1);
      bool ok = mbar_wait(smem_u32(kv_full), 0, abort_flag, p.status);
      // S^T = K Q^T and dP^T = V dO^T of the query block in ring stage `st`
      auto issue_scores = [&](int st) {
        const uint32_t qs = smem_u32(smem + L::kStageOff + st * 2 * L::kTile);
        const uint32_t dos = qs + L::kTile;
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tmem_base + kSCol, desc_kmajor(k_smem + (k / 4) * 16384, k % 4),
                       desc_kmajor(qs + (k / 4) * 16384, k % 4), idesc_s, k != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tmem_base + kDPCol, desc_kmajor(v_smem + (k / 4) * 16384, k % 4),
                       desc_kmajor(dos + (k / 4) * 16384, k % 4), idesc_s, k != 0 ? 1u : 0u);
        umma_commit(smem_u32(sp_full));
      };
      // dV += P^T dO, dK += dS^T Q (contraction over the 128 queries of the block)
      auto issue_dkv = [&](int st, int it) {
        const uint32_t qs = smem_u32(smem + L::kStageOff + st * 2 * L::kTile);
        const uint32_t dos = qs + L::kTile;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + kDVCol, desc_kmajor(p_smem + (k / 4) * 16384, k % 4),
                       desc_mnmajor(dos, k, 128), idesc_dkv, (it | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + kDKCol, desc_kmajor(ds_smem + (k / 4) * 16384, k % 4),
                       desc_mnmajor(qs, k, 128), idesc_dkv, (it | k) != 0 ? 1u : 0u);
      };
      // dQ partial = dS K (contraction over the 128 keys of this CTA)
      auto issue_dq = [&](uint32_t col) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + col, desc_mnmajor(ds_smem, k, 128), desc_mnmajor(k_smem, k, 128),
                       idesc_dq, k != 0 ? 1u : 0u);
      };
      if constexpr (D == 64) {
        // stage of block `it` is it % 2 (kStages == 2); its full-barrier phase is (it / 2) & 1
        if (ok) ok = mbar_wait(smem_u32(&qdo_full[0]), 0, abort_flag, p.status);
        if (ok) {
          tc_fence_after();
          issue_scores(0);
        }
        for (int it = 0; it < total_iters && ok; ++it) {
          const int stage = it & 1;
          if (it + 1 < total_iters) {
            ok = mbar_wait(smem_u32(&qdo_full[stage ^ 1]), ((it + 1) >> 1) & 1, abort_flag, p.status) &&
                 mbar_wait(smem_u32(sdp_free), it & 1, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after();
            issue_scores(stage ^ 1);
          }
          ok = mbar_wait(smem_u32(pds_full), it & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          issue_dkv(stage, it);
          if (it >= 2) {   // the drain of the partial that used this dQ buffer two blocks ago
            ok = mbar_wait(smem_u32(&dq_empty[it & 1]), ((it >> 1) - 1) & 1, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after();
          }
          issue_dq(kDQCol + (it & 1) * 64);
          umma_commit(smem_u32(&qdo_empty[stage]));
          umma_commit(smem_u32(dq_full));
        }
      } else {
        int stage = 0;
        uint32_t phase = 0;
        for (int it = 0; it < total_iters && ok; ++it) {
          ok = mbar_wait(smem_u32(&qdo_full[stage]), phase, abort_flag, p.status);
          if (!ok) break;
          if (it > 0) {   // the dQ partial shares the S^T columns
            ok = mbar_wait(smem_u32(&dq_empty[0]), (it - 1) & 1, abort_flag, p.status);
            if (!ok) break;
          }
          tc_fence_after();
          issue_scores(stage);
          ok = mbar_wait(smem_u32(pds_full), it & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          issue_dkv(stage, it);
          issue_dq(kDQCol);
          umma_commit(smem_u32(&qdo_empty[stage]));
          umma_commit(smem_u32(dq_full));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (ok) umma_commit(smem_u32(dkv_full));
    }
  } else {
    // ------------------------------- compute warps -------------------------------
    const int cw = warp - 2;                 // 0..7
    const int wg = cw >> 2;                  // column half
    const int quad = warp & 3;               // TMEM lane quadrant
    const int r = quad * 32 + lane;          // key row inside the block (also query row for dQ)
    const int key = k0 + r;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int tid_c = threadIdx.x - 64;      // 0..255
    const float kbias = (p.key_bias && key < p.Lk) ? p.key_bias[(long long)b * p.Lk + key] * 1.4426950408889634f : 0.f;
    bool ok = true;

    // Every warp stages the statistics of its own 64 query columns (no barrier between warps):
    // lane l fetches lse (log2 units) and delta * scale of columns l and l + 32 of the warp's half.
    const bool drop = p.p_drop > 0.f;
    const float keep_scale = drop ? 1.f / (1.f - p.p_drop) : 1.f;
    const uint32_t drop_thresh = attn_drop_thresh(p.p_drop);
    const uint32_t drop_base = drop ? attn_drop_base(p.rng[0], p.rng[1] + p.call_id) : 0u;
    struct Stat { float lse0, lse1, dl0, dl1; uint32_t rk0, rk1; };
    auto load_stat = [&](int it) -> Stat {
      const int h = hkv * group + it / iters_per_head;
      const int q = (j_begin + it % iters_per_head) * 128 + wg * 64 + lane;
      const long long off = ((long long)b * p.H + h) * p.Lq + q;
      Stat v;
      v.lse0 = q < p.Lq ? __ldg(p.lse + off) * 1.4426950408889634f : INFINITY;
      v.lse1 = q + 32 < p.Lq ? __ldg(p.lse + off + 32) * 1.4426950408889634f : INFINITY;
      v.dl0 = q < p.Lq ? __ldg(p.delta + off) * p.scale : 0.f;
      v.dl1 = q + 32 < p.Lq ? __ldg(p.delta + off + 32) * p.scale : 0.f;
      v.rk0 = drop ? attn_drop_rowkey(drop_base, (uint32_t)(b * p.H + h), (uint32_t)q) : 0u;
      v.rk1 = drop ? attn_drop_rowkey(drop_base, (uint32_t)(b * p.H + h), (uint32_t)(q + 32)) : 0u;
      return v;
    };
    // P^T and dS^T of 32 query columns (col0 .. col0+31 of the block) of this thread's key row;
    // `st` points at the 32 lse values of these columns, the delta values follow 64 floats later and
    // the dropout row keys 128 floats later
    // (`masked` is a compile-time tag: a per-element branch would end the basic block at every
    // element and leave each exp2 -> multiply -> pack chain exposed at its full latency)
    auto chunk = [&](auto masked, const uint32_t* s, const uint32_t* dp, const float* st, int col0, int q0,
                     uint32_t* pk, uint32_t* dsk) {
#pragma unroll
      for (int i8 = 0; i8 < 32; i8 += 8) {
        // the per-query statistics are the same for every lane: 16-byte broadcast loads, 8 columns at a time
        const float4 l0 = *reinterpret_cast<const float4*>(st + i8);
        const float4 l1 = *reinterpret_cast<const float4*>(st + i8 + 4);
        const float4 d0 = *reinterpret_cast<const float4*>(st + 64 + i8);
        const float4 d1 = *reinterpret_cast<const float4*>(st + 64 + i8 + 4);
        const float lse8[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const float dl8[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          float pv[2], dv_[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = i8 + j + e;
            const float x = fmaf(__uint_as_float(s[i]), p.scale_log2, kbias - lse8[j + e]);
            float pe = exp2f(x);
            float mt = 1.f;        // dropout mask times 1 / (1 - p)
            if constexpr (decltype(masked)::value) {
              const int q = q0 + col0 + i;
              if (key >= p.Lk || (p.causal && key > q + shift)) pe = 0.f;
              if (drop)
                mt = attn_drop_keep(reinterpret_cast<const uint32_t*>(st)[128 + i], (uint32_t)key, drop_thresh) ? keep_scale : 0.f;
            }
            pv[e] = pe * mt;       // the dV product sees the dropped probabilities
            dv_[e] = pe * fmaf(__uint_as_float(dp[i]) * mt, p.scale, -dl8[j + e]);   // delta was staged times scale
          }
          pk[(i8 + j) >> 1] = pack_bf16x2(pv[0], pv[1]);
          dsk[(i8 + j) >> 1] = pack_bf16x2(dv_[0], dv_[1]);
        }
      }
    };
    // 32 columns of P^T / dS^T -> atom (col0/64), 16-byte chunks ((col0%64)/8)..+3 of row r
    auto store_chunk = [&](int col0, const uint32_t* pk, const uint32_t* dsk) {
      const uint32_t atom = (uint32_t)(col0 >> 6), ch0 = (uint32_t)((col0 & 63) >> 3);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint32_t off = atom * 16384 + sw128_offset((uint32_t)r, ch0 + q4);
        *reinterpret_cast<uint4*>(smem + L::kPOff + off) =
            make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        *reinterpret_cast<uint4*>(smem + L::kDSOff + off) =
            make_uint4(dsk[4 * q4], dsk[4 * q4 + 1], dsk[4 * q4 + 2], dsk[4 * q4 + 3]);
      }
    };
    // dQ partial of query block `it` (TMEM columns `col`) -> fp32 accumulator in global memory
    auto drain_dq = [&](int it, uint32_t col) {
      const int h = hkv * group + it / iters_per_head;
      const int q = (j_begin + it % iters_per_head) * 128 + r;
      float* dst = p.dq_acc + (((long long)b * p.Lq + q) * p.H + h) * D + wg * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_off + col + wg * (D / 2) + c * 32, v);
        tmem_wait_ld();
        if (q < p.Lq) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            red_add_v4(dst + c * 32 + i, __uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                       __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));   // dS already carries the scale
        }
      }
    };

    // head dim 64: dQ partial of query block `it` -> shared memory -> bulk tensor reduction.  Each
    // warp owns 32 query rows x 32 columns and a staging tile of its own, so the warps never wait
    // for one another.
    uint8_t* dq_stage = smem + L::kDQStageOff + cw * 4096;
    const bool dq_leader = lane == 0;
    auto drain_dq_tma = [&](int it) {
      const int h = hkv * group + it / iters_per_head;
      const int q0 = (j_begin + it % iters_per_head) * 128;
      uint32_t v[32];
      tmem_ld32(tmem_base + lane_off + kDQCol + (it & 1) * 64 + wg * 32, v);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(smem_u32(&dq_empty[it & 1]));
      if (dq_leader) tma_store_wait_read<0>();      // the previous reduction has read the staging tile
      __syncwarp();
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4)
        *reinterpret_cast<uint4*>(dq_stage + sw128_offset((uint32_t)lane, (uint32_t)q4)) =
            make_uint4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (dq_leader) {   // rows past Lq fall outside the tensor map and are dropped
        tma_reduce_add_4d(&tdq, smem_u32(dq_stage), wg * 32, h, q0 + quad * 32, b);
        tma_store_commit();
      }
    };

    Stat stat_next = total_iters > 0 ? load_stat(0) : Stat{0.f, 0.f, 0.f, 0.f, 0u, 0u};
    float* stat_w = stat + cw * 384;
    for (int it = 0; it < total_iters && ok; ++it) {
      const int q0 = (j_begin + it % iters_per_head) * 128;
      float* st = stat_w + (it & 1) * 192;
      st[lane] = stat_next.lse0;
      st[32 + lane] = stat_next.lse1;
      st[64 + lane] = stat_next.dl0;
      st[96 + lane] = stat_next.dl1;
      reinterpret_cast<uint32_t*>(st)[128 + lane] = stat_next.rk0;
      reinterpret_cast<uint32_t*>(st)[160 + lane] = stat_next.rk1;
      if (it + 1 < total_iters) stat_next = load_stat(it + 1);   // in flight during this block's work
      __syncwarp();
      ok = mbar_wait(smem_u32(sp_full), it & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (key >= p.Lk) || (p.causal && (k0 + 127 > q0 + shift)) || drop;
      if constexpr (D == 64) {
        // two halves of 32 columns: the second half's TMEM loads are in flight while the first half
        // is stored, and the element-wise step never holds more than 64 inputs in registers
        const int col0 = wg * 64;
        uint32_t sa[32], da[32], sb[32], db[32];
        tmem_ld32(tmem_base + lane_off + kSCol + col0, sa);
        tmem_ld32(tmem_base + lane_off + kDPCol + col0, da);
        tmem_wait_ld();
        uint32_t pk[16], dsk[16];
        if (need_mask) chunk(std::true_type{}, sa, da, st, col0, q0, pk, dsk);
        else chunk(std::false_type{}, sa, da, st, col0, q0, pk, dsk);
        tmem_ld32(tmem_base + lane_off + kSCol + col0 + 32, sb);
        tmem_ld32(tmem_base + lane_off + kDPCol + col0 + 32, db);
        if (it > 0) {   // the products of the previous block have read P^T / dS^T; its dQ partial is ready
          ok = mbar_wait(smem_u32(dq_full), (it - 1) & 1, abort_flag, p.status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) { tmem_wait_ld(); break; }
        }
        store_chunk(col0, pk, dsk);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(smem_u32(sdp_free));       // the tensor core may overwrite S^T / dP^T now
        if (need_mask) chunk(std::true_type{}, sb, db, st + 32, col0 + 32, q0, pk, dsk);
        else chunk(std::false_type{}, sb, db, st + 32, col0 + 32, q0, pk, dsk);
        store_chunk(col0 + 32, pk, dsk);
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(pds_full));
        if (it > 0) {
          tc_fence_after();
          drain_dq_tma(it - 1);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          const int col0 = wg * 64 + c * 32;
          uint32_t s[32], dp[32];
          tmem_ld32(tmem_base + lane_off + kSCol + col0, s);
          tmem_ld32(tmem_base + lane_off + kDPCol + col0, dp);
          tmem_wait_ld();
          uint32_t pk[16], dsk[16];
          if (need_mask) chunk(std::true_type{}, s, dp, st + c * 32, col0, q0, pk, dsk);
          else chunk(std::false_type{}, s, dp, st + c * 32, col0, q0, pk, dsk);
          store_chunk(col0, pk, dsk);
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(pds_full));
        ok = mbar_wait(smem_u32(dq_full), it & 1, abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        drain_dq(it, kDQCol);
        tc_fence_before();
        mbar_arrive(smem_u32(&dq_empty[0]));
      }
    }
    if (D == 64 && total_iters > 0 && ok) {   // the last block's dQ partial
      ok = mbar_wait(smem_u32(dq_full), (total_iters - 1) & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        drain_dq_tma(total_iters - 1);
      }
    }
    if (D == 64 && dq_leader) tma_store_wait_read<0>();   // shared memory stays valid until the last reduction has read it
    // dK, dV of this key block
    if (total_iters > 0 && ok) {
      ok = mbar_wait(smem_u32(dkv_full), 0, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      // dK and dV leave through shared memory (the P^T / dS^T tiles are free now) as bulk tensor
      // stores: a thread holds one key row, so direct stores would touch 32 lines per instruction.
      // Tile (tensor, 64-column half) is [128 keys][64] bf16 in the 128-byte swizzle; rows past Lk
      // fall outside the tensor map and are dropped.
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t a[32], v[32];
        if (total_iters > 0) {
          tmem_ld32(tmem_base + lane_off + kDKCol + wg * (D / 2) + c * 32, a);
          tmem_ld32(tmem_base + lane_off + kDVCol + wg * (D / 2) + c * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0u; v[i] = 0u; }
        }
        const int col = wg * (D / 2) + c * 32;            // first of these 32 columns
        uint8_t* tile_k = smem + L::kPOff + (col >> 6) * 16384;
        uint8_t* tile_v = smem + L::kPOff + (D / 64) * 16384 + (col >> 6) * 16384;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 wk, wv;
          // dS^T was already multiplied by the softmax scale
          wk.x = pack_bf16x2(__uint_as_float(a[8 * q4]), __uint_as_float(a[8 * q4 + 1]));
          wk.y = pack_bf16x2(__uint_as_float(a[8 * q4 + 2]), __uint_as_float(a[8 * q4 + 3]));
          wk.z = pack_bf16x2(__uint_as_float(a[8 * q4 + 4]), __uint_as_float(a[8 * q4 + 5]));
          wk.w = pack_bf16x2(__uint_as_float(a[8 * q4 + 6]), __uint_as_float(a[8 * q4 + 7]));
          wv.x = pack_bf16x2(__uint_as_float(v[8 * q4]), __uint_as_float(v[8 * q4 + 1]));
          wv.y = pack_bf16x2(__uint_as_float(v[8 * q4 + 2]), __uint_as_float(v[8 * q4 + 3]));
          wv.z = pack_bf16x2(__uint_as_float(v[8 * q4 + 4]), __uint_as_float(v[8 * q4 + 5]));
          wv.w = pack_bf16x2(__uint_as_float(v[8 * q4 + 6]), __uint_as_float(v[8 * q4 + 7]));
          const uint32_t off = sw128_offset((uint32_t)r, (uint32_t)(((col & 63) >> 3) + q4));
          *reinterpret_cast<uint4*>(tile_k + off) = wk;
          *reinterpret_cast<uint4*>(tile_v + off) = wv;
        }
      }
      fence_proxy_async_smem();
    }
    // every compute thread reaches this barrier, whatever happened above
    named_bar_sync(1, 256);
    if (tid_c == 0 && !*abort_flag) {
#pragma unroll
      for (int a = 0; a < D / 64; ++a) {
        tma_store_4d(&tdk, smem_u32(smem + L::kPOff + a * 16384), a * 64, k0, hkv, b);
        tma_store_4d(&tdv, smem_u32(smem + L::kPOff + (D / 64) * 16384 + a * 16384), a * 64, k0, hkv, b);
      }
      tma_store_commit();
      tma_store_wait_read<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[b,h,q] = sum_d dO[b,q,h,d] * O[b,q,h,d]; also zeroes the fp32 dQ accumulator row.
template <int D>
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ delta, float* __restrict__ dq_acc, int B, int H, int Lq,
                                     long long o_sb, long long o_ss, long long o_sh, long long do_sb,
                                     long long do_ss, long long do_sh) {
  // D/8 lanes per (b, q, h) row, 16-byte loads: a warp covers 4 rows (D = 64) or 2 rows (D = 128)
  constexpr int kLanes = D / 8;
  constexpr int kRowsPerWarp = 32 / kLanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / kLanes, l = lane % kLanes;
  const long long warp_id = (long long)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const long long row = warp_id * kRowsPerWarp + sub;
  const long long total = (long long)B * Lq * H;
  const bool live = row < total;
  float acc = 0.f;
  int h = 0, q = 0, b = 0;
  if (live) {
    h = (int)(row % H);
    const long long bq = row / H;
    q = (int)(bq % Lq);
    b = (int)(bq / Lq);
    const uint4 ua = __ldg(reinterpret_cast<const uint4*>(o + b * o_sb + q * o_ss + h * o_sh) + l);
    const uint4 uc = __ldg(reinterpret_cast<const uint4*>(dout + b * do_sb + q * do_ss + h * do_sh) + l);
    const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wc[4] = {uc.x, uc.y, uc.z, uc.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16x2(wa[k]), c = unpack_bf16x2(wc[k]);
      acc += a.x * c.x + a.y * c.y;
    }
  }
#pragma unroll
  for (int s = kLanes / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (live) {
    if (l == 0) delta[((long long)b * H + h) * Lq + q] = acc;
    float4* z = reinterpret_cast<float4*>(dq_acc + row * D + l * 8);
    z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// dq (bf16, strided [B,Lq,H,D]) = dq_acc (fp32 contiguous)
__global__ void attn_bwd_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int H, int Lq,
                                        int D, long long total_vec, long long sb, long long ss, long long sh) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one 8-element vector each
  if (i >= total_vec) return;
  const int vec_per_row = D / 8;
  const long long row = i / vec_per_row;
  const int vc = (int)(i % vec_per_row);
  const int h = (int)(row % H);
  const long long bq = row / H;
  const int q = (int)(bq % Lq);
  const long long b = bq / Lq;
  const float4 x = reinterpret_cast<const float4*>(acc)[2 * i], y = reinterpret_cast<const float4*>(acc)[2 * i + 1];
  uint4 w = make_uint4(pack_bf16x2(x.x, x.y), pack_bf16x2(x.z, x.w), pack_bf16x2(y.x, y.y), pack_bf16x2(y.z, y.w));
  *reinterpret_cast<uint4*>(dq + b * sb + q * ss + h * sh + vc * 8) = w;
}

template <int D>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const CUtensorMap& tdq, const CUtensorMap& tdk, const CUtensorMap& tdv, const AttnBwdParams& p,
                      cudaStream_t stream) {
  using L = AttnBwdSmem<D>;
  static bool configured[64] = {false};
  int dev = 0;
  MRK_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MRK_CUDA_OK(cudaFuncSetAttribute(attn_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured[dev & 63] = true;
  }
  dim3 grid((p.Lk + 127) / 128, p.Hkv, p.B);
  attn_bwd_kernel<D><<<grid, kBwdThreads, L::kTotal, stream>>>(tq, tk, tv, tdo, tdq, tdk, tdv, p);
  MRK_CHECK_LAUNCH();
  return 0;
}

}  // namespace mrk

using namespace mrk;

MRK_API int mrk_attn_bwd_drop(const void* q, const void* k, const void* v, const void* o, const void* dout,
                              const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                              const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                              const long long* strides /* q,k,v,o,do,dq,dk,dv: (sb,ss,sh) each = 24 values */,
                              int causal, float scale, float p_drop, const void* rng, unsigned long long call_id,
                              void* stream) {
  MRK_REQUIRE(p_drop >= 0.f && p_drop < 1.f && (p_drop == 0.f || rng != nullptr), "attention backward: bad dropout arguments");
  MRK_REQUIRE(D == 64 || D == 128, "attention backward: head dim %d not supported (64 or 128)", D);
  MRK_REQUIRE(B > 0 && H > 0 && Hkv > 0 && Lq > 0 && Lk > 0 && H % Hkv == 0, "attention backward: bad sizes");
  const long long* sq = strides, *sk = strides + 3, *sv = strides + 6, *so = strides + 9, *sdo = strides + 12,
                 *sdq = strides + 15, *sdk = strides + 18, *sdv = strides + 21;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_bshd_tmap(&tq, q, D, Lq, H, B, sq[0], sq[1], sq[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tk, k, D, Lk, Hkv, B, sk[0], sk[1], sk[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tv, v, D, Lk, Hkv, B, sv[0], sv[1], sv[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tdo, dout, D, Lq, H, B, sdo[0], sdo[1], sdo[2], 128))) return rc;
  CUtensorMap tdq;   // the fp32 dQ accumulator [B, Lq, H, D]: boxes of 32 queries x 32 columns of one head
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)Lq, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)D, (uint64_t)H * D, (uint64_t)Lq * H * D};
    const uint32_t box[4] = {32, 1, 32, 1};
    if ((rc = make_tmap_4d(&tdq, dq_acc, 4, dims, strides, box, 3))) return rc;
  }
  CUtensorMap tdk, tdv;
  if ((rc = make_bshd_tmap(&tdk, dk, D, Lk, Hkv, B, sdk[0], sdk[1], sdk[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tdv, dv, D, Lk, Hkv, B, sdv[0], sdv[1], sdv[2], 128))) return rc;
  const long long rows = (long long)B * Lq * H;
  {
    const int warps_per_block = 8;
    const long long rows_per_block = warps_per_block * (32 / (D / 8));      // D/8 lanes per row
    const long long blocks = (rows + rows_per_block - 1) / rows_per_block;
    if (D == 64)
      attn_bwd_prep_kernel<64><<<(unsigned)blocks, warps_per_block * 32, 0, s>>>(
          (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, dq_acc, B, H, Lq, so[0], so[1], so[2], sdo[0],
          sdo[1], sdo[2]);
    else
      attn_bwd_prep_kernel<128><<<(unsigned)blocks, warps_per_block * 32, 0, s>>>(
          (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, dq_acc, B, H, Lq, so[0], so[1], so[2], sdo[0],
          sdo[1], sdo[2]);
    MRK_CHECK_LAUNCH();
  }
  AttnBwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.dk_sb = sdk[0]; p.dk_ss = sdk[1]; p.dk_sh = sdk[2];
  p.dv_sb = sdv[0]; p.dv_ss = sdv[1]; p.dv_sh = sdv[2];
  p.key_bias = key_bias;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Lq = Lq; p.Lk = Lk; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.p_drop = p_drop; p.rng = reinterpret_cast<const unsigned long long*>(rng); p.call_id = call_id;
  p.status = status_word_device();
  MRK_REQUIRE(p.status != nullptr, "attention backward: status word unavailable");
  rc = (D == 64) ? launch_bwd<64>(tq, tk, tv, tdo, tdq, tdk, tdv, p, s)
                 : launch_bwd<128>(tq, tk, tv, tdo, tdq, tdk, tdv, p, s);
  if (rc) return rc;
  {
    const long long total_vec = rows * (D / 8);
    const int threads = 256;
    attn_bwd_dq_cast_kernel<<<(unsigned)((total_vec + threads - 1) / threads), threads, 0, s>>>(
        dq_acc, (__nv_bfloat16*)dq, H, Lq, D, total_vec, sdq[0], sdq[1], sdq[2]);
    MRK_CHECK_LAUNCH();
  }
  return 0;
}

MRK_API int mrk_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                         const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                         const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                         const long long* strides, int causal, float scale, void* stream) {
  return mrk_attn_bwd_drop(q, k, v, o, dout, lse, delta, dq_acc, dq, dk, dv, key_bias, B, H, Hkv, Lq, Lk, D, strides,
                           causal, scale, 0.f, nullptr, 0ull, stream);
}
