// Flash attention forward on tcgen05: O = softmax(scale * Q K^T + mask) V, plus the row
// log-sum-exp needed by the backward pass.  One CTA owns one 128-row query block of one
// (batch, head); key/value blocks of 128 stream through a TMA-fed shared-memory ring.
//
//   warp 0       TMA producer (Q once, then K/V blocks)
//   warp 1       UMMA issuer:  S_j = Q K_j^T  (TMEM, double buffered)   and   O_j = P_j V_j (TMEM)
//   warps 2..5   softmax: thread r owns query row r (TMEM lane r): row max / exp2 / row sum need
//                no shuffles; P_j is written to shared memory as the 128B-swizzled A operand of
//                the second product; the running output is rescaled and accumulated in registers.
// S_{j+1} is issued before P_j V_j, so the tensor core works on the next score block while the
// softmax warps process the current one.
//
// Replaces the eager matmul -> softmax -> dropout -> matmul attention the reference's models use
// (examples/models/gpt2/config.py:28 forces eager attention) and the SDPA/FlashAttention-2 calls
// of its sequence-parallel Llama layer (Merak/core/sequence_parallel/modeling/llama.py:24-160).
#include "attention.h"
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace mrk {

constexpr int kQ = 128;   // query rows per CTA
constexpr int kKV = 128;  // keys per block
constexpr int kAttnThreads = 192;

struct AttnFwdParams {
  __nv_bfloat16* out;           // [B, Lq, H, D] with strides below
  long long o_sb, o_ss, o_sh;   // batch / seq / head strides (elements)
  float* lse;                   // [B, H, Lq]
  const float* key_bias;        // optional [B, Lk], added to every score column
  int B, H, Hkv, Lq, Lk;
  int causal;
  float scale_log2;             // softmax scale * log2(e)
  unsigned* status;
};

template <int D>
struct AttnFwdSmem {
  static constexpr int kTile = 128 * D * 2;                  // one Q / K / V tile
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = kTile;
  static constexpr int kPOff = kKVOff + kStages * 2 * kTile;
  static constexpr int kBarOff = kPOff + kPBytes;
  static constexpr int kBiasOff = kBarOff + 256;             // 2 x 128 floats: key bias of the current / next block
  static constexpr int kTotal = kBiasOff + 1024 + 1024;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnFwdParams p) {
  using L = AttnFwdSmem<D>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kOCol = 256;  // S buffers at columns 0 and 128, O at 256

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // kStages
  uint64_t* kv_empty = kv_full + kStages;  // kStages
  uint64_t* s_full = kv_empty + kStages;   // 2
  uint64_t* s_empty = s_full + 2;          // 2
  uint64_t* p_full = s_empty + 2;          // 1
  uint64_t* o_full = p_full + 1;           // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (p.H / p.Hkv);
  const int q0 = q_blk * kQ;

  int n_blocks = (p.Lk + kKV - 1) / kKV;
  if (p.causal) {
    // keys visible to the last row of this block: row + (Lk - Lq)
    const int last_key = min(p.Lk - 1, q0 + kQ - 1 + (p.Lk - p.Lq));
    n_blocks = last_key < 0 ? 0 : min(n_blocks, last_key / kKV + 1);
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 128);
    }
    mbar_init(smem_u32(p_full), 128);
    mbar_init(smem_u32(o_full), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t q_smem = smem_u32(smem + L::kQOff);
  const uint32_t p_smem = smem_u32(smem + L::kPOff);

  if (warp == 0) {
    if (lane == 0 && n_blocks > 0) {
      mbar_arrive_expect_tx(smem_u32(q_full), L::kTile);
#pragma unroll
      for (int a = 0; a < D / 64; ++a)
        tma_load_4d(q_smem + a * 16384, &tq, smem_u32(q_full), a * 64, q0, h, b);
      int stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j < n_blocks; ++j) {
        if (!mbar_wait(smem_u32(&kv_empty[stage]), phase ^ 1u, abort_flag, p.status)) break;
        const uint32_t fb = smem_u32(&kv_full[stage]);
        const uint32_t ks = smem_u32(smem + L::kKVOff + stage * 2 * L::kTile);
        const uint32_t vs = ks + L::kTile;
        mbar_arrive_expect_tx(fb, 2 * L::kTile);
#pragma unroll
        for (int a = 0; a < D / 64; ++a) {
          tma_load_4d(ks + a * 16384, &tk, fb, a * 64, j * kKV, hkv, b);
          tma_load_4d(vs + a * 16384, &tv, fb, a * 64, j * kKV, hkv, b);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_blocks > 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);  // Q (K-major) x K (K-major)
      const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);    // P (K-major) x V (MN-major)
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status);
      int stage = 0;
      uint32_t phase = 0;
      int pv_stage = 0;
      for (int j = 0; j <= n_blocks && ok; ++j) {
        if (j < n_blocks) {
          ok = mbar_wait(smem_u32(&kv_full[stage]), phase, abort_flag, p.status);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&s_empty[j & 1]), ((j >> 1) & 1) ^ 1u, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t ks = smem_u32(smem + L::kKVOff + stage * 2 * L::kTile);
          const uint32_t s_tmem = tmem_base + (j & 1) * 128;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t da = desc_kmajor(q_smem + (k / 4) * 16384, k % 4);
            const uint64_t db = desc_kmajor(ks + (k / 4) * 16384, k % 4);
            umma_bf16_ss(s_tmem, da, db, idesc_s, k != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&s_full[j & 1]));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (j >= 1) {
          const int jj = j - 1;
          ok = mbar_wait(smem_u32(p_full), jj & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t vs = smem_u32(smem + L::kKVOff + pv_stage * 2 * L::kTile) + L::kTile;
#pragma unroll
          for (int k = 0; k < kKV / 16; ++k) {
            const uint64_t da = desc_kmajor(p_smem + (k / 4) * 16384, k % 4);
            const uint64_t db = desc_mnmajor(vs, k, 128);
            umma_bf16_ss(tmem_base + kOCol, da, db, idesc_o, k != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&kv_empty[pv_stage]));
          umma_commit(smem_u32(o_full));
          if (++pv_stage == kStages) pv_stage = 0;
        }
      }
    }
  } else {
    // ------------------------------- softmax / output -------------------------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // row inside the block == TMEM lane
    const int row = q0 + r;                  // query index
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int causal_shift = p.Lk - p.Lq;    // key j visible to query i iff j <= i + shift
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    const float* kb = p.key_bias ? p.key_bias + (long long)b * p.Lk : nullptr;
    float* kbs_base = reinterpret_cast<float*>(smem + L::kBiasOff);

    for (int j = 0; j < n_blocks && ok; ++j) {
      ok = mbar_wait(smem_u32(&s_full[j & 1]), (j >> 1) & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + lane_off + (j & 1) * 128;
      const int k0 = j * kKV;
      // Key bias of this block goes to shared memory once (thread r stages key k0+r); blocks whose
      // bias is all zero (no padding) take the unbiased path.
      bool has_bias = false;
      float* kbs = kbs_base + (j & 1) * 128;   // double buffered: a fast thread may already stage block j+1
      if (kb != nullptr) {
        const float bv = (k0 + r < p.Lk) ? __ldg(kb + k0 + r) * 1.4426950408889634f : 0.f;
        uint32_t any_nz;
        kbs[r] = bv;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.f32 q, %1, 0f00000000;\n\t"
            "bar.red.or.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(any_nz) : "f"(bv) : "memory");
        has_bias = any_nz != 0;
      }
      const bool need_mask = (k0 + kKV > p.Lk) || (p.causal && (k0 + kKV - 1 > q0 + causal_shift)) || has_bias;
      // pass 1: row maximum
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld32(s_tmem + c * 32, s);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = k0 + c * 32 + i;
            float v = __uint_as_float(s[i]) * p.scale_log2;
            if (has_bias) v += kbs[c * 32 + i];
            if (col >= p.Lk || (p.causal && col > row + causal_shift)) v = -INFINITY;
            m_blk = fmaxf(m_blk, v);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) m_blk = fmaxf(m_blk, __uint_as_float(s[i]) * p.scale_log2);
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);   // m_run = -inf -> 0
      // fold in the previous block's product, then rescale
      if (j > 0) {
        ok = mbar_wait(smem_u32(o_full), (j - 1) & 1, abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_off + kOCol + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = (acc[c * 32 + i] + __uint_as_float(o[i])) * alpha;
        }
      }
      // pass 2: probabilities -> shared memory (A operand of P V), row sum
      float l_blk = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld32(s_tmem + c * 32, s);
        tmem_wait_ld();
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(s[i]) * p.scale_log2;
          if (need_mask) {
            const int col = k0 + c * 32 + i;
            if (has_bias) v += kbs[c * 32 + i];
            if (col >= p.Lk || (p.causal && col > row + causal_shift)) v = -INFINITY;
          }
          pr[i] = exp2f(v - m_use);
        }
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          packed[i] = pack_bf16x2(pr[2 * i], pr[2 * i + 1]);
          const float2 back = unpack_bf16x2(packed[i]);  // sum what the tensor core will see
          l_blk += back.x + back.y;
        }
        // columns c*32 .. c*32+31 live in k-atom (c/2), 16-byte chunks (c%2)*4 .. +3 of row r
        uint8_t* tile = smem + L::kPOff + (c >> 1) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off = sw128_offset((uint32_t)r, (uint32_t)((c & 1) * 4 + q));
          *reinterpret_cast<uint4*>(tile + off) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      tc_fence_before();
      mbar_arrive(smem_u32(&s_empty[j & 1]));
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(p_full));
    }
    if (n_blocks > 0 && ok) {
      ok = mbar_wait(smem_u32(o_full), (n_blocks - 1) & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_off + kOCol + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(o[i]);
        }
      }
    }
    if (row < p.Lq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = p.out + (long long)b * p.o_sb + (long long)row * p.o_ss + (long long)h * p.o_sh;
#pragma unroll
      for (int q = 0; q < D / 8; ++q) {
        uint4 w = make_uint4(pack_bf16x2(acc[8 * q] * inv, acc[8 * q + 1] * inv),
                             pack_bf16x2(acc[8 * q + 2] * inv, acc[8 * q + 3] * inv),
                             pack_bf16x2(acc[8 * q + 4] * inv, acc[8 * q + 5] * inv),
                             pack_bf16x2(acc[8 * q + 6] * inv, acc[8 * q + 7] * inv));
        reinterpret_cast<uint4*>(dst)[q] = w;
      }
      if (p.lse)
        p.lse[((long long)b * p.H + h) * p.Lq + row] =
            l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
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

template <int D>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const AttnFwdParams& p, cudaStream_t stream) {
  using L = AttnFwdSmem<D>;
  static bool configured[64] = {false};
  int dev = 0;
  MRK_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MRK_CUDA_OK(cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured[dev & 63] = true;
  }
  dim3 grid((p.Lq + kQ - 1) / kQ, p.H, p.B);
  attn_fwd_kernel<D><<<grid, kAttnThreads, L::kTotal, stream>>>(tq, tk, tv, p);
  MRK_CHECK_LAUNCH();
  return 0;
}

int make_bshd_tmap(CUtensorMap* out, const void* base, int D, int L, int H, int B, long long sb, long long ss,
                   long long sh, int box_rows) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)L, (uint64_t)H, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)ss, (uint64_t)sh, (uint64_t)sb};
  const uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tmap_4d(out, base, 2, dims, strides, box, 3);
}

}  // namespace mrk

using namespace mrk;

MRK_API int mrk_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                         const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                         long long q_sb, long long q_ss, long long q_sh,
                         long long k_sb, long long k_ss, long long k_sh,
                         long long v_sb, long long v_ss, long long v_sh,
                         long long o_sb, long long o_ss, long long o_sh,
                         int causal, float scale, void* stream) {
  MRK_REQUIRE(D == 64 || D == 128, "attention: head dim %d not supported (64 or 128)", D);
  MRK_REQUIRE(B > 0 && H > 0 && Hkv > 0 && Lq > 0 && Lk > 0 && H % Hkv == 0, "attention: bad sizes");
  MRK_REQUIRE((o_ss % 8) == 0 && (o_sh % 8) == 0 && (o_sb % 8) == 0 && ((uintptr_t)out & 15) == 0,
              "attention: output must be 16-byte aligned per row");
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_bshd_tmap(&tq, q, D, Lq, H, B, q_sb, q_ss, q_sh, 128))) return rc;
  if ((rc = make_bshd_tmap(&tk, k, D, Lk, Hkv, B, k_sb, k_ss, k_sh, 128))) return rc;
  if ((rc = make_bshd_tmap(&tv, v, D, Lk, Hkv, B, v_sb, v_ss, v_sh, 128))) return rc;
  AttnFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.o_sb = o_sb; p.o_ss = o_ss; p.o_sh = o_sh;
  p.lse = lse; p.key_bias = key_bias;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Lq = Lq; p.Lk = Lk;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word_device();
  MRK_REQUIRE(p.status != nullptr, "attention: status word unavailable");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return D == 64 ? launch_fwd<64>(tq, tk, tv, p, s) : launch_fwd<128>(tq, tk, tv, p, s);
}
