// Flash attention forward on tcgen05: O = softmax(scale * Q K^T + mask) V, plus the row
// log-sum-exp needed by the backward pass.
//
// One CTA owns NT query tiles of 128 rows of one (batch, head) (NT = 2 for head dim 64, 1 for 128);
// key/value blocks of 128 stream through a TMA-fed shared-memory ring shared by the tiles.
//
//   warp 0          TMA producer (Q tiles once, then K/V blocks)
//   warp 1          UMMA issuer: per tile t and key block j:  S_t = Q_t K_j^T  and  O_t = P_t V_j
//   warps 2..5      softmax warpgroup of tile 0      (thread r owns query row r = TMEM lane r:
//   warps 6..9      softmax warpgroup of tile 1       row max / exp2 / row sum need no shuffles)
//
// The two warpgroups ping-pong: while one runs the softmax of its score block on the CUDA cores,
// the tensor core computes the other tile's scores and P V product.  P goes to shared memory as
// the 128B-swizzled A operand of the second product; each block's P V result is read back from
// TMEM and folded into a register accumulator with the (deferred) rescale factor, one FMA per
// element.
//
// Replaces the eager matmul -> softmax -> dropout -> matmul attention the reference's models use
// (examples/models/gpt2/config.py:28 forces eager attention) and the SDPA/FlashAttention-2 calls
// of its sequence-parallel Llama layer (Merak/core/sequence_parallel/modeling/llama.py:24-160).
#include "attention.h"
#include "host_common.h"
#include "sm100_ptx.cuh"
#include "attention_dropout.cuh"

namespace mrk {

constexpr int kKV = 128;  // keys per block

struct AttnFwdParams {
  __nv_bfloat16* out;           // [B, Lq, H, D] with strides below
  long long o_sb, o_ss, o_sh;   // batch / seq / head strides (elements)
  float* lse;                   // [B, H, Lq]
  const float* key_bias;        // optional [B, Lk], added to every score column
  int B, H, Hkv, Lq, Lk;
  int causal;
  float scale_log2;             // softmax scale * log2(e)
  float p_drop;                 // dropout on the probabilities (0 = off)
  const unsigned long long* rng;   // [seed, offset] on the device when p_drop > 0
  unsigned long long call_id;
  unsigned* status;
};

template <int D, int NT>
struct AttnFwdSmem {
  static constexpr int kTile = 128 * D * 2;                  // one Q / K / V tile
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = NT * kTile;
  static constexpr int kPOff = kKVOff + kStages * 2 * kTile;
  static constexpr int kBarOff = kPOff + NT * kPBytes;
  static constexpr int kBiasOff = kBarOff + 256;             // NT x 2 x 128 floats: staged key bias
  static constexpr int kTotal = kBiasOff + NT * 1024 + 1024;
  static constexpr int kThreads = 64 + NT * 128;
};

// Barrier over the 128 threads of one softmax warpgroup that also ORs a predicate (v != 0).
__device__ __forceinline__ bool named_bar_any_nonzero(uint32_t bar_id, float v) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.f32 q, %1, 0f00000000;\n\t"
      "bar.red.or.pred p, %2, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "f"(v), "r"(bar_id) : "memory");
  return r != 0;
}

template <int D, int NT>
__global__ void __launch_bounds__(AttnFwdSmem<D, NT>::kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap to,
                const AttnFwdParams p) {
  using L = AttnFwdSmem<D, NT>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kOCol = 256;  // S_t at column t*128, O_t at 256 + t*D

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // kStages
  uint64_t* kv_empty = kv_full + kStages;  // kStages
  uint64_t* s_full = kv_empty + kStages;   // per tile
  uint64_t* p_full = s_full + 2;           // per tile (128 arrivals): P_t written, S_t and O_t consumed
  uint64_t* o_full = p_full + 2;           // per tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (p.H / p.Hkv);
  const int q0 = q_blk * (128 * NT);
  const int causal_shift = p.Lk - p.Lq;    // key j visible to query i iff j <= i + shift

  // key blocks needed by tile t (causal: up to the diagonal of its last row)
  int n_tile[2] = {0, 0};
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    int n = (p.Lk + kKV - 1) / kKV;
    if (q0 + t * 128 >= p.Lq) n = 0;
    else if (p.causal) {
      const int last_key = min(p.Lk - 1, q0 + t * 128 + 127 + causal_shift);
      n = last_key < 0 ? 0 : min(n, last_key / kKV + 1);
    }
    n_tile[t] = n;
  }
  const int n_blocks = max(n_tile[0], n_tile[1]);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&s_full[t]), 1);
      mbar_init(smem_u32(&p_full[t]), 128);
      mbar_init(smem_u32(&o_full[t]), 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
    tma_prefetch_desc(&to);
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
      mbar_arrive_expect_tx(smem_u32(q_full), NT * L::kTile);
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int a = 0; a < D / 64; ++a)
          tma_load_4d(q_smem + t * L::kTile + a * 16384, &tq, smem_u32(q_full), a * 64, q0 + t * 128, h, b);
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
      int stage = 0, pv_stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j <= n_blocks && ok; ++j) {
        uint32_t ks = 0;
        if (j < n_blocks) {
          ok = mbar_wait(smem_u32(&kv_full[stage]), phase, abort_flag, p.status);
          if (!ok) break;
          ks = smem_u32(smem + L::kKVOff + stage * 2 * L::kTile);
        }
        const uint32_t vs = smem_u32(smem + L::kKVOff + pv_stage * 2 * L::kTile) + L::kTile;
        for (int t = 0; t < NT && ok; ++t) {
          const bool do_s = j < n_tile[t];
          const bool do_pv = j >= 1 && (j - 1) < n_tile[t];
          if (do_pv) {   // softmax of block j-1 finished: S_t and O_t are free, P_t is ready
            ok = mbar_wait(smem_u32(&p_full[t]), (j - 1) & 1, abort_flag, p.status);
            if (!ok) break;
          }
          tc_fence_after();
          if (do_s) {
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint64_t da = desc_kmajor(q_smem + t * L::kTile + (k / 4) * 16384, k % 4);
              const uint64_t db = desc_kmajor(ks + (k / 4) * 16384, k % 4);
              umma_bf16_ss(tmem_base + t * 128, da, db, idesc_s, k != 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&s_full[t]));
          }
          if (do_pv) {
#pragma unroll
            for (int k = 0; k < kKV / 16; ++k) {
              const uint64_t da = desc_kmajor(p_smem + t * L::kPBytes + (k / 4) * 16384, k % 4);
              const uint64_t db = desc_mnmajor(vs, k, 128);
              umma_bf16_ss(tmem_base + kOCol + t * D, da, db, idesc_o, k != 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&o_full[t]));
          }
        }
        if (!ok) break;
        if (j >= 1) {
          umma_commit(smem_u32(&kv_empty[pv_stage]));    // block j-1 fully consumed by every tile
          if (++pv_stage == kStages) pv_stage = 0;
        }
        if (j < n_blocks) {
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
#include "attention_fwd_softmax.inc"
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, int NT>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                      const AttnFwdParams& p, cudaStream_t stream) {
  using L = AttnFwdSmem<D, NT>;
  static bool configured[64] = {false};
  int dev = 0;
  MRK_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MRK_CUDA_OK(cudaFuncSetAttribute(attn_fwd_kernel<D, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured[dev & 63] = true;
  }
  dim3 grid((p.Lq + 128 * NT - 1) / (128 * NT), p.H, p.B);
  attn_fwd_kernel<D, NT><<<grid, L::kThreads, L::kTotal, stream>>>(tq, tk, tv, to, p);
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

MRK_API int mrk_attn_fwd_drop(const void* q, const void* k, const void* v, void* out, float* lse,
                              const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                              long long q_sb, long long q_ss, long long q_sh,
                              long long k_sb, long long k_ss, long long k_sh,
                              long long v_sb, long long v_ss, long long v_sh,
                              long long o_sb, long long o_ss, long long o_sh,
                              int causal, float scale, float p_drop, const void* rng, unsigned long long call_id,
                              void* stream) {
  MRK_REQUIRE(p_drop >= 0.f && p_drop < 1.f && (p_drop == 0.f || rng != nullptr), "attention: bad dropout arguments");
  MRK_REQUIRE(D == 64 || D == 128, "attention: head dim %d not supported (64 or 128)", D);
  MRK_REQUIRE(B > 0 && H > 0 && Hkv > 0 && Lq > 0 && Lk > 0 && H % Hkv == 0, "attention: bad sizes");
  MRK_REQUIRE((o_ss % 8) == 0 && (o_sh % 8) == 0 && (o_sb % 8) == 0 && ((uintptr_t)out & 15) == 0,
              "attention: output must be 16-byte aligned per row");
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_bshd_tmap(&tq, q, D, Lq, H, B, q_sb, q_ss, q_sh, 128))) return rc;
  if ((rc = make_bshd_tmap(&tk, k, D, Lk, Hkv, B, k_sb, k_ss, k_sh, 128))) return rc;
  if ((rc = make_bshd_tmap(&tv, v, D, Lk, Hkv, B, v_sb, v_ss, v_sh, 128))) return rc;
  CUtensorMap to;
  if ((rc = make_bshd_tmap(&to, out, D, Lq, H, B, o_sb, o_ss, o_sh, 128))) return rc;
  AttnFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.o_sb = o_sb; p.o_ss = o_ss; p.o_sh = o_sh;
  p.lse = lse; p.key_bias = key_bias;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Lq = Lq; p.Lk = Lk;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.p_drop = p_drop;
  p.rng = reinterpret_cast<const unsigned long long*>(rng);
  p.call_id = call_id;
  p.status = status_word_device();
  MRK_REQUIRE(p.status != nullptr, "attention: status word unavailable");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 64) return Lq > 128 ? launch_fwd<64, 2>(tq, tk, tv, to, p, s) : launch_fwd<64, 1>(tq, tk, tv, to, p, s);
  return launch_fwd<128, 1>(tq, tk, tv, to, p, s);
}

MRK_API int mrk_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                         const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                         long long q_sb, long long q_ss, long long q_sh,
                         long long k_sb, long long k_ss, long long k_sh,
                         long long v_sb, long long v_ss, long long v_sh,
                         long long o_sb, long long o_ss, long long o_sh,
                         int causal, float scale, void* stream) {
  return mrk_attn_fwd_drop(q, k, v, out, lse, key_bias, B, H, Hkv, Lq, Lk, D, q_sb, q_ss, q_sh, k_sb, k_ss, k_sh,
                           v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, causal, scale, 0.f, nullptr, 0ull, stream);
}
