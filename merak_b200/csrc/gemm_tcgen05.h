// C interface of the tcgen05 GEMM.  All pointers are device pointers; `stream` is a cudaStream_t.
// Every function returns 0 on success; on failure the text is available from mrk_last_error().
#pragma once

enum MrkAct { MRK_ACT_NONE = 0, MRK_ACT_GELU_ERF = 1, MRK_ACT_GELU_TANH = 2, MRK_ACT_RELU = 3, MRK_ACT_SILU = 4 };

// What the epilogue does with `aux_in` ([M,N] bf16):
//   ADD : out = act(acc*alpha + bias) + aux_in              (residual connection)
//   DACT: out = (acc*alpha + bias) * act'(aux_in)            (backward through an activation whose
//                                                             pre-activation input was saved)
enum MrkAuxMode { MRK_AUX_NONE = 0, MRK_AUX_ADD = 1, MRK_AUX_DACT = 2 };

enum MrkGemmFlags {
  MRK_GEMM_OUT_F32 = 1,      // C is fp32 (default bf16)
  MRK_GEMM_ACCUMULATE = 2,   // C += result (gradient accumulation across micro-batches)
  MRK_GEMM_BIAS_F32 = 4,     // bias vector is fp32 (default bf16)
  MRK_GEMM_A_MN = 8,         // A is stored [K, M] row-major (default [M, K])
  MRK_GEMM_B_MN = 16,        // B is stored [K, N] row-major (default [N, K])
};

#ifdef __cplusplus
extern "C" {
#endif
// C[M,N] = epilogue(alpha * op(A) * op(B)^T).  lda/ldb/ldc/ld_aux_* are row pitches in elements.
// aux_out (optional, bf16 [M,N]) receives acc*alpha + bias before the activation.
// block_n: 0 = choose, or 64 / 128 / 256.
int mrk_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                  long long ldb, long long ldc, const void* bias, const void* aux_in,
                  long long ld_aux_in, void* aux_out, long long ld_aux_out, int act, int aux_mode,
                  int flags, float alpha, int block_n, void* stream);
// All-gather -> GEMM for tensor parallelism over peer-mapped memory (see gemm_common.cuh).
int mrk_gemm_bf16_ag(void* gathered, void* const* peer_shards, const void* B, void* C, int M, int N, int K,
                     long long ldb, long long ldc, const void* bias, void* aux_out, long long ld_aux_out, int act,
                     int flags, float alpha, void* const* ctrls, unsigned* seg_flags, unsigned flag_target,
                     int gather_ctas, int n, int rank, int seg_rows, unsigned epoch, int budget_ms, void* stream);
// GEMM -> reduce-scatter in one launch over peer-mapped partial-product buffers (gemm_common.cuh, mode 1).
int mrk_gemm_bf16_rs_units(int M, int N);
int mrk_gemm_bf16_rs(const void* A, const void* B, void* const* parts, void* const* tile_flags, void* out,
                     const void* bias, int M, int N, int K, long long lda, long long ldb, int flags, int n, int rank,
                     int seg_rows, unsigned epoch, int phase, int reduce_ctas, unsigned* queue, int budget_ms,
                     void* stream);
#ifdef __cplusplus
}
#endif
