// C interface of the tcgen05 flash-attention kernels.  Tensors are bf16 with layout
// [batch, seq, head, dim] described by element strides (dim contiguous), so Q, K and V may be
// views into one fused QKV projection output.  lse is fp32 [batch, head, seq_q].
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int mrk_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                 const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                 long long q_sb, long long q_ss, long long q_sh,
                 long long k_sb, long long k_ss, long long k_sh,
                 long long v_sb, long long v_ss, long long v_sh,
                 long long o_sb, long long o_ss, long long o_sh,
                 int causal, float scale, void* stream);
// The same with dropout on the probabilities (attention_dropout.cuh): `rng` points at [seed, offset]
// (two 64-bit words on the device), `call_id` distinguishes the attention calls of a step; the
// backward call must get the same three values.
int mrk_attn_fwd_drop(const void* q, const void* k, const void* v, void* out, float* lse,
                      const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                      long long q_sb, long long q_ss, long long q_sh,
                      long long k_sb, long long k_ss, long long k_sh,
                      long long v_sb, long long v_ss, long long v_sh,
                      long long o_sb, long long o_ss, long long o_sh,
                      int causal, float scale, float p_drop, const void* rng, unsigned long long call_id,
                      void* stream);
#ifdef __cplusplus
}
#endif
#ifdef __cplusplus
extern "C" {
#endif
// Backward.  `delta` ([B,H,Lq] fp32) and `dq_acc` ([B,Lq,H,D] fp32) are scratch the caller provides;
// `strides` holds (batch, seq, head) element strides for q, k, v, o, dout, dq, dk, dv in that order.
int mrk_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                 const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                 const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                 const long long* strides, int causal, float scale, void* stream);
int mrk_attn_bwd_drop(const void* q, const void* k, const void* v, const void* o, const void* dout,
                      const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                      const float* key_bias, int B, int H, int Hkv, int Lq, int Lk, int D,
                      const long long* strides, int causal, float scale, float p_drop, const void* rng,
                      unsigned long long call_id, void* stream);
#ifdef __cplusplus
}
#endif
