// C interface of the memory-bound kernels (norms, cross entropy, AdamW, embedding, RoPE, SwiGLU,
// column sums, dropout, casts).  Device pointers; `stream` is a cudaStream_t; 0 = success.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int mrk_norm_fwd(const void* x, const void* residual, const void* gamma, const void* beta, void* y, void* z,
                 float* mean, float* rstd, const void* rng, unsigned long long call_id, float p_drop, float eps,
                 long long M, int H, int rms, int params_f32, void* stream);
int mrk_norm_bwd(const void* dy, const void* z, const void* dz_extra, const void* gamma, const float* mean,
                 const float* rstd, void* dres, void* dx, float* dgamma, float* dbeta, float* workspace,
                 const void* rng, unsigned long long call_id, float p_drop, long long M, int H, int rms,
                 int params_f32, void* stream);
int mrk_norm_bwd_workspace_rows();
int mrk_ce_stats(const void* logits, const long long* labels, float* stats, long long M, int V, long long ld,
                 int vocab_start, int ignore_index, int logits_f32, void* stream);
int mrk_ce_finalize(const float* stats, int tp_parts, long long part_stride, const long long* labels, float* lse,
                    float* loss_rows, float* loss_sum, float* valid_count, long long M, int ignore_index, void* stream);
int mrk_ce_grad(const void* logits, const long long* labels, const float* lse, const float* grad_scale, void* dlogits,
                long long M, int V, long long ld, long long ldd, int vocab_start, int ignore_index, int logits_f32,
                void* stream);
int mrk_adamw(float* master, float* m, float* v, const void* grad, void* model_out, const float* hp,
              const float* grad_scale, const int* skip, long long n, int grad_f32, int out_f32, void* stream);
int mrk_sumsq(const void* x, long long n, float* out2, int is_f32, void* stream);
int mrk_clip_coef(const float* sumsq2, float base_scale, float max_norm, float* scale_out, int* skip_out,
                  float* norm_out, void* stream);
int mrk_embedding_fwd(const void* const* tables, const long long* const* idx, const int* rows, const int* starts,
                      int count, void* out, long long T, int H, void* stream);
int mrk_embedding_bwd(const void* dout, const long long* idx, void* dtable, long long T, int H, int rows, int start,
                      int grad_f32, void* stream);
int mrk_rope(const void* x, void* y, const float* cosb, const float* sinb, const long long* pos, long long B, int L,
             int H, int D, long long sb, long long ss, long long sh, long long ysb, long long yss, long long ysh,
             int inverse, void* stream);
int mrk_swiglu_fwd(const void* gu, void* out, long long M, int F, long long ld, void* stream);
int mrk_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long M, int F, long long ld, void* stream);
int mrk_act_fwd(const void* x, void* y, long long n, int act, void* stream);
int mrk_act_bwd(const void* d, const void* h, void* out, float* colsum_out, long long M, int N, long long ld, int act,
                void* stream);
int mrk_colsum(const void* x, float* out, long long M, int N, long long ld, void* stream);
// Next-token sampling (csrc/sampling.cu): temperature / top-k (1..1024) / top-p / draw for a batch of rows.
int mrk_sample_topk_topp(const void* logits, int is_bf16, long long rows, int V, long long row_stride, int top_k,
                         float top_p, float temperature, int greedy, const float* uniforms, unsigned long long seed,
                         unsigned long long step, long long* out_token, float* out_prob, void* stream);
int mrk_dropout(const void* x, void* y, long long n, float p, const void* rng, unsigned long long call_id, void* stream);
int mrk_scaled_cast(const void* x, void* y, long long n, const float* scale_ptr, float scale, int in_f32, int out_f32,
                    int accumulate, void* stream);
#ifdef __cplusplus
}
#endif
