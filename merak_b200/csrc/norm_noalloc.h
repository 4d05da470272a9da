// mrk_norm_bwd_noalloc: LayerNorm / RMSNorm backward that allocates nothing.
//
// This entry point has no counterpart in the reference framework (which has no CUDA code of its
// own); it exists for callers of this library that are not allowed to obtain device memory at the
// moment they need the gradient: code running while an allocator lock is held or inside a
// memory-pool callback, a process whose whole GPU memory was handed out up front, or an embedding
// application that may launch kernels but must not call cudaMalloc.  Such callers cannot supply the
// partial-sum workspace mrk_norm_bwd asks for, so here the workspace is a fixed array inside the
// library (512 KiB per GPU, held from library load until the process exits).
//
// Differences from mrk_norm_bwd:
//   * no workspace argument and no dropout (rng) arguments; everything else means the same;
//   * hidden size H must be a multiple of 8 and at most 2048, otherwise the call fails with an
//     error text (mrk_last_error) and launches nothing;
//   * the first call on each device looks up the device address of the built-in array; make that
//     first call with the device current and before any stream capture is started;
//   * all calls share the one array: two calls that may overlap on the same GPU (different
//     streams, different threads) race on it and must be ordered by the caller.  Every call
//     clears the array on the caller's stream before it accumulates into it and a completed call
//     leaves it zero again, so a call that failed between its two launches (the return code says
//     so) does not spoil later calls;
//   * it calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// dy, z, dz_extra (optional), dres, dx: bf16 [M, H]; gamma: bf16 or fp32 [H] (params_f32);
// mean (nullptr for RMSNorm), rstd: fp32 [M]; dgamma, dbeta (optional): fp32 [H], overwritten.
// dx may equal dres.  Returns 0 on success.
int mrk_norm_bwd_noalloc(const void* dy, const void* z, const void* dz_extra, const void* gamma, const float* mean,
                         const float* rstd, void* dres, void* dx, float* dgamma, float* dbeta, long long M, int H,
                         int rms, int params_f32, void* stream);
#ifdef __cplusplus
}
#endif
