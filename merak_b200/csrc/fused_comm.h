// C interface of the symmetric-memory data plane and the fused compute+collective kernels.
// Pointer arrays (`*_ptrs`) are host arrays of `n` device pointers, one per rank of the group,
// entry `rank` being this process's own buffer.  0 = success.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int mrk_symm_alloc(unsigned long long bytes, void** out);
int mrk_symm_free(void* p);
int mrk_symm_ctrl_bytes();
int mrk_ipc_handle_bytes();
int mrk_ipc_get_handle(void* p, unsigned char* out);
int mrk_ipc_open(const unsigned char* handle, void** out);
int mrk_ipc_close(void* p);
int mrk_dp_reduce_scatter(void* const* grad_ptrs, void* const* ctrl_ptrs, int n, int rank, long long lo, long long cnt,
                          const unsigned char* flags, unsigned epoch, int sync, int budget_ms, void* stream);
// One device-to-device copy on `stream` (copy engine; either side may be peer-mapped memory).
int mrk_memcpy_d2d_async(void* dst, const void* src, unsigned long long bytes, void* stream);
int mrk_dp_adamw_allgather(void* const* model_ptrs, void* const* ctrl_ptrs, int n, int rank, long long lo,
                           long long cnt, const float* grad_shard, float* master, float* m, float* v,
                           const unsigned char* flags, const float* hp, float grad_scale, float max_norm,
                           const float* sumsq_src, float* norm_out, int* skip_out, unsigned epoch, int sync,
                           int wait_partials, int budget_ms, void* stream);
int mrk_dp_norm_gather(void* const* ctrl_ptrs, int n, int rank, float* out2, unsigned epoch, int sync, int budget_ms,
                       void* stream);
int mrk_symm_barrier(void* const* ctrl_ptrs, int n, int rank, int which, unsigned epoch, int signal, int budget_ms,
                     void* stream);
int mrk_tp_reduce_pull(void* const* part_ptrs, void* const* ctrl_ptrs, int n, int rank, void* out, long long rows_local,
                       int N, int seg_rows, const void* bias, unsigned epoch, int sync, int budget_ms, void* stream);
int mrk_tp_gather_rows(void* const* red_ptrs, void* const* ctrl_ptrs, int n, int rank, void* out, long long M, int N,
                       int seg_rows, unsigned epoch, int sync, int budget_ms, void* stream);
int mrk_moe_alltoall_push(void* const* recv_ptrs, void* const* ctrl_ptrs, int n, int rank, const void* send,
                          const long long* send_begin, const long long* dst_row, int H, int elem_bytes, unsigned epoch,
                          int sync, int budget_ms, void* stream);
#ifdef __cplusplus
}
#endif
