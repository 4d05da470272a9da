// Host-side helpers shared by every translation unit of the kernel library:
// error reporting through a thread-local message, the per-device status word that device
// code raises when a bounded wait gives up, and TMA tensor-map construction.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MRK_API extern "C" __attribute__((visibility("default")))

namespace mrk {

// Records `msg` as the calling thread's last error and returns `code` (non-zero).
int fail(int code, const char* fmt, ...);

#define MRK_CUDA_OK(expr)                                                                \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return ::mrk::fail(100 + (int)_e, "%s failed: %s (%s:%d)", #expr,                  \
                         cudaGetErrorString(_e), __FILE__, __LINE__);                    \
  } while (0)

// After every kernel launch: count it (mrk_launch_count) and surface launch errors.
#define MRK_CHECK_LAUNCH()                                                               \
  do {                                                                                   \
    ::mrk::count_launch();                                                               \
    MRK_CUDA_OK(cudaGetLastError());                                                     \
  } while (0)

#define MRK_REQUIRE(cond, ...)                                                           \
  do {                                                                                   \
    if (!(cond)) return ::mrk::fail(2, __VA_ARGS__);                                     \
  } while (0)

// Device-visible pointer to the current device's status word (mapped pinned host memory,
// so the host can read it while a kernel is still running).  nullptr on failure.
unsigned* status_word_device();

// 2-D bf16/fp16/fp32 row-major tensor map: `inner` contiguous elements per row, `outer` rows,
// row pitch `ld_elems` elements.  The box is box_inner x box_outer elements.
// swizzle: 0 = none, 1 = 32B, 2 = 64B, 3 = 128B.
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer, int swizzle);

// 3-D variant: dims (inner, mid, outer) with strides in elements for mid and outer.
int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t mid,
                 uint64_t outer, uint64_t stride_mid_elems, uint64_t stride_outer_elems,
                 uint32_t box_inner, uint32_t box_mid, uint32_t box_outer, int swizzle);

// 4-D variant used for [batch, seq, head, dim] tensors: dims (d0..d3), strides for d1..d3 in elements.
int make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims[4],
                 const uint64_t strides_elems[3], const uint32_t box[4], int swizzle);

int sm_count();

void count_launch();

}  // namespace mrk
