#include "host_common.h"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

namespace mrk {

static thread_local char g_last_error[512] = {0};
static unsigned long long g_launches = 0;

void count_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code ? code : 1;
}

static constexpr int kMaxDevices = 64;
static unsigned* g_status_host[kMaxDevices] = {nullptr};
static unsigned* g_status_dev[kMaxDevices] = {nullptr};
static int g_sm_count[kMaxDevices] = {0};

unsigned* status_word_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status_dev[dev]) return g_status_dev[dev];
  unsigned* h = nullptr;
  if (cudaHostAlloc((void**)&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess)
    return nullptr;
  memset(h, 0, 64);
  unsigned* d = nullptr;
  if (cudaHostGetDevicePointer((void**)&d, h, 0) != cudaSuccess) return nullptr;
  g_status_host[dev] = h;
  g_status_dev[dev] = d;
  return d;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The encode call is a driver-API function: it needs the primary context bound to the calling
// thread, which a thread that has only seen cudaSetDevice (autograd worker threads) may lack.
static void bind_context_once() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  bind_context_once();
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

static CUtensorMapDataType dtype_of(int elem_bytes, bool is_float32) {
  if (elem_bytes == 2) return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (elem_bytes == 4) return is_float32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  return CU_TENSOR_MAP_DATA_TYPE_UINT8;
}

static CUtensorMapSwizzle swizzle_of(int s) {
  switch (s) {
    case 1: return CU_TENSOR_MAP_SWIZZLE_32B;
    case 2: return CU_TENSOR_MAP_SWIZZLE_64B;
    case 3: return CU_TENSOR_MAP_SWIZZLE_128B;
    default: return CU_TENSOR_MAP_SWIZZLE_NONE;
  }
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  MRK_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled entry point not found");
  MRK_REQUIRE(((uintptr_t)base & 15) == 0, "tensor map base %p is not 16-byte aligned", base);
  MRK_REQUIRE((ld_elems * elem_bytes) % 16 == 0,
              "tensor map row pitch %llu elements is not a multiple of 16 bytes",
              (unsigned long long)ld_elems);
  MRK_REQUIRE(box_inner <= 256 && box_outer <= 256, "tensor map box too large");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype_of(elem_bytes, true), 2, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of(swizzle),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MRK_REQUIRE(r == CUDA_SUCCESS,
              "cuTensorMapEncodeTiled(2d) failed with %d (inner=%llu outer=%llu ld=%llu box=%ux%u)",
              (int)r, (unsigned long long)inner, (unsigned long long)outer,
              (unsigned long long)ld_elems, box_inner, box_outer);
  return 0;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t mid,
                 uint64_t outer, uint64_t stride_mid_elems, uint64_t stride_outer_elems,
                 uint32_t box_inner, uint32_t box_mid, uint32_t box_outer, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  MRK_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled entry point not found");
  MRK_REQUIRE(((uintptr_t)base & 15) == 0, "tensor map base %p is not 16-byte aligned", base);
  MRK_REQUIRE((stride_mid_elems * elem_bytes) % 16 == 0 && (stride_outer_elems * elem_bytes) % 16 == 0,
              "tensor map strides must be multiples of 16 bytes");
  cuuint64_t dims[3] = {inner, mid, outer};
  cuuint64_t strides[2] = {stride_mid_elems * (uint64_t)elem_bytes,
                           stride_outer_elems * (uint64_t)elem_bytes};
  cuuint32_t box[3] = {box_inner, box_mid, box_outer};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype_of(elem_bytes, true), 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of(swizzle),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MRK_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(3d) failed with %d", (int)r);
  return 0;
}

int make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims[4],
                 const uint64_t strides_elems[3], const uint32_t box[4], int swizzle) {
  EncodeTiledFn fn = encode_fn();
  MRK_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled entry point not found");
  MRK_REQUIRE(((uintptr_t)base & 15) == 0, "tensor map base %p is not 16-byte aligned", base);
  cuuint64_t d[4], st[3];
  cuuint32_t bx[4], estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 4; ++i) { d[i] = dims[i]; bx[i] = box[i]; }
  for (int i = 0; i < 3; ++i) {
    st[i] = strides_elems[i] * (uint64_t)elem_bytes;
    MRK_REQUIRE(st[i] % 16 == 0, "tensor map stride %d (%llu elements) is not a multiple of 16 bytes", i,
                (unsigned long long)strides_elems[i]);
  }
  CUresult r = fn(out, dtype_of(elem_bytes, true), 4, const_cast<void*>(base), d, st, bx, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of(swizzle), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MRK_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(4d) failed with %d dims=(%llu,%llu,%llu,%llu)", (int)r,
              (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
              (unsigned long long)dims[3]);
  return 0;
}

}  // namespace mrk

// -------------------------------------------------------------------------------------------------
// exported C entry points
// -------------------------------------------------------------------------------------------------
MRK_API const char* mrk_last_error() { return mrk::g_last_error; }

// Reads (and optionally clears) the current device's status word. 0 = no kernel reported a problem.
MRK_API unsigned mrk_status_read(int clear) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= mrk::kMaxDevices) return 0xFFFFFFFFu;
  if (!mrk::g_status_host[dev]) return 0;
  unsigned v = *(volatile unsigned*)mrk::g_status_host[dev];
  if (clear) *(volatile unsigned*)mrk::g_status_host[dev] = 0;
  return v;
}

MRK_API int mrk_abi_version() { return 1; }

// Number of kernels this library has launched in this process (all devices, all threads).
MRK_API unsigned long long mrk_launch_count() { return mrk::g_launches; }
