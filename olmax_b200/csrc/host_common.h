// Host-side helpers shared by the .cu files: error strings, TMA tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda, so the library also builds on a machine without a driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

namespace ob {

// Last host-side error message of this library (per thread); returned by ob_last_error().
inline char* last_error_buf() {
  static thread_local char buf[512];
  return buf;
}
#define OB_FAIL(code, ...)                                   \
  do {                                                       \
    snprintf(::ob::last_error_buf(), 512, __VA_ARGS__);      \
    return (code);                                           \
  } while (0)

#define OB_CUDA_OK(expr)                                                                          \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess) OB_FAIL(-(int)_e, "%s failed: %s", #expr, cudaGetErrorString(_e));     \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Encode a rank-`rank` (<= 4) bf16/f32 tensor map with 128-byte swizzle.  dims/box innermost first;
// strides_bytes has rank-1 entries (stride of dims 1..rank-1).
inline int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) OB_FAIL(-1000, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t d[5];
  cuuint64_t s[5];
  cuuint32_t b[5];
  cuuint32_t e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) OB_FAIL(-1001, "TMA base address not 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (s[i] % 16 != 0) OB_FAIL(-1002, "TMA stride %d (%llu bytes) not a multiple of 16", i, (unsigned long long)s[i]);
  CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) OB_FAIL(-1003, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace ob
