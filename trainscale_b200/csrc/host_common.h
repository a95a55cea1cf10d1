// Host-side helpers shared by the launchers: error-word API, TMA tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda, so the libraries also build on machines
// without a driver), and argument checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

namespace ts {

#define TS_DEFINE_ERROR_API(prefix)                                                                   \
  extern "C" int prefix##_get_error(unsigned int* out4) {                                             \
    return (int)cudaMemcpyFromSymbol(out4, ts::g_ts_error, 4 * sizeof(unsigned int));                 \
  }                                                                                                   \
  extern "C" int prefix##_clear_error() {                                                             \
    unsigned int z[4] = {0, 0, 0, 0};                                                                 \
    return (int)cudaMemcpyToSymbol(ts::g_ts_error, z, sizeof(z));                                     \
  }

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point needs a current context in the calling thread; a thread that has not made a
// runtime call yet (e.g. an autograd worker) has none, so bind the primary context once per thread.
inline void ensure_thread_context() {
  static thread_local bool ready = false;
  if (!ready) {
    cudaFree(0);
    ready = true;
  }
}

inline PFN_encodeTiled get_encode_fn() {
  ensure_thread_context();
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

// 2-D row-major tensor [rows][cols] of `elem_bytes`-wide elements with row pitch `ld` elements;
// box = box_rows x box_cols, 128-byte swizzle (box_cols * elem_bytes must be 128).
// Returns 0 on success.
inline int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                        CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B) {
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || ((ld * elem_bytes) & 15u) != 0) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "[trainscale_b200] cuTensorMapEncodeTiled failed (%d): base=%p rows=%llu cols=%llu ld=%llu box=%ux%u\n",
            (int)r, base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows, box_cols);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D tensor [d2][d1][d0] (d0 contiguous), strides in elements for d1 and d2.
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t d0,
                        uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2,
                        CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B) {
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || ((s1 * elem_bytes) & 15u) != 0 ||
      ((s2 * elem_bytes) & 15u) != 0)
    return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * (uint64_t)elem_bytes, s2 * (uint64_t)elem_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
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

}  // namespace ts
