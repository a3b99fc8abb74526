// Host helper: encode a 2-D bf16 tensor map (row-major matrix, leading dimension in elements)
// with a {64 columns x box_rows} box and 128-byte swizzle, through the driver entry point the
// runtime hands out (the library links libcudart only).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace ceo {

typedef CUresult (*TmapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TmapEncodeFn tmap_encode_fn() {
  static TmapEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TmapEncodeFn>(p);
  }
  return fn;
}

// Returns 0, or the CUresult / -1 on failure.  ptr and ld_elems * 2 must be multiples of 16.
inline int encode_tmap_2d_bf16(CUtensorMap* tm, const void* ptr, uint64_t cols, uint64_t rows,
                               uint64_t ld_elems, uint32_t box_rows) {
  TmapEncodeFn fn = tmap_encode_fn();
  if (!fn) return -1;
  // The driver entry point needs a current context; a thread that has made no runtime call
  // yet (an autograd worker thread, for one) has none until the runtime binds it.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "ceo: tensor map rejected (%d): ptr=%p cols=%llu rows=%llu ld=%llu box_rows=%u\n",
            static_cast<int>(r), ptr, (unsigned long long)cols, (unsigned long long)rows,
            (unsigned long long)ld_elems, box_rows);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// The same matrix seen as (64 columns, rows, cols / 64): a box of {64, box_rows, box_panels}
// brings box_panels adjacent 64-column panels of box_rows rows with ONE request, laid out
// panel after panel (each panel box_rows x 128 bytes, 128-byte swizzle) - the layout the
// per-panel 2-D loads produce.  cols must be a multiple of 64.
inline int encode_tmap_panels_bf16(CUtensorMap* tm, const void* ptr, uint64_t cols, uint64_t rows,
                                   uint64_t ld_elems, uint32_t box_rows, uint32_t box_panels) {
  TmapEncodeFn fn = tmap_encode_fn();
  if (!fn || (cols & 63)) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[3] = {64, rows, cols / 64};
  cuuint64_t strides[2] = {ld_elems * 2, 128};
  cuuint32_t box[3] = {64, box_rows, box_panels};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "ceo: panel tensor map rejected (%d): ptr=%p cols=%llu rows=%llu ld=%llu\n",
            static_cast<int>(r), ptr, (unsigned long long)cols, (unsigned long long)rows,
            (unsigned long long)ld_elems);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace ceo
