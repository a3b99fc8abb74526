// Checked indexing for the debug build of the library (-DCEO_BOUNDS_CHECK, built by
// `python -m ceo_b200.build --bounds-check` into libceo_b200_chk.so).
//
// CEO_IDX(i, n, site) is `i` in the normal build.  In the checked build an index outside
// [0, n) is recorded - the first violation of each source file wins: site, index, extent -
// and redirected to element 0, so a wrong index neither traps nor touches memory outside the
// tensor; ceo_bounds_status() collects the records of all files.  Role of the reference's
// `compute-sanitizer --tool memcheck` pass over its smoke test (scripts/profile.sh:51-66) on
// machines where that tool is not available.
#pragma once
#include <cuda_runtime.h>

#ifdef CEO_BOUNDS_CHECK
// One record per translation unit (no relocatable device code in this build).
#define CEO_BOUNDS_TU(name)                                                                   \
  namespace ceo {                                                                             \
  static __device__ unsigned long long g_bounds_rec[4]; /* count, site, index, extent */      \
  }                                                                                           \
  extern "C" int ceo_bounds_collect_##name(unsigned long long* out, int reset) {              \
    cudaError_t e = cudaMemcpyFromSymbol(out, ceo::g_bounds_rec, 4 * sizeof(unsigned long long)); \
    if (e == cudaSuccess && reset) {                                                          \
      const unsigned long long z[4] = {0, 0, 0, 0};                                           \
      e = cudaMemcpyToSymbol(ceo::g_bounds_rec, z, sizeof(z));                                \
    }                                                                                         \
    return static_cast<int>(e);                                                               \
  }
#define CEO_IDX(i, n, site) ceo_checked_index(ceo::g_bounds_rec, (i), (n), (site))
__device__ __forceinline__ long long ceo_checked_index(unsigned long long* rec, long long i,
                                                       long long n, int site) {
  if (i >= 0 && i < n) return i;
  if (atomicAdd(rec, 1ull) == 0) {
    rec[1] = static_cast<unsigned long long>(site);
    rec[2] = static_cast<unsigned long long>(i);
    rec[3] = static_cast<unsigned long long>(n);
  }
  return 0;
}
#else
#define CEO_BOUNDS_TU(name)
#define CEO_IDX(i, n, site) (i)
#endif
