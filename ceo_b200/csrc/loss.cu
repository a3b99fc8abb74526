// Softmax cross-entropy: loss and d(logits) in one kernel, with label smoothing
// and an ignore index.  One CTA per row; online max/sum in the first pass, the
// gradient in the second (the row is L2-resident between them).  Used on
// row-chunks of the LM-head output so the full (tokens x vocab) logits are never
// materialised.  The reference declares cross_entropy_{forward,backward}_cuda
// (kernels/cuda/include/kernels.h:248-270) without a source; the math follows
// its CPU reference (src/kernels/nn_kernels.zig:200-248).
#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

template <typename T>
__device__ __forceinline__ float ld_f(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_f<bf16>(const bf16* p, long long i) {
  return __bfloat162float(p[i]);
}

// loss_row = lse - (1-ls)*z_t - ls/V * sum_j z_j
// dlogit_j = scale * (p_j - (1-ls)*[j==t] - ls/V)
template <typename T>
__global__ void __launch_bounds__(512)
cross_entropy_kernel(const T* __restrict__ logits, const long long* __restrict__ targets,
                     float* __restrict__ loss, bf16* __restrict__ dlogits, int rows, int V,
                     long long ld, long long ldd, float ls, const float* __restrict__ scale_ptr,
                     float scale, long long ignore_index) {
  __shared__ float red[33];
  const float gscale = scale * (scale_ptr ? *scale_ptr : 1.f);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* z = logits + row * ld;
    const long long t = targets[row];
    const bool ignored = (t == ignore_index) || t < 0 || t >= V;
    float m = -INFINITY, s = 0.f, zs = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = ld_f<T>(z, i);
      zs += v;
      if (v > m) {
        s = s * __expf(m - v) + 1.f;
        m = v;
      } else {
        s += __expf(v - m);
      }
    }
    const float gm = block_reduce_max(m, red);
    s = block_reduce_sum(s * __expf(m - gm), red);
    zs = block_reduce_sum(zs, red);
    const float lse = gm + __logf(s);
    if (threadIdx.x == 0 && loss) {
      float l = 0.f;
      if (!ignored) l = lse - (1.f - ls) * ld_f<T>(z, t) - ls * zs / V;
      loss[row] = l;
    }
    if (dlogits) {
      bf16* d = dlogits + row * ldd;
      const float inv = 1.f / s;
      const float sm = ls / V;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float g = 0.f;
        if (!ignored) {
          const float p = __expf(ld_f<T>(z, i) - gm) * inv;
          g = gscale * (p - sm - (i == t ? (1.f - ls) : 0.f));
        }
        d[i] = __float2bfloat16(g);
      }
    }
  }
}

}  // namespace ceo
using namespace ceo;

extern "C" int ceo_cross_entropy(const void* logits, int logits_f32, const long long* targets,
                                 float* loss, void* dlogits, int rows, int V, long long ld,
                                 long long ldd, float label_smoothing, const float* scale_ptr,
                                 float scale, long long ignore_index, cudaStream_t stream) {
  if (rows <= 0 || V <= 0) return -5;
  const int grid = rows < 148 * 64 ? rows : 148 * 64;
  if (logits_f32)
    cross_entropy_kernel<float><<<grid, 512, 0, stream>>>(
        static_cast<const float*>(logits), targets, loss, static_cast<bf16*>(dlogits), rows, V, ld,
        ldd, label_smoothing, scale_ptr, scale, ignore_index);
  else
    cross_entropy_kernel<bf16><<<grid, 512, 0, stream>>>(
        static_cast<const bf16*>(logits), targets, loss, static_cast<bf16*>(dlogits), rows, V, ld,
        ldd, label_smoothing, scale_ptr, scale, ignore_index);
  return static_cast<int>(cudaGetLastError());
}
