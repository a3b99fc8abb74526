// Softmax cross-entropy: loss and d(logits) in one kernel, with label smoothing
// and an ignore index.  fp32 rows of up to 32768 logits are read ONCE into registers
// (cross_entropy_reg_kernel: 16 x 16 bytes per thread, all requested before any is used);
// other shapes take one CTA per row with an online max/sum pass and a second pass for the
// gradient (the row is L2-resident between them).  Used on
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

// Register-resident rows: V = 4 * V4 <= 4 * 512 * NV fp32 logits, thread t holds the float4
// pieces t, t + 512, ...  One global read of the logits, 8-byte stores of the bf16 gradient.
template <int NV>
__global__ void __launch_bounds__(512)
cross_entropy_reg_kernel(const float* __restrict__ logits, const long long* __restrict__ targets,
                         float* __restrict__ loss, bf16* __restrict__ dlogits, int rows, int V,
                         long long ld, long long ldd, float ls,
                         const float* __restrict__ scale_ptr, float scale,
                         long long ignore_index) {
  __shared__ float red[33];
  __shared__ float red3[3][17];
  const int V4 = V >> 2, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float gscale = scale * (scale_ptr ? *scale_ptr : 1.f);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* z4 = reinterpret_cast<const float4*>(logits + row * ld);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = threadIdx.x + i * 512;
      v[i] = idx < V4 ? z4[idx] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    const long long t = targets[row];
    const bool ignored = (t == ignore_index) || t < 0 || t >= V;
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    const float gm = block_reduce_max(m, red);
    float sum = 0.f, zs = 0.f, zt = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = threadIdx.x + i * 512;
      if (idx < V4) {
        float* c = reinterpret_cast<float*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          zs += c[j];
          if (4 * idx + j == t) zt = c[j];
          c[j] = __expf(c[j] - gm);  // the registers now hold the unnormalised probabilities
          sum += c[j];
        }
      }
    }
    // three sums through one pair of barriers
    sum = warp_reduce_sum(sum);
    zs = warp_reduce_sum(zs);
    zt = warp_reduce_sum(zt);
    if (lane == 0) {
      red3[0][warp] = sum;
      red3[1][warp] = zs;
      red3[2][warp] = zt;
    }
    __syncthreads();
    if (warp < 3) {
      float x = lane < 16 ? red3[warp][lane] : 0.f;
      x = warp_reduce_sum(x);
      if (lane == 0) red3[warp][16] = x;
    }
    __syncthreads();
    sum = red3[0][16];
    zs = red3[1][16];
    zt = red3[2][16];
    if (threadIdx.x == 0 && loss)
      loss[row] = ignored ? 0.f : gm + __logf(sum) - (1.f - ls) * zt - ls * zs / V;
    if (dlogits) {
      uint2* d = reinterpret_cast<uint2*>(dlogits + row * ldd);
      const float inv = ignored ? 0.f : gscale / sum;
      const float sm = ignored ? 0.f : gscale * ls / V;
      const float hit = ignored ? 0.f : gscale * (1.f - ls);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int idx = threadIdx.x + i * 512;
        if (idx < V4) {
          const float* c = reinterpret_cast<const float*>(&v[i]);
          float g[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) g[j] = c[j] * inv - sm - (4 * idx + j == t ? hit : 0.f);
          uint2 o;
          bf162* h = reinterpret_cast<bf162*>(&o);
          h[0] = __floats2bfloat162_rn(g[0], g[1]);
          h[1] = __floats2bfloat162_rn(g[2], g[3]);
          d[idx] = o;
        }
      }
    }
    __syncthreads();  // red3 is rewritten by the next row
  }
}

}  // namespace ceo
using namespace ceo;

extern "C" int ceo_cross_entropy(const void* logits, int logits_f32, const long long* targets,
                                 float* loss, void* dlogits, int rows, int V, long long ld,
                                 long long ldd, float label_smoothing, const float* scale_ptr,
                                 float scale, long long ignore_index, cudaStream_t stream) {
  if (rows <= 0 || V <= 0) return -5;
  const bool reg_rows = logits_f32 && (V & 3) == 0 && V <= 4 * 512 * 16 && (ld & 3) == 0 &&
                        (ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0 &&
                        (reinterpret_cast<uintptr_t>(dlogits) & 7) == 0;
  if (reg_rows) {
    const int g = rows < 148 * 2 ? rows : 148 * 2;
    cross_entropy_reg_kernel<16><<<g, 512, 0, stream>>>(
        static_cast<const float*>(logits), targets, loss, static_cast<bf16*>(dlogits), rows, V, ld,
        ldd, label_smoothing, scale_ptr, scale, ignore_index);
    return static_cast<int>(cudaGetLastError());
  }
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
