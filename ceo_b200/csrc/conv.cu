// Causal depthwise short convolution (the ShortConv of the PRISM branch):
//   y[b,t,d] = sum_{w=0}^{W-1} x[b,t-w,d] * weight[d,w]
// forward, input gradient (the same stencil run anti-causally) and weight gradient.
// The reference declares shortconv_forward_cuda (kernels/cuda/include/kernels.h:107) and a
// backward (src/kernels/prism_kernels.zig:50-60) without sources; its CPU loop is
// src/model/prism.zig:448-476.
#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

constexpr int SC_CH = 256;  // channels per CTA (32 lanes x 8)
constexpr int SC_TT = 8;    // time steps per warp iteration

// dir = +1: causal (reads t-w); dir = -1: anti-causal (reads t+w) for the input gradient.
__global__ void __launch_bounds__(256)
shortconv_kernel(const bf16* __restrict__ x, const bf16* __restrict__ weight,
                 bf16* __restrict__ y, int T, int D, int Wn, int dir) {
  extern __shared__ float wsm[];  // [Wn][SC_CH]
  const int c0 = blockIdx.x * SC_CH;
  for (int i = threadIdx.x; i < Wn * SC_CH; i += blockDim.x) {
    const int w = i / SC_CH, c = i - w * SC_CH;
    wsm[i] = (c0 + c < D) ? __bfloat162float(weight[static_cast<size_t>(c0 + c) * Wn + w]) : 0.f;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = c0 + lane * 8;
  if (ch >= D) return;
  const int b = blockIdx.z;
  const bf16* xb = x + static_cast<size_t>(b) * T * D;
  bf16* yb = y + static_cast<size_t>(b) * T * D;
  for (int t = blockIdx.y * 8 + warp; t < T; t += gridDim.y * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < Wn; ++w) {
      const int ts = t - dir * w;
      if (ts < 0 || ts >= T) break;
      float xv[8];
      unpack8(*reinterpret_cast<const uint4*>(xb + static_cast<size_t>(ts) * D + ch), xv);
      const float* wr = wsm + w * SC_CH + lane * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += xv[j] * wr[j];
    }
    *reinterpret_cast<uint4*>(yb + static_cast<size_t>(t) * D + ch) = pack8(acc);
  }
}

// dW[d,w] = sum_{b,t} dy[b,t,d] * x[b,t-w,d];  grid (D/32, Wn), block (32 channels, 8 slices)
__global__ void __launch_bounds__(256)
shortconv_dw_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                    float* __restrict__ dw, int B, int T, int D, int Wn, int accumulate) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + lane;
  const int w = blockIdx.y;
  float s = 0.f;
  if (d < D) {
    for (int b = 0; b < B; ++b) {
      const bf16* dyb = dy + static_cast<size_t>(b) * T * D + d;
      const bf16* xb = x + static_cast<size_t>(b) * T * D + d;
      for (int t = w + slice; t < T; t += 8)
        s += __bfloat162float(dyb[static_cast<size_t>(t) * D]) *
             __bfloat162float(xb[static_cast<size_t>(t - w) * D]);
    }
  }
  red[slice][lane] = s;
  __syncthreads();
  if (slice == 0 && d < D) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i][lane];
    float* o = dw + static_cast<size_t>(d) * Wn + w;
    *o = accumulate ? *o + tot : tot;
  }
}

}  // namespace ceo
using namespace ceo;

static int shortconv_launch(const void* x, const void* weight, void* y, int B, int T, int D,
                            int Wn, int dir, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || D <= 0 || (D & 7) || Wn <= 0 || Wn > 192) return -5;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(shortconv_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         192 * SC_CH * 4);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg = true;
  }
  int gy = (T + 7) / 8;
  if (gy > 64) gy = 64;
  dim3 grid((D + SC_CH - 1) / SC_CH, gy, B);
  shortconv_kernel<<<grid, 256, Wn * SC_CH * 4, stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(weight), static_cast<bf16*>(y), T, D,
      Wn, dir);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_shortconv_fwd(const void* x, const void* weight, void* y, int B, int T, int D,
                                 int Wn, cudaStream_t stream) {
  return shortconv_launch(x, weight, y, B, T, D, Wn, 1, stream);
}
extern "C" int ceo_shortconv_bwd_input(const void* dy, const void* weight, void* dx, int B, int T,
                                       int D, int Wn, cudaStream_t stream) {
  return shortconv_launch(dy, weight, dx, B, T, D, Wn, -1, stream);
}
extern "C" int ceo_shortconv_bwd_weight(const void* dy, const void* x, float* dw, int B, int T,
                                        int D, int Wn, int accumulate, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || D <= 0 || Wn <= 0) return -5;
  dim3 grid((D + 31) / 32, Wn);
  shortconv_dw_kernel<<<grid, 256, 0, stream>>>(static_cast<const bf16*>(dy),
                                                static_cast<const bf16*>(x), dw, B, T, D, Wn,
                                                accumulate);
  return static_cast<int>(cudaGetLastError());
}
