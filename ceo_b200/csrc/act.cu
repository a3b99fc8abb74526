// SwiGLU / GELU / SiLU forward and backward and a row softmax; bf16 in/out, fp32 math.
// The reference has GELU kernels only (kernels/cuda/layernorm.cu:202-250); SiLU and
// SwiGLU exist there as CPU loops (src/nn/layers.zig:337-383) and its softmax takes
// the row max with an integer atomic on float bits (layernorm.cu:277).
#include "common/util.cuh"
#include "common/check.cuh"
#include "include/ceo_kernels.h"

CEO_BOUNDS_TU(act)

namespace ceo {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// 8 (gate, up) pairs of a row for output columns [8c, 8c+8): from the two halves of the row
// ([gate | up]) or, interleaved, from 16 consecutive values (gate_0, up_0, gate_1, ...).
__device__ __forceinline__ void load_gate_up(const uint4* row, int c, int fv, int il, float* g,
                                             float* u) {
  if (!il) {
    unpack8(row[c], g);
    unpack8(row[fv + c], u);
    return;
  }
  float a[8], b[8];
  unpack8(row[2 * c], a);
  unpack8(row[2 * c + 1], b);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    g[j] = a[2 * j]; u[j] = a[2 * j + 1];
    g[4 + j] = b[2 * j]; u[4 + j] = b[2 * j + 1];
  }
}

// gate_up: (rows, 2F) with gate in [:, :F] and up in [:, F:] (il = 0) or with gate and up in
// alternating columns (il = 1, the layout the fused GEMM epilogue uses).  out: (rows, F)
__global__ void swiglu_fwd_il_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out,
                                     long long rows, int F, int il) {
  const int fv = F >> 3;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / fv;
    const int c = static_cast<int>(i - r * fv);
    float g[8], u[8], o[8];
    load_gate_up(reinterpret_cast<const uint4*>(gu + r * 2 * F), CEO_IDX(c, fv, 204), fv, il, g, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j];
    reinterpret_cast<uint4*>(out)[CEO_IDX(r * fv + c, rows * fv, 205)] = pack8(o);
  }
}

__global__ void swiglu_bwd_il_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu,
                                     bf16* __restrict__ dgu, long long rows, int F, int il) {
  const int fv = F >> 3;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / fv;
    const int c = static_cast<int>(i - r * fv);
    float g[8], u[8], d[8], dg[8], du[8];
    load_gate_up(reinterpret_cast<const uint4*>(gu + r * 2 * F), c, fv, il, g, u);
    unpack8(reinterpret_cast<const uint4*>(dout + r * F)[c], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_(g[j]);
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    uint4* orow = reinterpret_cast<uint4*>(dgu + r * 2 * F);
    if (!il) {
      orow[c] = pack8(dg);
      orow[fv + c] = pack8(du);
    } else {
      float a[8], b[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a[2 * j] = dg[j]; a[2 * j + 1] = du[j];
        b[2 * j] = dg[4 + j]; b[2 * j + 1] = du[4 + j];
      }
      orow[2 * c] = pack8(a);
      orow[2 * c + 1] = pack8(b);
    }
  }
}

// gate_up: (rows, 2F) with gate in [:, :F] and up in [:, F:].  out: (rows, F)
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out,
                                  long long rows, int F) {
  const int fv = F >> 3;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / fv;
    const int c = static_cast<int>(i - r * fv);
    const uint4* row = reinterpret_cast<const uint4*>(gu + r * 2 * F);
    float g[8], u[8], o[8];
    unpack8(row[CEO_IDX(c, fv, 201)], g);
    unpack8(row[CEO_IDX(fv + c, 2 * fv, 202)], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j];
    reinterpret_cast<uint4*>(out)[CEO_IDX(r * fv + c, rows * fv, 203)] = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu,
                                  bf16* __restrict__ dgu, long long rows, int F) {
  const int fv = F >> 3;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / fv;
    const int c = static_cast<int>(i - r * fv);
    const uint4* row = reinterpret_cast<const uint4*>(gu + r * 2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[c], g);
    unpack8(row[fv + c], u);
    unpack8(reinterpret_cast<const uint4*>(dout + r * F)[c], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_(g[j]);
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    uint4* orow = reinterpret_cast<uint4*>(dgu + r * 2 * F);
    orow[c] = pack8(dg);
    orow[fv + c] = pack8(du);
  }
}

// ---------------------------------------------------------------------------- dropout
// y = x * keep / (1 - p) with keep decided by a stateless hash of (element index, seed), so
// the backward pass re-creates the mask from the seed instead of storing it: apply the same
// call to dy.  Counterpart of the reference's CPU Dropout layer (src/nn/layers.zig:461-503),
// which draws from a host RNG and keeps a mask tensor.
__device__ __forceinline__ unsigned dropout_hash(unsigned long long idx, unsigned seed) {
  unsigned x = static_cast<unsigned>(idx) ^ seed ^ (static_cast<unsigned>(idx >> 32) * 0x9E3779B9u);
  x ^= x >> 16; x *= 0x7feb352du;
  x ^= x >> 15; x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
__global__ void dropout_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n,
                               float p, float scale, unsigned seed) {
  const long long n8 = n >> 3;
  const unsigned thresh = static_cast<unsigned>(p * 16777216.f);  // keep iff top 24 bits >= p
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      f[j] = (dropout_hash(static_cast<unsigned long long>(i) * 8 + j, seed) >> 8) >= thresh
                 ? f[j] * scale : 0.f;
    reinterpret_cast<uint4*>(y)[i] = pack8(f);
  }
  // tail (n not a multiple of 8)
  for (long long i = (n8 << 3) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const bool keep = (dropout_hash(static_cast<unsigned long long>(i), seed) >> 8) >= thresh;
    y[i] = __float2bfloat16(keep ? __bfloat162float(x[i]) * scale : 0.f);
  }
}

// mode 0: tanh GELU, 1: erf GELU, 2: SiLU, 3: ReLU
__device__ __forceinline__ float act_f(float x, int mode) {
  if (mode == 0) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
  } else if (mode == 1) {
    return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  } else if (mode == 2) {
    return x * sigmoidf_(x);
  }
  return x > 0.f ? x : 0.f;
}
__device__ __forceinline__ float act_df(float x, int mode) {
  if (mode == 0) {
    const float k = 0.7978845608028654f;
    const float inner = k * (x + 0.044715f * x * x * x);
    const float t = tanhf(inner);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
  } else if (mode == 1) {
    const float cdf = 0.5f * (1.f + erff(x * 0.7071067811865476f));
    const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
    return cdf + x * pdf;
  } else if (mode == 2) {
    const float s = sigmoidf_(x);
    return s + x * s * (1.f - s);
  }
  return x > 0.f ? 1.f : 0.f;
}

__global__ void act_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n8,
                               int mode) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = act_f(v[j], mode);
    reinterpret_cast<uint4*>(y)[i] = pack8(v);
  }
}
__global__ void act_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                               bf16* __restrict__ dx, long long n8, int mode) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v[8], g[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], v);
    unpack8(reinterpret_cast<const uint4*>(dy)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= act_df(v[j], mode);
    reinterpret_cast<uint4*>(dx)[i] = pack8(g);
  }
}

// Row softmax over the last dimension (fp32 in, fp32 out), one CTA per row.
__global__ void __launch_bounds__(256)
softmax_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int n) {
  __shared__ float red[33];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + static_cast<size_t>(row) * n;
    float* yr = y + static_cast<size_t>(row) * n;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_reduce_max(m, red);
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += __expf(xr[i] - m);
    s = block_reduce_sum(s, red);
    const float inv = 1.f / s;
    for (int i = threadIdx.x; i < n; i += blockDim.x) yr[i] = __expf(xr[i] - m) * inv;
  }
}

}  // namespace ceo
using namespace ceo;

extern "C" int ceo_swiglu_fwd(const void* gate_up, void* out, long long rows, int F,
                              cudaStream_t stream) {
  if (rows <= 0 || F <= 0 || (F & 7)) return -5;
  swiglu_fwd_kernel<<<grid_for(rows * (F >> 3), 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(gate_up), static_cast<bf16*>(out), rows, F);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_swiglu_bwd(const void* dout, const void* gate_up, void* dgate_up,
                              long long rows, int F, cudaStream_t stream) {
  if (rows <= 0 || F <= 0 || (F & 7)) return -5;
  swiglu_bwd_kernel<<<grid_for(rows * (F >> 3), 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(dout), static_cast<const bf16*>(gate_up),
      static_cast<bf16*>(dgate_up), rows, F);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_swiglu_il_fwd(const void* gate_up, void* out, long long rows, int F,
                                 int interleaved, cudaStream_t stream) {
  if (rows <= 0 || F <= 0 || (F & 7)) return -5;
  swiglu_fwd_il_kernel<<<grid_for(rows * (F >> 3), 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(gate_up), static_cast<bf16*>(out), rows, F, interleaved);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_swiglu_il_bwd(const void* dout, const void* gate_up, void* dgate_up,
                                 long long rows, int F, int interleaved, cudaStream_t stream) {
  if (rows <= 0 || F <= 0 || (F & 7)) return -5;
  swiglu_bwd_il_kernel<<<grid_for(rows * (F >> 3), 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(dout), static_cast<const bf16*>(gate_up),
      static_cast<bf16*>(dgate_up), rows, F, interleaved);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_act_fwd(const void* x, void* y, long long n, int mode, cudaStream_t stream) {
  if (n <= 0 || (n & 7)) return -5;
  act_fwd_kernel<<<grid_for(n >> 3, 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(x), static_cast<bf16*>(y), n >> 3, mode);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_act_bwd(const void* dy, const void* x, void* dx, long long n, int mode,
                           cudaStream_t stream) {
  if (n <= 0 || (n & 7)) return -5;
  act_bwd_kernel<<<grid_for(n >> 3, 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(dy), static_cast<const bf16*>(x), static_cast<bf16*>(dx), n >> 3,
      mode);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_dropout(const void* x, void* y, long long n, float p, unsigned int seed,
                           cudaStream_t stream) {
  if (n <= 0 || !(p >= 0.f) || p >= 1.f ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15))
    return -5;
  dropout_kernel<<<grid_for(n, 256 * 8 * 2, 148 * 8), 256, 0, stream>>>(
      static_cast<const bf16*>(x), static_cast<bf16*>(y), n, p, 1.f / (1.f - p), seed);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_softmax_fwd(const float* x, float* y, int rows, int n, cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return -5;
  softmax_fwd_kernel<<<rows < 65535 ? rows : 65535, 256, 0, stream>>>(x, y, rows, n);
  return static_cast<int>(cudaGetLastError());
}
