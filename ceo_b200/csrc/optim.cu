// Fused optimizers on flat buffers: fp32 master weights + fp32 moments, bf16 or
// fp32 gradients, bf16 shadow parameters written by the same kernel.  Global-norm
// clipping never leaves the device: the squared norm is reduced into a device
// scalar, a 1-thread kernel turns it into a scale, and the update kernels read
// that scale through a pointer.
//
// Covers the reference's lion_step / adamw_step / muon_step / clip_grad_norm
// entry points (kernels/cuda/optim.cu:366, 657, 403, 711), which keep bf16
// parameters and moments, launch once per tensor, and synchronise the stream to
// read the norm on the host (optim.cu:511-527, 765-775).
#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

template <typename T>
__device__ __forceinline__ float ldg_f(const T* p, long long i);
template <>
__device__ __forceinline__ float ldg_f<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldg_f<bf16>(const bf16* p, long long i) {
  return __bfloat162float(p[i]);
}

// ---------------------------------------------------------------- sum of squares
template <typename T>
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[33];
  float s = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = ldg_f<T>(x, i);
    s += v * v;
  }
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256)
sumsq_final_kernel(const float* __restrict__ partial, int nblk, float* out, int accumulate) {
  __shared__ float red[33];
  float s = 0.f;
  for (int i = threadIdx.x; i < nblk; i += blockDim.x) s += partial[i];
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) *out = accumulate ? *out + s : s;
}

// scale = min(1, max_norm / (sqrt(sumsq) + 1e-6)); norm_out = sqrt(sumsq)
__global__ void clip_scale_kernel(const float* sumsq, float max_norm, float* scale_out,
                                  float* norm_out) {
  const float nrm = sqrtf(*sumsq);
  if (norm_out) *norm_out = nrm;
  float sc = 1.f;
  if (max_norm > 0.f && nrm > max_norm) sc = max_norm / (nrm + 1e-6f);
  if (!isfinite(nrm)) sc = 0.f;  // a non-finite gradient skips the step instead of poisoning it
  *scale_out = sc;
}

template <typename T>
__global__ void scale_kernel(T* x, long long n, const float* scale_ptr, float scale);
template <>
__global__ void scale_kernel<float>(float* x, long long n, const float* scale_ptr, float scale) {
  const float s = scale * (scale_ptr ? *scale_ptr : 1.f);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] *= s;
}
template <>
__global__ void scale_kernel<bf16>(bf16* x, long long n, const float* scale_ptr, float scale) {
  const float s = scale * (scale_ptr ? *scale_ptr : 1.f);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
}

// clamp to [-c, c]
__global__ void clip_value_kernel(float* x, long long n, float c) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] = fminf(fmaxf(x[i], -c), c);
}

// A clip scale of exactly zero marks a step whose gradient norm was not finite
// (clip_scale_kernel): every update kernel then leaves master weights, moments and shadow
// parameters untouched and only zeroes the gradients it was asked to zero.
__device__ __forceinline__ bool step_skipped(const float* gscale_ptr) {
  return gscale_ptr != nullptr && *gscale_ptr == 0.f;
}
template <typename G>
__device__ __forceinline__ void zero_range(G* grad, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    grad[i] = static_cast<G>(0.f);
}
__device__ __forceinline__ void zero_range4(float4* grad, long long n4) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    grad[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// ------------------------------------------------------------------------ AdamW
template <typename G>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             G* __restrict__ grad, bf16* __restrict__ shadow, long long n, float lr, float b1,
             float b2, float eps, float wd, float bc1_inv, float bc2_inv,
             const float* __restrict__ gscale_ptr, float gscale, int zero_grad) {
  if (step_skipped(gscale_ptr)) {
    if (zero_grad) zero_range<G>(grad, n);
    return;
  }
  const float gs = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = ldg_f<G>(grad, i) * gs;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float p = master[i];
    p = p * (1.f - lr * wd) - lr * (mi * bc1_inv) / (sqrtf(vi * bc2_inv) + eps);
    master[i] = p;
    if (shadow) shadow[i] = __float2bfloat16(p);
    if (zero_grad) grad[i] = static_cast<G>(0.f);
  }
}

// ------------------------------------------------------------------------- Lion
// u = b1*m + (1-b1)*g ; p = p*(1-lr*wd) - lr*sign(u) ; m = b2*m + (1-b2)*g
template <typename G>
__global__ void __launch_bounds__(256)
lion_kernel(float* __restrict__ master, float* __restrict__ m, G* __restrict__ grad,
            bf16* __restrict__ shadow, long long n, float lr, float b1, float b2, float wd,
            const float* __restrict__ gscale_ptr, float gscale, int zero_grad) {
  if (step_skipped(gscale_ptr)) {
    if (zero_grad) zero_range<G>(grad, n);
    return;
  }
  const float gs = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = ldg_f<G>(grad, i) * gs;
    const float mi = m[i];
    const float u = b1 * mi + (1.f - b1) * g;
    const float sgn = u > 0.f ? 1.f : (u < 0.f ? -1.f : 0.f);
    float p = master[i];
    p = p * (1.f - lr * wd) - lr * sgn;
    master[i] = p;
    m[i] = b2 * mi + (1.f - b2) * g;
    if (shadow) shadow[i] = __float2bfloat16(p);
    if (zero_grad) grad[i] = static_cast<G>(0.f);
  }
}

// ------------------------------------------------------------------------- Muon
// momentum: m = beta*m + g  (heavy ball, as the reference: src/optim/optimizer.zig:253-265)
template <typename G>
__global__ void __launch_bounds__(256)
muon_momentum_kernel(float* __restrict__ m, G* __restrict__ grad, long long n, float beta,
                     const float* __restrict__ gscale_ptr, float gscale, int zero_grad,
                     float* __restrict__ partial) {
  __shared__ float red[33];
  const bool skip = step_skipped(gscale_ptr);
  const float gs = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  float s = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    // a skipped step keeps the momentum (the apply kernel skips too); the sum is still formed
    const float mi = skip ? m[i] : beta * m[i] + ldg_f<G>(grad, i) * gs;
    if (!skip) m[i] = mi;
    s += mi * mi;
    if (zero_grad) grad[i] = static_cast<G>(0.f);
  }
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// y = m / (sqrt(sumsq) + eps)  -> bf16
__global__ void muon_normalize_kernel(const float* __restrict__ m, const float* sumsq,
                                      bf16* __restrict__ y, long long n, float eps) {
  const float inv = 1.f / (sqrtf(*sumsq) + eps);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16(m[i] * inv);
}
// g <- a*I + b*g + c*g2   (n x n, bf16): the polynomial step of Newton-Schulz
__global__ void ns_poly_kernel(bf16* __restrict__ g, const bf16* __restrict__ g2, int n, float a,
                               float b, float c) {
  const long long total = static_cast<long long>(n) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / n), col = static_cast<int>(i - static_cast<long long>(r) * n);
    float val = b * __bfloat162float(g[i]) + (g2 ? c * __bfloat162float(g2[i]) : 0.f);
    if (r == col) val += a;
    g[i] = __float2bfloat16(val);
  }
}
// p = p*(1-lr*wd) - lr*scale*y
__global__ void muon_apply_kernel(float* __restrict__ master, const bf16* __restrict__ y,
                                  bf16* __restrict__ shadow, long long n, float lr, float wd,
                                  float scale, const float* __restrict__ gscale_ptr) {
  if (step_skipped(gscale_ptr)) return;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p = master[i];
    p = p * (1.f - lr * wd) - lr * scale * __bfloat162float(y[i]);
    master[i] = p;
    if (shadow) shadow[i] = __float2bfloat16(p);
  }
}

// float4-vectorised variants for fp32 gradients (the flat main_grad buffer): 16-byte loads
// and stores on every stream, 8-byte stores for the bf16 shadow.
__global__ void __launch_bounds__(256)
adamw_vec4_kernel(float4* __restrict__ master, float4* __restrict__ m, float4* __restrict__ v,
                  float4* __restrict__ grad, uint2* __restrict__ shadow, long long n4, float lr,
                  float b1, float b2, float eps, float wd, float bc1_inv, float bc2_inv,
                  const float* __restrict__ gscale_ptr, float gscale, int zero_grad) {
  if (step_skipped(gscale_ptr)) {
    if (zero_grad) zero_range4(grad, n4);
    return;
  }
  const float gs = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  const float decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 g4 = grad[i], m4 = m[i], v4 = v[i], p4 = master[i];
    float* gp = reinterpret_cast<float*>(&g4);
    float* mp = reinterpret_cast<float*>(&m4);
    float* vp = reinterpret_cast<float*>(&v4);
    float* pp = reinterpret_cast<float*>(&p4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g = gp[j] * gs;
      mp[j] = b1 * mp[j] + (1.f - b1) * g;
      vp[j] = b2 * vp[j] + (1.f - b2) * g * g;
      pp[j] = pp[j] * decay - lr * (mp[j] * bc1_inv) / (sqrtf(vp[j] * bc2_inv) + eps);
    }
    m[i] = m4;
    v[i] = v4;
    master[i] = p4;
    if (shadow) {
      uint2 o;
      bf162* h = reinterpret_cast<bf162*>(&o);
      h[0] = __floats2bfloat162_rn(pp[0], pp[1]);
      h[1] = __floats2bfloat162_rn(pp[2], pp[3]);
      shadow[i] = o;
    }
    if (zero_grad) grad[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

__global__ void __launch_bounds__(256)
lion_vec4_kernel(float4* __restrict__ master, float4* __restrict__ m, float4* __restrict__ grad,
                 uint2* __restrict__ shadow, long long n4, float lr, float b1, float b2, float wd,
                 const float* __restrict__ gscale_ptr, float gscale, int zero_grad) {
  if (step_skipped(gscale_ptr)) {
    if (zero_grad) zero_range4(grad, n4);
    return;
  }
  const float gs = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  const float decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 g4 = grad[i], m4 = m[i], p4 = master[i];
    float* gp = reinterpret_cast<float*>(&g4);
    float* mp = reinterpret_cast<float*>(&m4);
    float* pp = reinterpret_cast<float*>(&p4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g = gp[j] * gs;
      const float u = b1 * mp[j] + (1.f - b1) * g;
      pp[j] = pp[j] * decay - lr * (u > 0.f ? 1.f : (u < 0.f ? -1.f : 0.f));
      mp[j] = b2 * mp[j] + (1.f - b2) * g;
    }
    m[i] = m4;
    master[i] = p4;
    if (shadow) {
      uint2 o;
      bf162* h = reinterpret_cast<bf162*>(&o);
      h[0] = __floats2bfloat162_rn(pp[0], pp[1]);
      h[1] = __floats2bfloat162_rn(pp[2], pp[3]);
      shadow[i] = o;
    }
    if (zero_grad) grad[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

constexpr int OPT_GRID_CAP = 148 * 8;

}  // namespace ceo
using namespace ceo;

extern "C" int ceo_sumsq_blocks(long long n) { return grid_for(n, 256 * 8, CEO_SUMSQ_MAX_BLOCKS); }

extern "C" int ceo_sumsq(const void* x, int is_f32, long long n, float* out, int accumulate,
                         float* partial_scratch, cudaStream_t stream) {
  if (n <= 0) return -5;
  const int nblk = ceo_sumsq_blocks(n);
  if (is_f32)
    sumsq_partial_kernel<float><<<nblk, 256, 0, stream>>>(static_cast<const float*>(x), n,
                                                          partial_scratch);
  else
    sumsq_partial_kernel<bf16><<<nblk, 256, 0, stream>>>(static_cast<const bf16*>(x), n,
                                                         partial_scratch);
  sumsq_final_kernel<<<1, 256, 0, stream>>>(partial_scratch, nblk, out, accumulate);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_clip_scale(const float* sumsq, float max_norm, float* scale_out,
                              float* norm_out, cudaStream_t stream) {
  clip_scale_kernel<<<1, 1, 0, stream>>>(sumsq, max_norm, scale_out, norm_out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_scale(void* x, int is_f32, long long n, const float* scale_ptr, float scale,
                         cudaStream_t stream) {
  if (n <= 0) return -5;
  const int g = grid_for(n, 256 * 4, OPT_GRID_CAP);
  if (is_f32)
    scale_kernel<float><<<g, 256, 0, stream>>>(static_cast<float*>(x), n, scale_ptr, scale);
  else
    scale_kernel<bf16><<<g, 256, 0, stream>>>(static_cast<bf16*>(x), n, scale_ptr, scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_clip_value(float* x, long long n, float clip, cudaStream_t stream) {
  if (n <= 0) return -5;
  clip_value_kernel<<<grid_for(n, 256 * 4, OPT_GRID_CAP), 256, 0, stream>>>(x, n, clip);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_adamw_step(float* master, float* m, float* v, void* grad, int grad_f32,
                              void* shadow_bf16, long long n, float lr, float beta1, float beta2,
                              float eps, float weight_decay, int step, const float* gscale_ptr,
                              float gscale, int zero_grad, cudaStream_t stream) {
  if (n <= 0 || step < 1) return -5;
  const float bc1_inv = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  const float bc2_inv = 1.f / (1.f - powf(beta2, static_cast<float>(step)));
  const int g = grid_for(n, 256 * 4, OPT_GRID_CAP);
  const bool vec = grad_f32 && (n & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(grad)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(shadow_bf16) & 7) == 0;
  if (vec)
    adamw_vec4_kernel<<<grid_for(n >> 2, 256 * 2, OPT_GRID_CAP * 2), 256, 0, stream>>>(
        reinterpret_cast<float4*>(master), reinterpret_cast<float4*>(m),
        reinterpret_cast<float4*>(v), static_cast<float4*>(grad),
        static_cast<uint2*>(shadow_bf16), n >> 2, lr, beta1, beta2, eps, weight_decay, bc1_inv,
        bc2_inv, gscale_ptr, gscale, zero_grad);
  else if (grad_f32)
    adamw_kernel<float><<<g, 256, 0, stream>>>(master, m, v, static_cast<float*>(grad),
                                               static_cast<bf16*>(shadow_bf16), n, lr, beta1,
                                               beta2, eps, weight_decay, bc1_inv, bc2_inv,
                                               gscale_ptr, gscale, zero_grad);
  else
    adamw_kernel<bf16><<<g, 256, 0, stream>>>(master, m, v, static_cast<bf16*>(grad),
                                              static_cast<bf16*>(shadow_bf16), n, lr, beta1, beta2,
                                              eps, weight_decay, bc1_inv, bc2_inv, gscale_ptr,
                                              gscale, zero_grad);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_lion_step(float* master, float* m, void* grad, int grad_f32, void* shadow_bf16,
                             long long n, float lr, float beta1, float beta2, float weight_decay,
                             const float* gscale_ptr, float gscale, int zero_grad,
                             cudaStream_t stream) {
  if (n <= 0) return -5;
  const int g = grid_for(n, 256 * 4, OPT_GRID_CAP);
  const bool vec = grad_f32 && (n & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(grad)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(shadow_bf16) & 7) == 0;
  if (vec)
    lion_vec4_kernel<<<grid_for(n >> 2, 256 * 2, OPT_GRID_CAP * 2), 256, 0, stream>>>(
        reinterpret_cast<float4*>(master), reinterpret_cast<float4*>(m),
        static_cast<float4*>(grad), static_cast<uint2*>(shadow_bf16), n >> 2, lr, beta1, beta2,
        weight_decay, gscale_ptr, gscale, zero_grad);
  else if (grad_f32)
    lion_kernel<float><<<g, 256, 0, stream>>>(master, m, static_cast<float*>(grad),
                                              static_cast<bf16*>(shadow_bf16), n, lr, beta1, beta2,
                                              weight_decay, gscale_ptr, gscale, zero_grad);
  else
    lion_kernel<bf16><<<g, 256, 0, stream>>>(master, m, static_cast<bf16*>(grad),
                                             static_cast<bf16*>(shadow_bf16), n, lr, beta1, beta2,
                                             weight_decay, gscale_ptr, gscale, zero_grad);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_muon_momentum(float* m, void* grad, int grad_f32, long long n, float beta,
                                 const float* gscale_ptr, float gscale, int zero_grad,
                                 float* sumsq_out, float* partial_scratch, cudaStream_t stream) {
  if (n <= 0) return -5;
  const int nblk = ceo_sumsq_blocks(n);
  if (grad_f32)
    muon_momentum_kernel<float><<<nblk, 256, 0, stream>>>(m, static_cast<float*>(grad), n, beta,
                                                          gscale_ptr, gscale, zero_grad,
                                                          partial_scratch);
  else
    muon_momentum_kernel<bf16><<<nblk, 256, 0, stream>>>(m, static_cast<bf16*>(grad), n, beta,
                                                         gscale_ptr, gscale, zero_grad,
                                                         partial_scratch);
  sumsq_final_kernel<<<1, 256, 0, stream>>>(partial_scratch, nblk, sumsq_out, 0);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_muon_normalize(const float* m, const float* sumsq, void* y_bf16, long long n,
                                  float eps, cudaStream_t stream) {
  if (n <= 0) return -5;
  muon_normalize_kernel<<<grid_for(n, 256 * 4, OPT_GRID_CAP), 256, 0, stream>>>(
      m, sumsq, static_cast<bf16*>(y_bf16), n, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_ns_poly(void* g_bf16, const void* g2_bf16, int n, float a, float b, float c,
                           cudaStream_t stream) {
  if (n <= 0) return -5;
  ns_poly_kernel<<<grid_for(static_cast<long long>(n) * n, 256 * 4, OPT_GRID_CAP), 256, 0,
                   stream>>>(static_cast<bf16*>(g_bf16), static_cast<const bf16*>(g2_bf16), n, a,
                             b, c);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_muon_apply(float* master, const void* y_bf16, void* shadow_bf16, long long n,
                              float lr, float weight_decay, float scale,
                              const float* gscale_ptr, cudaStream_t stream) {
  if (n <= 0) return -5;
  muon_apply_kernel<<<grid_for(n, 256 * 4, OPT_GRID_CAP), 256, 0, stream>>>(
      master, static_cast<const bf16*>(y_bf16), static_cast<bf16*>(shadow_bf16), n, lr,
      weight_decay, scale, gscale_ptr);
  return static_cast<int>(cudaGetLastError());
}
