// Fill / cast / copy / reductions / FP8 quantisation with amax tracking.
// Counterparts of the reference's fill_cuda, copy_cuda, cast_cuda, sum_reduce_cuda,
// norm_cuda (kernels/cuda/init.cu:308-444, which reduce through a library device
// reduction and a stream-ordered allocation) and of the header-only
// quantize_fp8_cuda / dequantize_fp8_cuda (kernels/cuda/include/kernels.h:378-395).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

// dtype codes of the C ABI: 0 fp32, 1 fp16, 2 bf16
__device__ __forceinline__ float load_as_f32(const void* p, int dt, long long i) {
  if (dt == 0) return static_cast<const float*>(p)[i];
  if (dt == 1) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, int dt, long long i, float v) {
  if (dt == 0) static_cast<float*>(p)[i] = v;
  else if (dt == 1) static_cast<__half*>(p)[i] = __float2half_rn(v);
  else static_cast<bf16*>(p)[i] = __float2bfloat16(v);
}

#define CEO_GRID_STRIDE(i, n)                                                              \
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; \
       i += static_cast<long long>(gridDim.x) * blockDim.x)

__global__ void fill_kernel(void* x, int dt, long long n, float v) {
  CEO_GRID_STRIDE(i, n) store_from_f32(x, dt, i, v);
}
__global__ void cast_kernel(const void* src, int sdt, void* dst, int ddt, long long n) {
  CEO_GRID_STRIDE(i, n) store_from_f32(dst, ddt, i, load_as_f32(src, sdt, i));
}
__global__ void copy16_kernel(const uint4* src, uint4* dst, long long n16) {
  CEO_GRID_STRIDE(i, n16) dst[i] = src[i];
}
__global__ void copy1_kernel(const uint8_t* src, uint8_t* dst, long long n) {
  CEO_GRID_STRIDE(i, n) dst[i] = src[i];
}
__global__ void axpby_kernel(float* y, const float* x, long long n, float a, float b) {
  CEO_GRID_STRIDE(i, n) y[i] = (a != 0.f ? a * y[i] : 0.f) + b * x[i];
}

// partial[blk] = sum (or sum of squares) of this CTA's strided share, in fp32
__global__ void __launch_bounds__(256)
reduce_partial_kernel(const void* x, int dt, long long n, int squares, float* partial) {
  __shared__ float red[33];
  float s = 0.f;
  CEO_GRID_STRIDE(i, n) {
    const float v = load_as_f32(x, dt, i);
    s += squares ? v * v : v;
  }
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256)
reduce_final_kernel(const float* partial, int nblk, float* out, int take_sqrt) {
  __shared__ float red[33];
  float s = 0.f;
  for (int i = threadIdx.x; i < nblk; i += blockDim.x) s += partial[i];
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) *out = take_sqrt ? sqrtf(s) : s;
}

// ---- FP8: q = sat(x * scale); amax_out = max(amax_out, max|x|) ; kind 0 e4m3, 1 e5m2
__global__ void __launch_bounds__(256)
fp8_quant_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, long long n,
                 const float* __restrict__ scale, float* amax_out, int kind) {
  __shared__ float red[33];
  const float s = *scale;
  const __nv_fp8_interpretation_t fmt = kind == 0 ? __NV_E4M3 : __NV_E5M2;
  float am = 0.f;
  // 8 elements per thread and step (16-byte load, 8-byte store) when the pointers allow it
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) | (reinterpret_cast<uintptr_t>(q) & 7)) == 0;
  const long long n8 = vec ? n >> 3 : 0;
  CEO_GRID_STRIDE(i, n8) {
    const uint4 in = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in);
    uint2 o;
    uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = __bfloat1622float2(h[j]);
      am = fmaxf(am, fmaxf(fabsf(v.x), fabsf(v.y)));
      const __nv_fp8x2_storage_t pr =
          __nv_cvt_float2_to_fp8x2(make_float2(v.x * s, v.y * s), __NV_SATFINITE, fmt);
      ob[2 * j] = static_cast<uint8_t>(pr & 0xff);
      ob[2 * j + 1] = static_cast<uint8_t>(pr >> 8);
    }
    reinterpret_cast<uint2*>(q)[i] = o;
  }
  for (long long i = (n8 << 3) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = __bfloat162float(x[i]);
    am = fmaxf(am, fabsf(v));
    q[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v * s, __NV_SATFINITE, fmt));
  }
  am = block_reduce_max(am, red);
  if (threadIdx.x == 0 && amax_out) atomicMax(reinterpret_cast<int*>(amax_out), __float_as_int(am));
}
// Quantise a (rows, cols) bf16 matrix and write the codes transposed, qt (cols, rows), and
// optionally in place order too, q (rows, cols), from one read of x.  64 x 64 tiles go through
// shared memory; rows and cols are multiples of 16 so every global access is a 16-byte one.
__global__ void __launch_bounds__(256)
fp8_quant_t_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ qt,
                   int rows, int cols, long long ldx, const float* __restrict__ scale,
                   float* amax_out, int kind) {
  __shared__ __align__(16) uint8_t tile[64][80];
  __shared__ float red[33];
  const float s = *scale;
  const __nv_fp8_interpretation_t fmt = kind == 0 ? __NV_E4M3 : __NV_E5M2;
  const int t = threadIdx.x;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  float am = 0.f;
  {
    const int row = r0 + (t >> 2), col = c0 + (t & 3) * 16;
    uint4 codes = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows && col < cols) {
      uint8_t* cb = reinterpret_cast<uint8_t*>(&codes);
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx + col);
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const uint4 in = __ldg(src + h2);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 v = __bfloat1622float2(h[j]);
          am = fmaxf(am, fmaxf(fabsf(v.x), fabsf(v.y)));
          const __nv_fp8x2_storage_t pr =
              __nv_cvt_float2_to_fp8x2(make_float2(v.x * s, v.y * s), __NV_SATFINITE, fmt);
          cb[h2 * 8 + 2 * j] = static_cast<uint8_t>(pr & 0xff);
          cb[h2 * 8 + 2 * j + 1] = static_cast<uint8_t>(pr >> 8);
        }
      }
      if (q) *reinterpret_cast<uint4*>(q + static_cast<long long>(row) * cols + col) = codes;
    }
    *reinterpret_cast<uint4*>(&tile[t >> 2][(t & 3) * 16]) = codes;
  }
  __syncthreads();
  {
    // a warp reads 32 neighbouring columns of the same 16 tile rows: conflict-free
    const int c = t & 63, rseg = (t >> 6) * 16;
    if (c0 + c < cols && r0 + rseg < rows) {
      uint4 o;
      uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
      for (int i = 0; i < 16; ++i) ob[i] = tile[rseg + i][c];
      *reinterpret_cast<uint4*>(qt + static_cast<long long>(c0 + c) * rows + r0 + rseg) = o;
    }
  }
  am = block_reduce_max(am, red);
  if (t == 0 && amax_out) atomicMax(reinterpret_cast<int*>(amax_out), __float_as_int(am));
}
__global__ void fp8_dequant_kernel(const uint8_t* __restrict__ q, bf16* __restrict__ x,
                                   long long n, const float* __restrict__ scale, int kind) {
  const float inv = 1.f / *scale;
  CEO_GRID_STRIDE(i, n) {
    const __half_raw h =
        __nv_cvt_fp8_to_halfraw(q[i], kind == 0 ? __NV_E4M3 : __NV_E5M2);
    x[i] = __float2bfloat16(__half2float(__half(h)) * inv);
  }
}
// Delayed scaling: push amax into a ring history, scale = fp8_max / (max(history) * 2^margin)
__global__ void fp8_update_scale_kernel(float* history, int hist_len, int* cursor, float* amax,
                                        float* scale, float fp8_max, float margin_pow2) {
  history[*cursor % hist_len] = *amax;
  *cursor = (*cursor + 1) % hist_len;
  float m = 0.f;
  for (int i = 0; i < hist_len; ++i) m = fmaxf(m, history[i]);
  *scale = (m > 0.f && isfinite(m)) ? fp8_max / (m * margin_pow2) : 1.f;
  *amax = 0.f;
}

constexpr int GEN_CAP = 148 * 8;

}  // namespace ceo
using namespace ceo;

#ifdef CEO_BOUNDS_CHECK
extern "C" int ceo_bounds_collect_scan(unsigned long long*, int);
extern "C" int ceo_bounds_collect_act(unsigned long long*, int);
extern "C" int ceo_bounds_collect_embed(unsigned long long*, int);
extern "C" int ceo_bounds_collect_gemm(unsigned long long*, int);
extern "C" int ceo_bounds_collect_comm(unsigned long long*, int);
#endif
// Checked build: synchronises the device, then out[0..3] = {violations, site, index, extent} of
// the first recorded violation (sites: 1xx scan / gather / scatter / transpose, 2xx
// activations, 3xx embedding, 4xx GEMM epilogue staging and the reduce-scatter reduction, 5xx
// the fused optimizer step) and returns 0; `reset` clears the records.  Normal build:
// returns -1 (no checks compiled in).
extern "C" int ceo_bounds_status(long long* out, int reset) {
#ifdef CEO_BOUNDS_CHECK
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  int (*const fns[])(unsigned long long*, int) = {ceo_bounds_collect_scan, ceo_bounds_collect_act,
                                                  ceo_bounds_collect_embed, ceo_bounds_collect_gemm,
                                                  ceo_bounds_collect_comm};
  unsigned long long total = 0, first[4] = {0, 0, 0, 0};
  for (auto fn : fns) {
    unsigned long long rec[4];
    const int rc = fn(rec, reset);
    if (rc) return rc;
    if (rec[0] && !first[0]) for (int i = 0; i < 4; ++i) first[i] = rec[i];
    total += rec[0];
  }
  out[0] = static_cast<long long>(total);
  for (int i = 1; i < 4; ++i) out[i] = static_cast<long long>(first[i]);
  return 0;
#else
  (void)out; (void)reset;
  return -1;
#endif
}

extern "C" int ceo_fill(void* x, int dtype, long long n, float value, cudaStream_t stream) {
  if (n <= 0 || dtype < 0 || dtype > 2) return -5;
  fill_kernel<<<grid_for(n, 1024, GEN_CAP), 256, 0, stream>>>(x, dtype, n, value);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
                        cudaStream_t stream) {
  if (n <= 0 || src_dtype < 0 || src_dtype > 2 || dst_dtype < 0 || dst_dtype > 2) return -5;
  cast_kernel<<<grid_for(n, 1024, GEN_CAP), 256, 0, stream>>>(src, src_dtype, dst, dst_dtype, n);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_copy(const void* src, void* dst, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return -5;
  const bool al = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                    static_cast<uintptr_t>(bytes)) & 15) == 0;
  if (al)
    copy16_kernel<<<grid_for(bytes >> 4, 1024, GEN_CAP), 256, 0, stream>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), bytes >> 4);
  else
    copy1_kernel<<<grid_for(bytes, 1024, GEN_CAP), 256, 0, stream>>>(
        static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), bytes);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_axpby_f32(float* y, const float* x, long long n, float a, float b,
                             cudaStream_t stream) {
  if (n <= 0) return -5;
  axpby_kernel<<<grid_for(n, 1024, GEN_CAP), 256, 0, stream>>>(y, x, n, a, b);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_reduce_blocks(long long n) { return grid_for(n, 2048, CEO_SUMSQ_MAX_BLOCKS); }
// mode 0: sum, 1: sum of squares, 2: L2 norm
extern "C" int ceo_reduce(const void* x, int dtype, long long n, int mode, float* out,
                          float* partial_scratch, cudaStream_t stream) {
  if (n <= 0 || dtype < 0 || dtype > 2 || mode < 0 || mode > 2) return -5;
  const int nblk = ceo_reduce_blocks(n);
  reduce_partial_kernel<<<nblk, 256, 0, stream>>>(x, dtype, n, mode != 0, partial_scratch);
  reduce_final_kernel<<<1, 256, 0, stream>>>(partial_scratch, nblk, out, mode == 2);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_fp8_quantize(const void* x_bf16, void* q, long long n, const float* scale,
                                float* amax_out, int kind, cudaStream_t stream) {
  if (n <= 0 || kind < 0 || kind > 1) return -5;
  fp8_quant_kernel<<<grid_for(n, 1024, GEN_CAP), 256, 0, stream>>>(
      static_cast<const bf16*>(x_bf16), static_cast<uint8_t*>(q), n, scale, amax_out, kind);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_fp8_quantize_t(const void* x_bf16, void* q, void* qt, int rows, int cols,
                                  long long ldx, const float* scale, float* amax_out, int kind,
                                  cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || kind < 0 || kind > 1 || !qt) return -5;
  if ((rows & 15) || (cols & 15) || (ldx & 7)) return -5;
  if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(q) |
       reinterpret_cast<uintptr_t>(qt)) & 15)
    return -2;
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  if (grid.y > 65535) return -5;
  fp8_quant_t_kernel<<<grid, 256, 0, stream>>>(static_cast<const bf16*>(x_bf16),
                                               static_cast<uint8_t*>(q),
                                               static_cast<uint8_t*>(qt), rows, cols, ldx, scale,
                                               amax_out, kind);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_fp8_dequantize(const void* q, void* x_bf16, long long n, const float* scale,
                                  int kind, cudaStream_t stream) {
  if (n <= 0 || kind < 0 || kind > 1) return -5;
  fp8_dequant_kernel<<<grid_for(n, 1024, GEN_CAP), 256, 0, stream>>>(
      static_cast<const uint8_t*>(q), static_cast<bf16*>(x_bf16), n, scale, kind);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_fp8_update_scale(float* history, int hist_len, int* cursor, float* amax,
                                    float* scale, float fp8_max, float margin_pow2,
                                    cudaStream_t stream) {
  if (hist_len <= 0) return -5;
  fp8_update_scale_kernel<<<1, 1, 0, stream>>>(history, hist_len, cursor, amax, scale, fp8_max,
                                               margin_pow2);
  return static_cast<int>(cudaGetLastError());
}
