// Fused RMSNorm / LayerNorm forward and backward, bf16 in/out, fp32 math.
//
// Forward can fold the residual add of a pre-norm block (h = x + r; y = norm(h))
// and writes h once.  Backward folds the incoming residual gradient and builds
// the weight gradient from per-CTA fp32 partial sums (a scratch buffer) that a
// second kernel reduces - the reference adds floats into a bf16 buffer through a
// reinterpret cast (kernels/cuda/layernorm.cu:121-124) and has no LayerNorm
// backward at all (layernorm.cu:133-183).
#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;  // 8-element vectors per thread -> D <= 8192

// ------------------------------------------------------------- RMSNorm fwd
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                   const bf16* __restrict__ w, bf16* __restrict__ y, bf16* __restrict__ h_out,
                   float* __restrict__ rstd, int rows, int D, float eps) {
  __shared__ float red[33];
  const int nv = D >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * D);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * D)
                          : nullptr;
    float v[NORM_MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        unpack8(xr[c], v[i]);
        if (rr) {
          float t[8];
          unpack8(rr[c], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += t[j];
          if (h_out) {
            uint4 hv = pack8(v[i]);
            reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * D)[c] = hv;
            unpack8(hv, v[i]);  // normalise exactly what was stored
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = block_reduce_sum(ss, red);
    const float rs = rsqrtf(ss / D + eps);
    if (threadIdx.x == 0 && rstd) rstd[row] = rs;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        float wv[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(w)[c], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rs * wv[j];
        reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * D)[c] = pack8(o);
      }
    }
  }
}

// ------------------------------------------------------------- RMSNorm bwd
// dx = rs * (dy*w) - x * rs^3 * mean(dy*w*x)   (+ dres when given)
// dw partial[blk][c] = sum over this CTA's rows of dy * x * rs
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                   const bf16* __restrict__ w, const float* __restrict__ rstd,
                   const bf16* __restrict__ dres, bf16* __restrict__ dx,
                   float* __restrict__ partial, int rows, int D) {
  __shared__ float red[33];
  const int nv = D >> 3;
  float dwacc[NORM_MAXV][8];
  float wv[NORM_MAXV][8];
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (c < nv) unpack8(reinterpret_cast<const uint4*>(w)[c], wv[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * D;
    const float rs = rstd[row];
    float xv[NORM_MAXV][8], gv[NORM_MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        unpack8(reinterpret_cast<const uint4*>(x + off)[c], xv[i]);
        unpack8(reinterpret_cast<const uint4*>(dy + off)[c], gv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += gv[i][j] * xv[i][j] * rs;
          gv[i][j] *= wv[i][j];
          dot += gv[i][j] * xv[i][j];
        }
      }
    }
    dot = block_reduce_sum(dot, red);
    const float coef = dot * rs * rs * rs / D;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = gv[i][j] * rs - xv[i][j] * coef;
        if (dres) {
          float t[8];
          unpack8(reinterpret_cast<const uint4*>(dres + off)[c], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += t[j];
        }
        reinterpret_cast<uint4*>(dx + off)[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nv) {
      float* pp = partial + static_cast<size_t>(blockIdx.x) * D + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) pp[j] = dwacc[i][j];
    }
  }
}

// Warp-per-row variant for D = NV*256 <= 2048: no block barriers inside the row loop, the
// row stays in registers as packed bf16, and 8 warps per CTA keep 8 rows of loads in flight.
template <int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_warp_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                        const bf16* __restrict__ w, const float* __restrict__ rstd,
                        const bf16* __restrict__ dres, bf16* __restrict__ dx,
                        float* __restrict__ partial, int rows) {
  constexpr int D = NV * 256;
  __shared__ float dws[D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) dws[i] = 0.f;
  __syncthreads();
  float dwacc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const size_t off = static_cast<size_t>(row) * D;
    const uint4* xr = reinterpret_cast<const uint4*>(x + off);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + off);
    uint4 xp[NV], gp[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      xp[i] = xr[lane + 32 * i];
      gp[i] = gr[lane + 32 * i];
    }
    const float rs = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float xv[8], gv[8], ww[8];
      unpack8(xp[i], xv);
      unpack8(gp[i], gv);
      unpack8(wv[lane + 32 * i], ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dwacc[i][j] += gv[j] * xv[j] * rs;
        dot += gv[j] * ww[j] * xv[j];
      }
    }
    dot = warp_reduce_sum(dot);
    const float coef = dot * rs * rs * rs / D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float xv[8], gv[8], ww[8], o[8];
      unpack8(xp[i], xv);
      unpack8(gp[i], gv);
      unpack8(wv[lane + 32 * i], ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = gv[j] * ww[j] * rs - xv[j] * coef;
      if (dres) {
        float t[8];
        unpack8(reinterpret_cast<const uint4*>(dres + off)[lane + 32 * i], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += t[j];
      }
      reinterpret_cast<uint4*>(dx + off)[lane + 32 * i] = pack8(o);
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&dws[(lane + 32 * i) * 8 + j], dwacc[i][j]);
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += NORM_THREADS)
    partial[static_cast<size_t>(blockIdx.x) * D + i] = dws[i];
}

// ---------------------------------------------- RMSNorm, several rows per iteration
// For D = NVT * 2048: thread t owns the 16-byte column chunks t, t + 256, ... of every row and
// the CTA walks R rows per iteration.  One block reduction (one barrier, the scratch is
// double-buffered) then serves R rows, a thread's weight-gradient partials are 8 * NVT
// registers, and R rows of loads are in flight per thread, which is what these kernels need
// to approach the memory bandwidth at two to four CTAs per SM.
template <int NVT, int R>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                        const bf16* __restrict__ w, bf16* __restrict__ y, bf16* __restrict__ h_out,
                        float* __restrict__ rstd, int rows, float eps) {
  constexpr int D = NVT * 2048, NW = NORM_THREADS / 32;
  __shared__ float red[2][NW][R];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4 wp[NVT];
#pragma unroll
  for (int i = 0; i < NVT; ++i) wp[i] = reinterpret_cast<const uint4*>(w)[threadIdx.x + i * NORM_THREADS];
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, it ^= 1) {
    uint4 xv[R][NVT], rv[R][NVT];
    float ss[R];
    // every load of the iteration (x and the residual, R rows) is issued before any is used
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool okr = row0 + r < rows;
      const size_t off = static_cast<size_t>(okr ? row0 + r : row0) * D;
#pragma unroll
      for (int i = 0; i < NVT; ++i) {
        xv[r][i] = reinterpret_cast<const uint4*>(x + off)[threadIdx.x + i * NORM_THREADS];
        if (res) rv[r][i] = reinterpret_cast<const uint4*>(res + off)[threadIdx.x + i * NORM_THREADS];
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool okr = row0 + r < rows;
      const size_t off = static_cast<size_t>(okr ? row0 + r : row0) * D;
      ss[r] = 0.f;
#pragma unroll
      for (int i = 0; i < NVT; ++i) {
        float v[8];
        unpack8(xv[r][i], v);
        if (res) {
          float t[8];
          unpack8(rv[r][i], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += t[j];
          xv[r][i] = pack8(v);  // normalise exactly what is stored as h
          if (h_out && okr)
            reinterpret_cast<uint4*>(h_out + off)[threadIdx.x + i * NORM_THREADS] = xv[r][i];
          unpack8(xv[r][i], v);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss[r] += v[j] * v[j];
      }
      ss[r] = warp_reduce_sum(ss[r]);
      if (lane == 0) red[it][warp][r] = ss[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float tot = 0.f;
#pragma unroll
      for (int wi = 0; wi < NW; ++wi) tot += red[it][wi][r];
      const float rs = rsqrtf(tot / D + eps);
      if (row0 + r < rows) {
        if (threadIdx.x == 0 && rstd) rstd[row0 + r] = rs;
        const size_t off = static_cast<size_t>(row0 + r) * D;
#pragma unroll
        for (int i = 0; i < NVT; ++i) {
          float v[8], wv[8], o[8];
          unpack8(xv[r][i], v);
          unpack8(wp[i], wv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[j] * rs * wv[j];
          reinterpret_cast<uint4*>(y + off)[threadIdx.x + i * NORM_THREADS] = pack8(o);
        }
      }
    }
  }
}

template <int NVT, int R>
__global__ void __launch_bounds__(NORM_THREADS, 2)
rmsnorm_bwd_rows_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                        const bf16* __restrict__ w, const float* __restrict__ rstd,
                        const bf16* __restrict__ dres, bf16* __restrict__ dx,
                        float* __restrict__ partial, int rows) {
  constexpr int D = NVT * 2048, NW = NORM_THREADS / 32;
  __shared__ float red[2][NW][R];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float wv[NVT][8], dwacc[NVT][8];
#pragma unroll
  for (int i = 0; i < NVT; ++i) {
    unpack8(reinterpret_cast<const uint4*>(w)[threadIdx.x + i * NORM_THREADS], wv[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  }
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, it ^= 1) {
    uint4 xv[R][NVT], gv[R][NVT], dv[R][NVT];
    float rs[R];
    // x, dy and the residual stream's gradient of all R rows are requested together: the
    // second round trip a late dres load would add is as long as the first
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool okr = row0 + r < rows;
      const size_t off = static_cast<size_t>(okr ? row0 + r : row0) * D;
      rs[r] = okr ? rstd[row0 + r] : 0.f;
#pragma unroll
      for (int i = 0; i < NVT; ++i) {
        xv[r][i] = reinterpret_cast<const uint4*>(x + off)[threadIdx.x + i * NORM_THREADS];
        gv[r][i] = reinterpret_cast<const uint4*>(dy + off)[threadIdx.x + i * NORM_THREADS];
        if (dres) dv[r][i] = reinterpret_cast<const uint4*>(dres + off)[threadIdx.x + i * NORM_THREADS];
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < NVT; ++i) {
        float xf[8], gf[8];
        unpack8(xv[r][i], xf);
        unpack8(gv[r][i], gf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += gf[j] * xf[j] * rs[r];  // rs = 0 for rows past the end
          dot += gf[j] * wv[i][j] * xf[j];
        }
      }
      dot = warp_reduce_sum(dot);
      if (lane == 0) red[it][warp][r] = dot;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= rows) continue;
      float tot = 0.f;
#pragma unroll
      for (int wi = 0; wi < NW; ++wi) tot += red[it][wi][r];
      const float coef = tot * rs[r] * rs[r] * rs[r] / D;
      const size_t off = static_cast<size_t>(row0 + r) * D;
#pragma unroll
      for (int i = 0; i < NVT; ++i) {
        float xf[8], gf[8], o[8];
        unpack8(xv[r][i], xf);
        unpack8(gv[r][i], gf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = gf[j] * wv[i][j] * rs[r] - xf[j] * coef;
        if (dres) {
          float t[8];
          unpack8(dv[r][i], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += t[j];
        }
        reinterpret_cast<uint4*>(dx + off)[threadIdx.x + i * NORM_THREADS] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NVT; ++i) {
    float* pp = partial + static_cast<size_t>(blockIdx.x) * D + (threadIdx.x + i * NORM_THREADS) * 8;
    *reinterpret_cast<float4*>(pp) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
    *reinterpret_cast<float4*>(pp + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
  }
}

// out[c] (+)= sum_b partial[b][c].  A CTA owns 32 columns; its eight warps take every eighth
// row (128-byte row segments, eight independent load streams per column) and meet in shared
// memory, so the serial chain per thread is nblk / 8 loads instead of nblk.
// Launch with (D + 31) / 32 CTAs of 256 threads.
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblk, int D,
                       int accumulate) {
  __shared__ float part[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s0 = 0.f, s1 = 0.f;
  if (c < D) {
    int b = warp;
    for (; b + 8 < nblk; b += 16) {
      s0 += partial[static_cast<size_t>(b) * D + c];
      s1 += partial[static_cast<size_t>(b + 8) * D + c];
    }
    if (b < nblk) s0 += partial[static_cast<size_t>(b) * D + c];
  }
  part[warp][lane] = s0 + s1;
  __syncthreads();
  if (warp == 0 && c < D) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w][lane];
    out[c] = accumulate ? out[c] + s : s;
  }
}

// ----------------------------------------------------------- LayerNorm fwd
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                     const bf16* __restrict__ b, bf16* __restrict__ y, float* __restrict__ mean,
                     float* __restrict__ rstd, int rows, int D, float eps) {
  __shared__ float red[33];
  const int nv = D >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * D;
    float v[NORM_MAXV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        unpack8(reinterpret_cast<const uint4*>(x + off)[c], v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      }
    }
    const float mu = block_reduce_sum(s, red) / D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[i][j] - mu;
          q += d * d;
        }
      }
    }
    const float rs = rsqrtf(block_reduce_sum(q, red) / D + eps);
    if (threadIdx.x == 0) {
      if (mean) mean[row] = mu;
      if (rstd) rstd[row] = rs;
    }
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        float wv[8], bv[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(w)[c], wv);
        if (b) unpack8(reinterpret_cast<const uint4*>(b)[c], bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mu) * rs * wv[j] + (b ? bv[j] : 0.f);
        reinterpret_cast<uint4*>(y + off)[c] = pack8(o);
      }
    }
  }
}

// ----------------------------------------------------------- LayerNorm bwd
// xhat = (x-mu)*rs; g = dy*w; dx = rs*(g - mean(g) - xhat*mean(g*xhat))
// partial rows: [blk][0:D] = dw, [blk][D:2D] = db
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                     const bf16* __restrict__ w, const float* __restrict__ mean,
                     const float* __restrict__ rstd, bf16* __restrict__ dx,
                     float* __restrict__ partial, int rows, int D) {
  __shared__ float red[33];
  const int nv = D >> 3;
  float dwacc[NORM_MAXV][8], dbacc[NORM_MAXV][8], wv[NORM_MAXV][8];
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = dbacc[i][j] = 0.f;
    if (c < nv) unpack8(reinterpret_cast<const uint4*>(w)[c], wv[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * D;
    const float mu = mean[row], rs = rstd[row];
    float xh[NORM_MAXV][8], g[NORM_MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        unpack8(reinterpret_cast<const uint4*>(x + off)[c], xh[i]);
        unpack8(reinterpret_cast<const uint4*>(dy + off)[c], g[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mu) * rs;
          dwacc[i][j] += g[i][j] * xh[i][j];
          dbacc[i][j] += g[i][j];
          g[i][j] *= wv[i][j];
          s1 += g[i][j];
          s2 += g[i][j] * xh[i][j];
        }
      }
    }
    s1 = block_reduce_sum(s1, red) / D;
    s2 = block_reduce_sum(s2, red) / D;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - s1 - xh[i][j] * s2);
        reinterpret_cast<uint4*>(dx + off)[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nv) {
      float* pw = partial + static_cast<size_t>(blockIdx.x) * 2 * D + c * 8;
      float* pb = pw + D;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        pw[j] = dwacc[i][j];
        pb[j] = dbacc[i][j];
      }
    }
  }
}

static bool norm_shape_ok(int rows, int D) {
  return rows > 0 && D > 0 && (D & 7) == 0 && D <= NORM_THREADS * 8 * NORM_MAXV;
}

}  // namespace ceo

using namespace ceo;

// CTAs of NORM_THREADS threads of `kernel` that the device holds at once.
template <typename K>
static int resident_ctas(K kernel) {
  int dev = 0, sms = 148, occ = 1;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, NORM_THREADS, 0) != cudaSuccess ||
      occ < 1)
    occ = 1;
  return sms * occ;
}

extern "C" int ceo_norm_bwd_blocks(int rows) {
  int g = rows < CEO_NORM_BWD_MAX_BLOCKS ? rows : CEO_NORM_BWD_MAX_BLOCKS;
  return g < 1 ? 1 : g;
}

extern "C" int ceo_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y,
                               void* h_out, float* rstd, int rows, int D, float eps,
                               cudaStream_t stream) {
  if (!norm_shape_ok(rows, D)) return -5;
  if (D == 2048 || D == 4096) {
    constexpr int R = 4;
    int g = (rows + R - 1) / R;
    // one wave: a grid larger than what is resident at once adds a partly filled second wave
    static int cap1 = 0, cap2 = 0;
    if (cap1 == 0) {
      cap1 = resident_ctas(rmsnorm_fwd_rows_kernel<1, R>);
      cap2 = resident_ctas(rmsnorm_fwd_rows_kernel<2, R>);
    }
    const int cap = D == 2048 ? cap1 : cap2;
    if (g > cap) g = cap;
    if (D == 2048)
      rmsnorm_fwd_rows_kernel<1, R><<<g, NORM_THREADS, 0, stream>>>(
          static_cast<const bf16*>(x), static_cast<const bf16*>(residual),
          static_cast<const bf16*>(w), static_cast<bf16*>(y), static_cast<bf16*>(h_out), rstd, rows,
          eps);
    else
      rmsnorm_fwd_rows_kernel<2, R><<<g, NORM_THREADS, 0, stream>>>(
          static_cast<const bf16*>(x), static_cast<const bf16*>(residual),
          static_cast<const bf16*>(w), static_cast<bf16*>(y), static_cast<bf16*>(h_out), rstd, rows,
          eps);
    return static_cast<int>(cudaGetLastError());
  }
  rmsnorm_fwd_kernel<<<rows, NORM_THREADS, 0, stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(residual), static_cast<const bf16*>(w),
      static_cast<bf16*>(y), static_cast<bf16*>(h_out), rstd, rows, D, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                               const void* dres, void* dx, float* dw, int dw_accumulate,
                               float* partial_scratch, int rows, int D, cudaStream_t stream) {
  if (!norm_shape_ok(rows, D)) return -5;
  int nblk = ceo_norm_bwd_blocks(rows);
  const bf16* dyp = static_cast<const bf16*>(dy);
  const bf16* xp = static_cast<const bf16*>(x);
  const bf16* wp = static_cast<const bf16*>(w);
  const bf16* rp = static_cast<const bf16*>(dres);
  bf16* dxp = static_cast<bf16*>(dx);
  if (D == 2048 || D == 4096) {
    const int R = D == 2048 ? 4 : 2;  // rows per iteration: bounded by the register budget
    int g = (rows + R - 1) / R;
    if (g > nblk) g = nblk;  // the partial scratch holds ceo_norm_bwd_blocks(rows) rows
    if (g > 148 * 2) g = 148 * 2;
    nblk = g;
    if (D == 2048)
      rmsnorm_bwd_rows_kernel<1, 4><<<g, NORM_THREADS, 0, stream>>>(dyp, xp, wp, rstd, rp, dxp,
                                                                    partial_scratch, rows);
    else
      rmsnorm_bwd_rows_kernel<2, 2><<<g, NORM_THREADS, 0, stream>>>(dyp, xp, wp, rstd, rp, dxp,
                                                                    partial_scratch, rows);
  } else if ((D & 255) == 0 && D <= 2048) {
    int g = (rows + 7) / 8;
    if (g > 296) g = 296;
    nblk = g;
#define CEO_RMS_BWD(NV)                                                                    \
  case NV:                                                                                 \
    rmsnorm_bwd_warp_kernel<NV><<<g, NORM_THREADS, 0, stream>>>(dyp, xp, wp, rstd, rp, dxp, \
                                                                partial_scratch, rows);    \
    break;
    switch (D / 256) {
      CEO_RMS_BWD(1) CEO_RMS_BWD(2) CEO_RMS_BWD(3) CEO_RMS_BWD(4)
      CEO_RMS_BWD(5) CEO_RMS_BWD(6) CEO_RMS_BWD(7) CEO_RMS_BWD(8)
    }
#undef CEO_RMS_BWD
  } else {
    rmsnorm_bwd_kernel<<<nblk, NORM_THREADS, 0, stream>>>(dyp, xp, wp, rstd, rp, dxp,
                                                          partial_scratch, rows, D);
  }
  reduce_partials_kernel<<<(D + 31) / 32, 256, 0, stream>>>(partial_scratch, dw, nblk, D,
                                                              dw_accumulate);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean,
                                 float* rstd, int rows, int D, float eps, cudaStream_t stream) {
  if (!norm_shape_ok(rows, D)) return -5;
  layernorm_fwd_kernel<<<rows, NORM_THREADS, 0, stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(w), static_cast<const bf16*>(b),
      static_cast<bf16*>(y), mean, rstd, rows, D, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                                 const float* rstd, void* dx, float* dw, float* db,
                                 int accumulate, float* partial_scratch, int rows, int D,
                                 cudaStream_t stream) {
  if (!norm_shape_ok(rows, D)) return -5;
  const int nblk = ceo_norm_bwd_blocks(rows);
  layernorm_bwd_kernel<<<nblk, NORM_THREADS, 0, stream>>>(
      static_cast<const bf16*>(dy), static_cast<const bf16*>(x), static_cast<const bf16*>(w), mean,
      rstd, static_cast<bf16*>(dx), partial_scratch, rows, D);
  // the partial buffer interleaves [dw | db] per CTA: reduce with a row stride of 2*D
  reduce_partials_kernel<<<(2 * D + 31) / 32, 256, 0, stream>>>(partial_scratch,
                                                                  partial_scratch, nblk, 2 * D, 0);
  // partial_scratch[0:2D] now holds the totals (row 0 is summed in place: a CTA reads its
  // columns of row 0 before its barrier and writes them once after it)
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  return ceo_axpby_f32(dw, partial_scratch, D, accumulate ? 1.f : 0.f, 1.f, stream) |
         (db ? ceo_axpby_f32(db, partial_scratch + D, D, accumulate ? 1.f : 0.f, 1.f, stream) : 0);
}

// ------------------------------------------------------------------------------------
// RMSNorm backward for callers that cannot allocate: the partial-sum scratch lives in this
// file-scope device array instead of a caller buffer (see include/ceo_noalloc.h for who
// needs this and for the rules: size limit, first-call set-up, shared contents, races).
#include <stdio.h>

#include "include/ceo_noalloc.h"

static __device__ __align__(256) float g_noalloc_partial[CEO_NORM_BWD_MAX_BLOCKS *
                                                         CEO_NOALLOC_MAX_D];

// In host code `g_noalloc_partial` is only a handle for the runtime, not an address the GPU
// can use, so the device address is looked up once per device and cached here.
static float* g_noalloc_ptr[64] = {nullptr};

extern "C" int ceo_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w,
                                       const float* rstd, const void* dres, void* dx, float* dw,
                                       int dw_accumulate, int rows, int D, cudaStream_t stream) {
  if (D > CEO_NOALLOC_MAX_D) {
    fprintf(stderr,
            "ceo_rmsnorm_bwd_noalloc: D = %d exceeds the built-in scratch (max D = %d); use "
            "ceo_rmsnorm_bwd with a caller-provided scratch buffer\n",
            D, CEO_NOALLOC_MAX_D);
    return CEO_ERR_NOALLOC_TOO_LARGE;
  }
  if (rows <= 0 || D <= 0 || (D & 7)) return -5;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return -5;
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partial);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_noalloc_ptr[dev] = p;
  }
  // Every partial row that the reduction reads is fully written by the first kernel of this
  // same call, so stale contents from an earlier call are never observed.
  return ceo_rmsnorm_bwd(dy, x, w, rstd, dres, dx, dw, dw_accumulate, g_noalloc_ptr[dev], rows,
                         D, stream);
}
