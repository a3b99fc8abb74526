// Chunked EFLA (delta-rule) forward and backward, bf16 operands, fp32 state.
//
//   S_t = (I - a_t k_t k_t^T) S_{t-1} + a_t k_t v_t^T ,   o_t = S_t^T q_t
//
// Per 64-token chunk (C = 64), with G = K K^T, A = strict_tril(diag(a) G),
// X = (I + A)^-1, Tm = X diag(a):
//   W = Tm K,  U = Tm V,  U' = U - W S_in,  O = Q S_in + tril(Q K^T) U',  S_out = S_in + K^T U'
//
// Forward = three kernels:
//   efla_wy_kernel         (parallel over chunks)   G, triangular solve, W, U
//   efla_state_fwd_kernel  (serial over chunks, parallel over (b,h) x value-column slices)
//                          U' and the fp32 state recurrence; snapshots S_in per chunk (bf16)
//   efla_out_kernel        (parallel over chunks)   O
// Backward = three kernels:
//   efla_bwd_local_kernel  (parallel)  dQ and D = tril(Q K^T)^T dO
//   efla_state_bwd_kernel  (serial, reverse)  dU' = D + K dS ;  dS <- dS + Q^T dO - W^T dU'
//   efla_bwd_final_kernel  (parallel)  dK, dV, d(alpha) (re-solves the 64x64 system)
//
// All products run on tensor cores (warp-level bf16 MMA out of shared memory); the only
// backward workspace is one d x d bf16 state per chunk, against one per *token* in the
// reference (kernels/cuda/efla.cu:235-313, 590-601), whose kernels walk the sequence token
// by token with the state in global memory (efla.cu:154-233, 315-454).
#include "common/mma.cuh"
#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

constexpr int CH = 64;    // chunk length
constexpr int GLD = 68;   // leading dimension of the fp32 64x64 Gram tile
constexpr int XLD = 72;   // leading dimension of bf16 64x64 tiles
constexpr int BV = 32;    // value columns per CTA in the serial kernels
constexpr int LDV = BV + 8;

// cp.async a [rows][COLS] bf16 tile (row stride `gstride` elements) into smem with leading dim `sld`
template <int COLS, int NTHR>
__device__ __forceinline__ void tile_load_async(bf16* s, int sld, const bf16* g, long long gstride,
                                                int rows) {
  constexpr int V = COLS / 8;
  for (int i = threadIdx.x; i < rows * V; i += NTHR) {
    const int r = i / V, c = i - r * V;
    cp_async16(s + r * sld + c * 8, g + r * gstride + c * 8);
  }
}

template <int NT>
__device__ __forceinline__ void frag_store_bf16(bf16* base, long long ld, float (*acc)[4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    *reinterpret_cast<bf162*>(base + g * ld + nt * 8 + 2 * tg) =
        __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<bf162*>(base + (g + 8) * ld + nt * 8 + 2 * tg) =
        __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
  }
}

// Column c of X = (I + diag(al) Gs)^-1 for a strictly-lower Gs, by forward substitution in
// registers; thread c of the first 64 threads calls this.  x[i] = 0 for i < c, x[c] = 1.
__device__ __forceinline__ void solve_column(const float* __restrict__ Gs,
                                             const float* __restrict__ al, int c, float* x) {
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int j = 0; j + 3 < i; j += 4) {
      const float4 gq = *reinterpret_cast<const float4*>(Gs + i * GLD + j);
      s0 += gq.x * x[j];
      s1 += gq.y * x[j + 1];
      s2 += gq.z * x[j + 2];
      s3 += gq.w * x[j + 3];
    }
#pragma unroll
    for (int j = (i / 4) * 4; j < i; ++j) s0 += Gs[i * GLD + j] * x[j];
    const float s = (s0 + s1) + (s2 + s3);
    x[i] = (i == c) ? 1.f : (i < c ? 0.f : -al[i] * s);
  }
}

// ============================================================ forward: W, U
template <int D>
__global__ void __launch_bounds__(128)
efla_wy_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v,
               const float* __restrict__ alpha, bf16* __restrict__ w, bf16* __restrict__ u, int T,
               int H, long long ks, long long vs) {
  constexpr int LD = D + 8;
  extern __shared__ __align__(16) uint8_t smem[];
  bf16* Ks = reinterpret_cast<bf16*>(smem);
  bf16* Vs = Ks + CH * LD;
  float* Gs = reinterpret_cast<float*>(Vs + CH * LD);
  bf16* Ts = reinterpret_cast<bf16*>(Gs + CH * GLD);
  float* al = reinterpret_cast<float*>(Ts + CH * XLD);

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const long long tok0 = static_cast<long long>(b) * T + blockIdx.x * CH;
  tile_load_async<D, 128>(Ks, LD, k + tok0 * ks + h * D, ks, CH);
  tile_load_async<D, 128>(Vs, LD, v + tok0 * vs + h * D, vs, CH);
  cp_async_commit();
  if (threadIdx.x < CH) al[threadIdx.x] = alpha[(tok0 + threadIdx.x) * H + h];
  cp_async_wait<0>();
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  {
    float acc[8][4];
    zero_acc<8>(acc);
    warp_gemm<8, D, false, false>(acc, Ks + 16 * warp * LD, LD, Ks, LD);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = 16 * warp + g + (e >> 1) * 8, col = nt * 8 + 2 * tg + (e & 1);
        Gs[row * GLD + col] = col < row ? acc[nt][e] : 0.f;
      }
  }
  __syncthreads();
  if (threadIdx.x < CH) {
    float x[CH];
    const int c = threadIdx.x;
    solve_column(Gs, al, c, x);
    const float ac = al[c];
#pragma unroll
    for (int i = 0; i < CH; ++i) Ts[i * XLD + c] = __float2bfloat16(x[i] * ac);
  }
  __syncthreads();
  const long long orow = (tok0 + 16 * warp) * H + h;  // row index into (B*T*H, D)
  {
    float acc[D / 8][4];
    zero_acc<D / 8>(acc);
    warp_gemm<D / 8, CH, false, true>(acc, Ts + 16 * warp * XLD, XLD, Ks, LD);
    frag_store_bf16<D / 8>(w + orow * D, static_cast<long long>(H) * D, acc);
  }
  {
    float acc[D / 8][4];
    zero_acc<D / 8>(acc);
    warp_gemm<D / 8, CH, false, true>(acc, Ts + 16 * warp * XLD, XLD, Vs, LD);
    frag_store_bf16<D / 8>(u + orow * D, static_cast<long long>(H) * D, acc);
  }
}

// ==================================================== forward: state recurrence
template <int D>
__global__ void __launch_bounds__(128)
efla_state_fwd_kernel(const bf16* __restrict__ k, const bf16* __restrict__ w,
                      const bf16* __restrict__ u, const float* __restrict__ s0,
                      bf16* __restrict__ up, bf16* __restrict__ states,
                      float* __restrict__ s_final, float* __restrict__ p_final, int T, int H,
                      long long ks) {
  constexpr int LD = D + 8, NT = BV / 8, MT = D / 64;
  extern __shared__ __align__(16) uint8_t smem[];
  bf16* Ws = reinterpret_cast<bf16*>(smem);
  bf16* Ks = Ws + CH * LD;
  bf16* Us = Ks + CH * LD;
  bf16* Ss = Us + CH * LDV;
  bf16* Ups = Ss + D * LDV;

  // With p_final the grid has twice the column slices: the second half runs the homogeneous
  // recurrence (U = 0) on the identity, i.e. the span's transfer matrix P = prod (I - K^T W),
  // which context parallelism needs next to the zero-state response.
  const bool ident = blockIdx.x >= D / BV;
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, v0 = (blockIdx.x % (D / BV)) * BV;
  const int n = T / CH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const long long HD = static_cast<long long>(H) * D;

  float sacc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = warp * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + nt * 8 + 2 * tg + (e & 1);
        sacc[mt][nt][e] = ident ? (row == col ? 1.f : 0.f)
                                : (s0 ? s0[(static_cast<long long>(bh) * D + row) * D + col] : 0.f);
      }

  auto issue_wu = [&](int c) {
    const long long tok0 = static_cast<long long>(b) * T + c * CH;
    tile_load_async<D, 128>(Ws, LD, w + tok0 * HD + h * D, HD, CH);
    if (!ident) tile_load_async<BV, 128>(Us, LDV, u + tok0 * HD + h * D + v0, HD, CH);
  };
  auto issue_k = [&](int c) {
    const long long tok0 = static_cast<long long>(b) * T + c * CH;
    tile_load_async<D, 128>(Ks, LD, k + tok0 * ks + h * D, ks, CH);
  };
  issue_wu(0);
  cp_async_commit();
  issue_k(0);
  cp_async_commit();

  for (int c = 0; c < n; ++c) {
    // snapshot of the state entering chunk c: bf16 MMA operand + saved for O and backward
    bf16* sg = states + ((static_cast<long long>(bh) * n + c) * D) * D + v0;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int r0 = warp * 16 * MT + mt * 16;
      frag_store_bf16<NT>(Ss + r0 * LDV, LDV, sacc[mt]);
      if (!ident) frag_store_bf16<NT>(sg + static_cast<long long>(r0) * D, D, sacc[mt]);
    }
    cp_async_wait<1>();
    __syncthreads();
    {
      float acc[NT][4];
      zero_acc<NT>(acc);
      warp_gemm<NT, D, false, true>(acc, Ws + 16 * warp * LD, LD, Ss, LDV);
      const long long tok0 = static_cast<long long>(b) * T + c * CH;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int row = 16 * warp + g + hf * 8, col = nt * 8 + 2 * tg;
          const float2 uu = ident ? make_float2(0.f, 0.f)
                                  : __bfloat1622float2(*reinterpret_cast<const bf162*>(
                                        Us + row * LDV + col));
          const bf162 r = __floats2bfloat162_rn(uu.x - acc[nt][2 * hf], uu.y - acc[nt][2 * hf + 1]);
          *reinterpret_cast<bf162*>(Ups + row * LDV + col) = r;
          if (!ident) *reinterpret_cast<bf162*>(up + (tok0 + row) * HD + h * D + v0 + col) = r;
        }
    }
    __syncthreads();
    if (c + 1 < n) issue_wu(c + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      warp_gemm<NT, CH, true, true>(sacc[mt], Ks + warp * 16 * MT + mt * 16, LD, Ups, LDV);
    __syncthreads();
    if (c + 1 < n) issue_k(c + 1);
    cp_async_commit();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = warp * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + nt * 8 + 2 * tg + (e & 1);
        (ident ? p_final : s_final)[(static_cast<long long>(bh) * D + row) * D + col] =
            sacc[mt][nt][e];
      }
}

// ================================================================ forward: O
template <int D>
__global__ void __launch_bounds__(256)
efla_out_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                const bf16* __restrict__ up, const bf16* __restrict__ states,
                bf16* __restrict__ o, int T, int H, long long qs, long long ks) {
  constexpr int LD = D + 8, NT = D / 16;
  extern __shared__ __align__(16) uint8_t smem[];
  bf16* Qs = reinterpret_cast<bf16*>(smem);
  bf16* Ks = Qs + CH * LD;
  bf16* Ups = Ks + CH * LD;
  bf16* Sb = Ups + CH * LD;
  bf16* Ps = Sb + D * LD;

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, n = T / CH;
  const long long tok0 = static_cast<long long>(b) * T + blockIdx.x * CH;
  const long long HD = static_cast<long long>(H) * D;
  tile_load_async<D, 256>(Qs, LD, q + tok0 * qs + h * D, qs, CH);
  tile_load_async<D, 256>(Ks, LD, k + tok0 * ks + h * D, ks, CH);
  tile_load_async<D, 256>(Ups, LD, up + tok0 * HD + h * D, HD, CH);
  tile_load_async<D, 256>(Sb, LD, states + (static_cast<long long>(bh) * n + blockIdx.x) * D * D, D,
                          D);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, half = warp >> 2;
  {
    float acc[4][4];
    zero_acc<4>(acc);
    warp_gemm<4, D, false, false>(acc, Qs + 16 * r * LD, LD, Ks + 32 * half * LD, LD);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = 32 * half + nt * 8 + 2 * tg;
        const float p0 = col <= row ? acc[nt][2 * hf] : 0.f;
        const float p1 = col + 1 <= row ? acc[nt][2 * hf + 1] : 0.f;
        *reinterpret_cast<bf162*>(Ps + row * XLD + col) = __floats2bfloat162_rn(p0, p1);
      }
  }
  __syncthreads();
  const int c0 = (D / 2) * half;
  float acc[NT][4];
  zero_acc<NT>(acc);
  warp_gemm<NT, D, false, true>(acc, Qs + 16 * r * LD, LD, Sb + c0, LD);
  warp_gemm<NT, CH, false, true>(acc, Ps + 16 * r * XLD, XLD, Ups + c0, LD);
  frag_store_bf16<NT>(o + (tok0 + 16 * r) * HD + h * D + c0, HD, acc);
}

// ============================================== backward: dQ and D = P^T dO
template <int D>
__global__ void __launch_bounds__(256)
efla_bwd_local_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                      const bf16* __restrict__ up, const bf16* __restrict__ states,
                      const bf16* __restrict__ dO, bf16* __restrict__ dq,
                      bf16* __restrict__ dloc, int T, int H, long long qs, long long ks,
                      long long dqs) {
  constexpr int LD = D + 8, NT = D / 16;
  extern __shared__ __align__(16) uint8_t smem[];
  bf16* Qs = reinterpret_cast<bf16*>(smem);
  bf16* Ks = Qs + CH * LD;
  bf16* Ups = Ks + CH * LD;
  bf16* dOs = Ups + CH * LD;
  bf16* Sb = dOs + CH * LD;
  bf16* Ps = Sb + D * LD;
  bf16* dPs = Ps + CH * XLD;

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, n = T / CH;
  const long long tok0 = static_cast<long long>(b) * T + blockIdx.x * CH;
  const long long HD = static_cast<long long>(H) * D;
  tile_load_async<D, 256>(Qs, LD, q + tok0 * qs + h * D, qs, CH);
  tile_load_async<D, 256>(Ks, LD, k + tok0 * ks + h * D, ks, CH);
  tile_load_async<D, 256>(Ups, LD, up + tok0 * HD + h * D, HD, CH);
  tile_load_async<D, 256>(dOs, LD, dO + tok0 * HD + h * D, HD, CH);
  tile_load_async<D, 256>(Sb, LD, states + (static_cast<long long>(bh) * n + blockIdx.x) * D * D, D,
                          D);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, half = warp >> 2;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    float acc[4][4];
    zero_acc<4>(acc);
    if (which == 0)
      warp_gemm<4, D, false, false>(acc, Qs + 16 * r * LD, LD, Ks + 32 * half * LD, LD);
    else
      warp_gemm<4, D, false, false>(acc, dOs + 16 * r * LD, LD, Ups + 32 * half * LD, LD);
    bf16* dst = which == 0 ? Ps : dPs;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = 32 * half + nt * 8 + 2 * tg;
        const float p0 = col <= row ? acc[nt][2 * hf] : 0.f;
        const float p1 = col + 1 <= row ? acc[nt][2 * hf + 1] : 0.f;
        *reinterpret_cast<bf162*>(dst + row * XLD + col) = __floats2bfloat162_rn(p0, p1);
      }
  }
  __syncthreads();
  const int c0 = (D / 2) * half;
  {
    float acc[NT][4];
    zero_acc<NT>(acc);
    warp_gemm<NT, D, false, false>(acc, dOs + 16 * r * LD, LD, Sb + c0 * LD, LD);
    warp_gemm<NT, CH, false, true>(acc, dPs + 16 * r * XLD, XLD, Ks + c0, LD);
    frag_store_bf16<NT>(dq + (tok0 + 16 * r) * dqs + h * D + c0, dqs, acc);
  }
  {
    float acc[NT][4];
    zero_acc<NT>(acc);
    warp_gemm<NT, CH, true, true>(acc, Ps + 16 * r, XLD, dOs + c0, LD);
    frag_store_bf16<NT>(dloc + (tok0 + 16 * r) * HD + h * D + c0, HD, acc);
  }
}

// ================================================ backward: reverse recurrence
template <int D>
__global__ void __launch_bounds__(128)
efla_state_bwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                      const bf16* __restrict__ w, const bf16* __restrict__ dO,
                      const bf16* __restrict__ dloc, const float* __restrict__ ds_final,
                      bf16* __restrict__ dup, bf16* __restrict__ dstates,
                      float* __restrict__ ds0, int T, int H, long long qs, long long ks) {
  constexpr int LD = D + 8, NT = BV / 8, MT = D / 64;
  extern __shared__ __align__(16) uint8_t smem[];
  bf16* Ks = reinterpret_cast<bf16*>(smem);
  bf16* Qs = Ks + CH * LD;
  bf16* Ws = Qs + CH * LD;
  bf16* Dls = Ws + CH * LD;
  bf16* dOs = Dls + CH * LDV;
  bf16* dSs = dOs + CH * LDV;
  bf16* dUps = dSs + D * LDV;

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, v0 = blockIdx.x * BV;
  const int n = T / CH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const long long HD = static_cast<long long>(H) * D;

  float dacc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = warp * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + nt * 8 + 2 * tg + (e & 1);
        dacc[mt][nt][e] =
            ds_final ? ds_final[(static_cast<long long>(bh) * D + row) * D + col] : 0.f;
      }

  auto issue_a = [&](int c) {
    const long long tok0 = static_cast<long long>(b) * T + c * CH;
    tile_load_async<D, 128>(Ks, LD, k + tok0 * ks + h * D, ks, CH);
    tile_load_async<BV, 128>(Dls, LDV, dloc + tok0 * HD + h * D + v0, HD, CH);
  };
  auto issue_b = [&](int c) {
    const long long tok0 = static_cast<long long>(b) * T + c * CH;
    tile_load_async<D, 128>(Qs, LD, q + tok0 * qs + h * D, qs, CH);
    tile_load_async<D, 128>(Ws, LD, w + tok0 * HD + h * D, HD, CH);
    tile_load_async<BV, 128>(dOs, LDV, dO + tok0 * HD + h * D + v0, HD, CH);
  };
  issue_a(n - 1);
  cp_async_commit();
  issue_b(n - 1);
  cp_async_commit();

  for (int c = n - 1; c >= 0; --c) {
    bf16* sg = dstates + ((static_cast<long long>(bh) * n + c) * D) * D + v0;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int r0 = warp * 16 * MT + mt * 16;
      frag_store_bf16<NT>(dSs + r0 * LDV, LDV, dacc[mt]);
      frag_store_bf16<NT>(sg + static_cast<long long>(r0) * D, D, dacc[mt]);
    }
    cp_async_wait<1>();
    __syncthreads();
    {
      float acc[NT][4];
      zero_acc<NT>(acc);
      warp_gemm<NT, D, false, true>(acc, Ks + 16 * warp * LD, LD, dSs, LDV);
      const long long tok0 = static_cast<long long>(b) * T + c * CH;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int row = 16 * warp + g + hf * 8, col = nt * 8 + 2 * tg;
          const float2 dl =
              __bfloat1622float2(*reinterpret_cast<const bf162*>(Dls + row * LDV + col));
          const float a0 = dl.x + acc[nt][2 * hf], a1 = dl.y + acc[nt][2 * hf + 1];
          // the recurrence subtracts W^T dU': keep the negated copy as the MMA operand
          *reinterpret_cast<bf162*>(dUps + row * LDV + col) = __floats2bfloat162_rn(-a0, -a1);
          *reinterpret_cast<bf162*>(dup + (tok0 + row) * HD + h * D + v0 + col) =
              __floats2bfloat162_rn(a0, a1);
        }
    }
    __syncthreads();
    if (c > 0) issue_a(c - 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m0 = warp * 16 * MT + mt * 16;
      warp_gemm<NT, CH, true, true>(dacc[mt], Qs + m0, LD, dOs, LDV);
      warp_gemm<NT, CH, true, true>(dacc[mt], Ws + m0, LD, dUps, LDV);
    }
    __syncthreads();
    if (c > 0) issue_b(c - 1);
    cp_async_commit();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = warp * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + nt * 8 + 2 * tg + (e & 1);
        ds0[(static_cast<long long>(bh) * D + row) * D + col] = dacc[mt][nt][e];
      }
}

// ================================================= backward: dK, dV, d(alpha)
template <int D>
__global__ void __launch_bounds__(256, 1)
efla_bwd_final_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                      const bf16* __restrict__ v, const float* __restrict__ alpha,
                      const bf16* __restrict__ up, const bf16* __restrict__ states,
                      const bf16* __restrict__ dO, const bf16* __restrict__ dup,
                      const bf16* __restrict__ dstates, bf16* __restrict__ dk,
                      bf16* __restrict__ dv, float* __restrict__ dalpha, int T, int H,
                      long long qs, long long ks, long long vs, long long dks, long long dvs) {
  constexpr int LD = D + 8, NT = D / 16;
  extern __shared__ __align__(16) uint8_t smem[];
  bf16* Qs = reinterpret_cast<bf16*>(smem);
  bf16* Ks = Qs + CH * LD;
  bf16* Ups = Ks + CH * LD;
  bf16* dOs = Ups + CH * LD;
  bf16* Zs = dOs + CH * LD;  // holds dU' first, then Z
  bf16* Sb = Zs + CH * LD;   // S_in first, then dS_out
  float* Gs = reinterpret_cast<float*>(Sb + D * LD);
  bf16* Xs = reinterpret_cast<bf16*>(Gs + CH * GLD);
  bf16* dGs = Xs + CH * XLD;
  bf16* dPs = dGs + CH * XLD;
  float* al = reinterpret_cast<float*>(dPs + CH * XLD);
  float* dal = al + CH;

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, n = T / CH;
  const long long tok0 = static_cast<long long>(b) * T + blockIdx.x * CH;
  const long long HD = static_cast<long long>(H) * D;
  const long long soff = (static_cast<long long>(bh) * n + blockIdx.x) * D * D;
  tile_load_async<D, 256>(Qs, LD, q + tok0 * qs + h * D, qs, CH);
  tile_load_async<D, 256>(Ks, LD, k + tok0 * ks + h * D, ks, CH);
  tile_load_async<D, 256>(Ups, LD, up + tok0 * HD + h * D, HD, CH);
  tile_load_async<D, 256>(dOs, LD, dO + tok0 * HD + h * D, HD, CH);
  tile_load_async<D, 256>(Zs, LD, dup + tok0 * HD + h * D, HD, CH);
  tile_load_async<D, 256>(Sb, LD, states + soff, D, D);
  cp_async_commit();
  if (threadIdx.x < CH) {
    al[threadIdx.x] = alpha[(tok0 + threadIdx.x) * H + h];
    dal[threadIdx.x] = 0.f;
  }
  cp_async_wait<0>();
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, half = warp >> 2;
  const int c0 = (D / 2) * half;

  // 1. G = K K^T, strictly lower part, fp32
  {
    float acc[4][4];
    zero_acc<4>(acc);
    warp_gemm<4, D, false, false>(acc, Ks + 16 * r * LD, LD, Ks + 32 * half * LD, LD);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = 16 * r + g + (e >> 1) * 8, col = 32 * half + nt * 8 + 2 * tg + (e & 1);
        Gs[row * GLD + col] = col < row ? acc[nt][e] : 0.f;
      }
  }
  __syncthreads();
  // 2. X = (I + diag(a) G)^-1
  if (threadIdx.x < CH) {
    float x[CH];
    const int c = threadIdx.x;
    solve_column(Gs, al, c, x);
#pragma unroll
    for (int i = 0; i < CH; ++i) Xs[i * XLD + c] = __float2bfloat16(x[i]);
  }
  __syncthreads();
  // 3. Z = X^T dU' ; R = V - K S_in ; dV = a Z ; d(alpha) += Z . R
  float zacc[NT][4];
  zero_acc<NT>(zacc);
  warp_gemm<NT, CH, true, true>(zacc, Xs + 16 * r, XLD, Zs + c0, LD);
  {
    float racc[NT][4];
    zero_acc<NT>(racc);
    warp_gemm<NT, D, false, true>(racc, Ks + 16 * r * LD, LD, Sb + c0, LD);
    float p[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = c0 + nt * 8 + 2 * tg;
        const float2 vv = __bfloat1622float2(
            *reinterpret_cast<const bf162*>(v + (tok0 + row) * vs + h * D + col));
        p[hf] += zacc[nt][2 * hf] * (vv.x - racc[nt][2 * hf]) +
                 zacc[nt][2 * hf + 1] * (vv.y - racc[nt][2 * hf + 1]);
        const float a = al[row];
        *reinterpret_cast<bf162*>(dv + (tok0 + row) * dvs + h * D + col) =
            __floats2bfloat162_rn(a * zacc[nt][2 * hf], a * zacc[nt][2 * hf + 1]);
      }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float s = p[hf];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (tg == 0) atomicAdd(&dal[16 * r + g + hf * 8], s);
    }
  }
  __syncthreads();  // every warp is done reading dU' out of Zs
  frag_store_bf16<NT>(Zs + 16 * r * LD + c0, LD, zacc);
  __syncthreads();
  // 4. dA = -strict_tril(Z U'^T) ; d(alpha) += dA . G ; dG = a dA ;  dP = tril(dO U'^T)
  {
    float acc[4][4];
    zero_acc<4>(acc);
    warp_gemm<4, D, false, false>(acc, Zs + 16 * r * LD, LD, Ups + 32 * half * LD, LD);
    float p[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = 32 * half + nt * 8 + 2 * tg;
        const float a = al[row];
        float d0 = col < row ? -acc[nt][2 * hf] : 0.f;
        float d1 = col + 1 < row ? -acc[nt][2 * hf + 1] : 0.f;
        p[hf] += d0 * Gs[row * GLD + col] + d1 * Gs[row * GLD + col + 1];
        *reinterpret_cast<bf162*>(dGs + row * XLD + col) = __floats2bfloat162_rn(a * d0, a * d1);
      }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float s = p[hf];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (tg == 0) atomicAdd(&dal[16 * r + g + hf * 8], s);
    }
    zero_acc<4>(acc);
    warp_gemm<4, D, false, false>(acc, dOs + 16 * r * LD, LD, Ups + 32 * half * LD, LD);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = 32 * half + nt * 8 + 2 * tg;
        const float p0 = col <= row ? acc[nt][2 * hf] : 0.f;
        const float p1 = col + 1 <= row ? acc[nt][2 * hf + 1] : 0.f;
        *reinterpret_cast<bf162*>(dPs + row * XLD + col) = __floats2bfloat162_rn(p0, p1);
      }
  }
  __syncthreads();
  // 5. dK = -a (Z S_in^T) + dG K + dG^T K + dP^T Q + U' dS_out^T
  float kacc[NT][4];
  zero_acc<NT>(kacc);
  warp_gemm<NT, D, false, false>(kacc, Zs + 16 * r * LD, LD, Sb + c0 * LD, LD);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) kacc[nt][e] *= -al[16 * r + g + (e >> 1) * 8];
  warp_gemm<NT, CH, false, true>(kacc, dGs + 16 * r * XLD, XLD, Ks + c0, LD);
  warp_gemm<NT, CH, true, true>(kacc, dGs + 16 * r, XLD, Ks + c0, LD);
  warp_gemm<NT, CH, true, true>(kacc, dPs + 16 * r, XLD, Qs + c0, LD);
  __syncthreads();  // S_in no longer needed: reuse the buffer for dS_out
  tile_load_async<D, 256>(Sb, LD, dstates + soff, D, D);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  warp_gemm<NT, D, false, false>(kacc, Ups + 16 * r * LD, LD, Sb + c0 * LD, LD);
  frag_store_bf16<NT>(dk + (tok0 + 16 * r) * dks + h * D + c0, dks, kacc);
  if (threadIdx.x < CH) dalpha[(tok0 + threadIdx.x) * H + h] = dal[threadIdx.x];
}

// ===================================================== q/k normalisation + coefficient
// One warp per (token, head).  normalize: qn = q/|q|, kn = k/|k| and lambda = 1, so
// alpha = 1 - exp(-beta); otherwise qn = q, kn = k and alpha = c(beta, |k|^2) with the
// small-lambda series of the reference (kernels/cuda/efla.cu:93-115).
__device__ __forceinline__ float efla_coeff(float beta, float lam) {
  if (lam <= 1e-6f) {
    const float bl = beta * lam;
    return beta * (1.f - bl * (0.5f - bl * (1.f / 6.f - bl * (1.f / 24.f))));
  }
  return -expm1f(-beta * lam) / lam;
}

template <int D>
__global__ void __launch_bounds__(256)
efla_prep_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                     const float* __restrict__ beta, int beta_scalar, bf16* __restrict__ qn,
                     bf16* __restrict__ kn, float* __restrict__ rq, float* __restrict__ rk,
                     float* __restrict__ alpha, long long rows, int H, long long qs, long long ks,
                     int normalize) {
  constexpr int E = D / 32;
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long id = wid; id < rows * H; id += nw) {
    const long long tok = id / H;
    const int h = static_cast<int>(id - tok * H);
    float qv[E], kv[E];
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int e = 0; e < E; e += 2) {
      const float2 a = __bfloat1622float2(
          *reinterpret_cast<const bf162*>(q + tok * qs + h * D + lane * E + e));
      const float2 b = __bfloat1622float2(
          *reinterpret_cast<const bf162*>(k + tok * ks + h * D + lane * E + e));
      qv[e] = a.x; qv[e + 1] = a.y; kv[e] = b.x; kv[e + 1] = b.y;
      sq += a.x * a.x + a.y * a.y;
      sk += b.x * b.x + b.y * b.y;
    }
    sq = warp_reduce_sum(sq);
    sk = warp_reduce_sum(sk);
    const float iq = normalize ? rsqrtf(sq + 1e-6f) : 1.f;
    const float ik = normalize ? rsqrtf(sk + 1e-6f) : 1.f;
#pragma unroll
    for (int e = 0; e < E; e += 2) {
      *reinterpret_cast<bf162*>(qn + id * D + lane * E + e) =
          __floats2bfloat162_rn(qv[e] * iq, qv[e + 1] * iq);
      *reinterpret_cast<bf162*>(kn + id * D + lane * E + e) =
          __floats2bfloat162_rn(kv[e] * ik, kv[e + 1] * ik);
    }
    if (lane == 0) {
      const float b = beta_scalar ? beta[0] : beta[id];
      rq[id] = iq;
      rk[id] = ik;
      alpha[id] = normalize ? -expm1f(-b) : efla_coeff(b, sk);
    }
  }
}

// dq = iq (dqn - qn (qn.dqn)),  same for k (normalize); d(beta) = d(alpha) * exp(-beta*lam);
// without normalisation dk += d(alpha) * dc/dlam * 2k.
template <int D>
__global__ void __launch_bounds__(256)
efla_prep_bwd_kernel(const bf16* __restrict__ dqn, const bf16* __restrict__ dkn,
                     const bf16* __restrict__ qn, const bf16* __restrict__ kn,
                     const float* __restrict__ rq, const float* __restrict__ rk,
                     const float* __restrict__ beta, int beta_scalar,
                     const float* __restrict__ dalpha, bf16* __restrict__ dq,
                     bf16* __restrict__ dk, float* __restrict__ dbeta, long long rows, int H,
                     long long dqs, long long dks, int normalize) {
  constexpr int E = D / 32;
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long id = wid; id < rows * H; id += nw) {
    const long long tok = id / H;
    const int h = static_cast<int>(id - tok * H);
    float qv[E], kv[E], gq[E], gk[E];
    float dq_dot = 0.f, dk_dot = 0.f, sk = 0.f;
#pragma unroll
    for (int e = 0; e < E; e += 2) {
      const long long o = id * D + lane * E + e;
      const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(qn + o));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(kn + o));
      const float2 ga = __bfloat1622float2(*reinterpret_cast<const bf162*>(dqn + o));
      const float2 gb = __bfloat1622float2(*reinterpret_cast<const bf162*>(dkn + o));
      qv[e] = a.x; qv[e + 1] = a.y; kv[e] = b.x; kv[e + 1] = b.y;
      gq[e] = ga.x; gq[e + 1] = ga.y; gk[e] = gb.x; gk[e + 1] = gb.y;
      dq_dot += a.x * ga.x + a.y * ga.y;
      dk_dot += b.x * gb.x + b.y * gb.y;
      sk += b.x * b.x + b.y * b.y;
    }
    dq_dot = warp_reduce_sum(dq_dot);
    dk_dot = warp_reduce_sum(dk_dot);
    sk = warp_reduce_sum(sk);
    const float b = beta_scalar ? beta[0] : beta[id];
    const float da = dalpha[id];
    float kcoef = 0.f, db;
    if (normalize) {
      db = da * __expf(-b);
    } else {
      const float lam = sk;
      const float ex = __expf(-b * lam);
      db = da * ex;
      float dcdl;
      if (lam <= 1e-6f) dcdl = -0.5f * b * b + b * b * b * lam * (1.f / 3.f);
      else dcdl = (b * lam * ex + expm1f(-b * lam)) / (lam * lam);
      kcoef = 2.f * da * dcdl;
    }
    const float iq = rq[id], ik = rk[id];
#pragma unroll
    for (int e = 0; e < E; e += 2) {
      float o0, o1, p0, p1;
      if (normalize) {
        o0 = iq * (gq[e] - qv[e] * dq_dot);
        o1 = iq * (gq[e + 1] - qv[e + 1] * dq_dot);
        p0 = ik * (gk[e] - kv[e] * dk_dot);
        p1 = ik * (gk[e + 1] - kv[e + 1] * dk_dot);
      } else {
        o0 = gq[e]; o1 = gq[e + 1];
        p0 = gk[e] + kcoef * kv[e];
        p1 = gk[e + 1] + kcoef * kv[e + 1];
      }
      *reinterpret_cast<bf162*>(dq + tok * dqs + h * D + lane * E + e) =
          __floats2bfloat162_rn(o0, o1);
      *reinterpret_cast<bf162*>(dk + tok * dks + h * D + lane * E + e) =
          __floats2bfloat162_rn(p0, p1);
    }
    if (lane == 0) dbeta[id] = db;
  }
}

// ------------------------------------------------------------------ host side
template <int D> constexpr int smem_wy() { return 2 * CH * (D + 8) * 2 + CH * GLD * 4 + CH * XLD * 2 + CH * 4; }
template <int D> constexpr int smem_state_fwd() { return 2 * CH * (D + 8) * 2 + CH * LDV * 2 + D * LDV * 2 + CH * LDV * 2; }
template <int D> constexpr int smem_out() { return 3 * CH * (D + 8) * 2 + D * (D + 8) * 2 + CH * XLD * 2; }
template <int D> constexpr int smem_bwd_local() { return 4 * CH * (D + 8) * 2 + D * (D + 8) * 2 + 2 * CH * XLD * 2; }
template <int D> constexpr int smem_state_bwd() { return 3 * CH * (D + 8) * 2 + 2 * CH * LDV * 2 + D * LDV * 2 + CH * LDV * 2; }
template <int D> constexpr int smem_bwd_final() { return 5 * CH * (D + 8) * 2 + D * (D + 8) * 2 + CH * GLD * 4 + 3 * CH * XLD * 2 + 2 * CH * 4; }

template <typename Kern>
static cudaError_t set_smem(Kern kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <int D>
static int efla_fwd_impl(const bf16* q, const bf16* k, const bf16* v, const float* alpha,
                         const float* s0, bf16* w, bf16* up, bf16* states, bf16* o, float* s_final,
                         int B, int T, int H, long long qs, long long ks, long long vs,
                         cudaStream_t st) {
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e;
    if ((e = set_smem(efla_wy_kernel<D>, smem_wy<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_state_fwd_kernel<D>, smem_state_fwd<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_out_kernel<D>, smem_out<D>())) != cudaSuccess) return e;
    cfg = true;
  }
  const int n = T / CH;
  dim3 gpar(n, B * H), gser(D / BV, B * H);
  // U is staged in `o` (same shape, overwritten by the last kernel)
  efla_wy_kernel<D><<<gpar, 128, smem_wy<D>(), st>>>(k, v, alpha, w, o, T, H, ks, vs);
  efla_state_fwd_kernel<D><<<gser, 128, smem_state_fwd<D>(), st>>>(k, w, o, s0, up, states,
                                                                    s_final, nullptr, T, H, ks);
  efla_out_kernel<D><<<gpar, 256, smem_out<D>(), st>>>(q, k, up, states, o, T, H, qs, ks);
  return static_cast<int>(cudaGetLastError());
}

template <int D>
static int efla_bwd_impl(const bf16* q, const bf16* k, const bf16* v, const float* alpha,
                         const bf16* w, const bf16* up, const bf16* states, const bf16* dO,
                         const float* ds_final, bf16* dloc, bf16* dup, bf16* dstates, bf16* dq,
                         bf16* dk, bf16* dv, float* dalpha, float* ds0, int B, int T, int H,
                         long long qs, long long ks, long long vs, long long dqs, long long dks,
                         long long dvs, cudaStream_t st) {
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e;
    if ((e = set_smem(efla_bwd_local_kernel<D>, smem_bwd_local<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_state_bwd_kernel<D>, smem_state_bwd<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_bwd_final_kernel<D>, smem_bwd_final<D>())) != cudaSuccess) return e;
    cfg = true;
  }
  const int n = T / CH;
  dim3 gpar(n, B * H), gser(D / BV, B * H);
  efla_bwd_local_kernel<D><<<gpar, 256, smem_bwd_local<D>(), st>>>(q, k, up, states, dO, dq, dloc,
                                                                    T, H, qs, ks, dqs);
  efla_state_bwd_kernel<D><<<gser, 128, smem_state_bwd<D>(), st>>>(q, k, w, dO, dloc, ds_final, dup,
                                                                    dstates, ds0, T, H, qs, ks);
  efla_bwd_final_kernel<D><<<gpar, 256, smem_bwd_final<D>(), st>>>(
      q, k, v, alpha, up, states, dO, dup, dstates, dk, dv, dalpha, T, H, qs, ks, vs, dks, dvs);
  return static_cast<int>(cudaGetLastError());
}

static bool efla_args_ok(int B, int T, int H, int D, long long qs, long long ks, long long vs) {
  return B > 0 && T > 0 && H > 0 && (T % CH) == 0 && (D == 64 || D == 128) && (qs & 7) == 0 &&
         (ks & 7) == 0 && (vs & 7) == 0;
}

}  // namespace ceo
using namespace ceo;

extern "C" int ceo_efla_fwd(const void* q, const void* k, const void* v, const float* alpha,
                            const float* s0, void* w, void* up, void* states, void* o,
                            float* s_final, int B, int T, int H, int D, long long q_stride,
                            long long k_stride, long long v_stride, int* status,
                            cudaStream_t stream) {
  (void)status;
  if (!efla_args_ok(B, T, H, D, q_stride, k_stride, v_stride)) return -5;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -2;
#define CEO_EFLA_FWD(DD)                                                                        \
  return efla_fwd_impl<DD>(static_cast<const bf16*>(q), static_cast<const bf16*>(k),            \
                           static_cast<const bf16*>(v), alpha, s0, static_cast<bf16*>(w),       \
                           static_cast<bf16*>(up), static_cast<bf16*>(states),                  \
                           static_cast<bf16*>(o), s_final, B, T, H, q_stride, k_stride, v_stride, \
                           stream)
  if (D == 64) CEO_EFLA_FWD(64);
  CEO_EFLA_FWD(128);
#undef CEO_EFLA_FWD
}

extern "C" int ceo_efla_bwd(const void* q, const void* k, const void* v, const float* alpha,
                            const void* w, const void* up, const void* states, const void* dO,
                            const float* ds_final, void* dloc, void* dup, void* dstates, void* dq,
                            void* dk, void* dv, float* dalpha, float* ds0, int B, int T, int H,
                            int D, long long q_stride, long long k_stride, long long v_stride,
                            long long dq_stride, long long dk_stride, long long dv_stride,
                            int* status, cudaStream_t stream) {
  (void)status;
  if (!efla_args_ok(B, T, H, D, q_stride, k_stride, v_stride)) return -5;
  if ((dq_stride | dk_stride | dv_stride) & 1) return -2;
#define CEO_EFLA_BWD(DD)                                                                         \
  return efla_bwd_impl<DD>(static_cast<const bf16*>(q), static_cast<const bf16*>(k),             \
                           static_cast<const bf16*>(v), alpha, static_cast<const bf16*>(w),      \
                           static_cast<const bf16*>(up), static_cast<const bf16*>(states),       \
                           static_cast<const bf16*>(dO), ds_final, static_cast<bf16*>(dloc),     \
                           static_cast<bf16*>(dup), static_cast<bf16*>(dstates),                 \
                           static_cast<bf16*>(dq), static_cast<bf16*>(dk), static_cast<bf16*>(dv), \
                           dalpha, ds0, B, T, H, q_stride, k_stride, v_stride, dq_stride,   \
                           dk_stride, dv_stride, stream)
  if (D == 64) CEO_EFLA_BWD(64);
  CEO_EFLA_BWD(128);
#undef CEO_EFLA_BWD
}

extern "C" int ceo_efla_prep_fwd(const void* q, const void* k, const float* beta, int beta_scalar,
                                 void* qn, void* kn, float* rq, float* rk, float* alpha,
                                 long long rows, int H, int D, long long q_stride,
                                 long long k_stride, int normalize, cudaStream_t stream) {
  if (rows <= 0 || H <= 0 || (D != 64 && D != 128) || (q_stride & 1) || (k_stride & 1)) return -5;
  const int grid = grid_for(rows * H, 8, 148 * 16);
  if (D == 64)
    efla_prep_fwd_kernel<64><<<grid, 256, 0, stream>>>(
        static_cast<const bf16*>(q), static_cast<const bf16*>(k), beta, beta_scalar,
        static_cast<bf16*>(qn), static_cast<bf16*>(kn), rq, rk, alpha, rows, H, q_stride, k_stride,
        normalize);
  else
    efla_prep_fwd_kernel<128><<<grid, 256, 0, stream>>>(
        static_cast<const bf16*>(q), static_cast<const bf16*>(k), beta, beta_scalar,
        static_cast<bf16*>(qn), static_cast<bf16*>(kn), rq, rk, alpha, rows, H, q_stride, k_stride,
        normalize);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_efla_prep_bwd(const void* dqn, const void* dkn, const void* qn, const void* kn,
                                 const float* rq, const float* rk, const float* beta,
                                 int beta_scalar, const float* dalpha, void* dq, void* dk,
                                 float* dbeta, long long rows, int H, int D, long long dq_stride,
                                 long long dk_stride, int normalize, cudaStream_t stream) {
  if (rows <= 0 || H <= 0 || (D != 64 && D != 128) || (dq_stride & 1) || (dk_stride & 1)) return -5;
  const int grid = grid_for(rows * H, 8, 148 * 16);
  if (D == 64)
    efla_prep_bwd_kernel<64><<<grid, 256, 0, stream>>>(
        static_cast<const bf16*>(dqn), static_cast<const bf16*>(dkn), static_cast<const bf16*>(qn),
        static_cast<const bf16*>(kn), rq, rk, beta, beta_scalar, dalpha, static_cast<bf16*>(dq),
        static_cast<bf16*>(dk), dbeta, rows, H, dq_stride, dk_stride, normalize);
  else
    efla_prep_bwd_kernel<128><<<grid, 256, 0, stream>>>(
        static_cast<const bf16*>(dqn), static_cast<const bf16*>(dkn), static_cast<const bf16*>(qn),
        static_cast<const bf16*>(kn), rq, rk, beta, beta_scalar, dalpha, static_cast<bf16*>(dq),
        static_cast<bf16*>(dk), dbeta, rows, H, dq_stride, dk_stride, normalize);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------
// Stage-by-stage access to the six kernels, for callers that interleave them with other work
// (context parallelism runs the state recurrences more than once around a state exchange).
// ptrs: 0 q, 1 k, 2 v, 3 alpha, 4 w, 5 u, 6 up, 7 states, 8 o, 9 s0, 10 s_final, 11 dO,
//       12 dloc, 13 dup, 14 dstates, 15 ds_final, 16 ds0, 17 dq, 18 dk, 19 dv, 20 dalpha,
//       21 p_final (stage 1 only, optional: also computes the span's transfer matrix)
// strides (elements per token): 0 q, 1 k, 2 v, 3 dq, 4 dk, 5 dv
// stage: 0 wy, 1 state_fwd, 2 out, 3 bwd_local, 4 state_bwd, 5 bwd_final
namespace ceo {
template <int D>
static int efla_stage_impl(int stage, void* const* P, const long long* S, int B, int T, int H,
                           cudaStream_t st) {
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e;
    if ((e = set_smem(efla_wy_kernel<D>, smem_wy<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_state_fwd_kernel<D>, smem_state_fwd<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_out_kernel<D>, smem_out<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_bwd_local_kernel<D>, smem_bwd_local<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_state_bwd_kernel<D>, smem_state_bwd<D>())) != cudaSuccess) return e;
    if ((e = set_smem(efla_bwd_final_kernel<D>, smem_bwd_final<D>())) != cudaSuccess) return e;
    cfg = true;
  }
  const int n = T / CH;
  dim3 gpar(n, B * H), gser(D / BV, B * H);
  auto b16 = [&](int i) { return static_cast<bf16*>(P[i]); };
  auto f32 = [&](int i) { return static_cast<float*>(P[i]); };
  switch (stage) {
    case 0:
      efla_wy_kernel<D><<<gpar, 128, smem_wy<D>(), st>>>(b16(1), b16(2), f32(3), b16(4), b16(5), T,
                                                         H, S[1], S[2]);
      break;
    case 1:
      efla_state_fwd_kernel<D><<<dim3(P[21] ? 2 * (D / BV) : D / BV, B * H), 128,
                                 smem_state_fwd<D>(), st>>>(
          b16(1), b16(4), b16(5), f32(9), b16(6), b16(7), f32(10), f32(21), T, H, S[1]);
      break;
    case 2:
      efla_out_kernel<D><<<gpar, 256, smem_out<D>(), st>>>(b16(0), b16(1), b16(6), b16(7), b16(8),
                                                           T, H, S[0], S[1]);
      break;
    case 3:
      efla_bwd_local_kernel<D><<<gpar, 256, smem_bwd_local<D>(), st>>>(
          b16(0), b16(1), b16(6), b16(7), b16(11), b16(17), b16(12), T, H, S[0], S[1], S[3]);
      break;
    case 4:
      efla_state_bwd_kernel<D><<<gser, 128, smem_state_bwd<D>(), st>>>(
          b16(0), b16(1), b16(4), b16(11), b16(12), f32(15), b16(13), b16(14), f32(16), T, H, S[0],
          S[1]);
      break;
    case 5:
      efla_bwd_final_kernel<D><<<gpar, 256, smem_bwd_final<D>(), st>>>(
          b16(0), b16(1), b16(2), f32(3), b16(6), b16(7), b16(11), b16(13), b16(14), b16(18),
          b16(19), f32(20), T, H, S[0], S[1], S[2], S[4], S[5]);
      break;
    default:
      return -5;
  }
  return static_cast<int>(cudaGetLastError());
}
}  // namespace ceo

extern "C" int ceo_efla_stage(int stage, void* const* ptrs, const long long* strides, int B, int T,
                              int H, int D, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0 || (T % ceo::CH) || (D != 64 && D != 128)) return -5;
  for (int i = 0; i < 6; ++i)
    if (strides[i] & 7) return -2;
  return D == 64 ? ceo::efla_stage_impl<64>(stage, ptrs, strides, B, T, H, stream)
                 : ceo::efla_stage_impl<128>(stage, ptrs, strides, B, T, H, stream);
}
