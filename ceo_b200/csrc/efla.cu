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
// Every tile enters shared memory through TMA (tensor maps, 128-byte swizzle, completion on
// mbarriers, requested up front in the order the steps need them); the serial kernels also
// leave through TMA stores issued by a dedicated copy warp.  All products run on tensor cores
// (warp-level bf16 MMA, fragments read conflict-free from the swizzled tiles); the only
// backward workspace is one d x d bf16 state per chunk, against one per *token* in the
// reference (kernels/cuda/efla.cu:235-313, 590-601), whose kernels walk the sequence token
// by token with the state in global memory (efla.cu:154-233, 315-454).
#include "common/mma.cuh"
#include "common/ptx.cuh"
#include "common/tmap.h"
#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

constexpr int CH = 64;    // chunk length
constexpr int GLD = 68;   // leading dimension of the fp32 64x64 Gram tile
constexpr int BV = 64;    // value columns per CTA in the serial kernels
// column groups of warps in efla_bwd_final_kernel (4 x BF_CG warps): 16 warps at 125 registers
// measured 1-3 % slower than 8 warps at 198 (the kernel is not short of warps to hide latency)
constexpr int BF_CG = 2;
#ifndef CEO_BF_PREFETCH
#define CEO_BF_PREFETCH 1
#endif
constexpr int BF_AHEAD = 148;  // CTAs of efla_bwd_final_kernel in flight (one per SM)

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

// ---- tiles moved by TMA ------------------------------------------------------------------
// Token-major tensors (q, k, v, w, u, ...) are mapped as matrices [B*T][H*D] with the token
// stride as leading dimension, the state snapshots as [B*H*n*D][D]; both with 64-column boxes
// and 128-byte swizzle, so a 64 x D token tile lands as D/64 panels of 64 rows x 128 bytes and
// a D x D state as D/64 panels of D rows x 128 bytes (SwzTile in common/mma.cuh).
constexpr int EFLA_WAIT_STATUS = 0x4546;
constexpr int PANEL = CH * 128;  // bytes of a 64-row x 64-column swizzled panel

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}
// Whole tiles come through "panel" maps (the matrix seen as (64, rows, cols / 64), see
// common/tmap.h): one request per tile whatever D is.  x0 = first column, a multiple of 64.
template <int D>
__device__ __forceinline__ void tma_tok_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar,
                                             int x0, int tok0) {
  tma_load_3d(dst, tm, bar, 0, tok0, x0 >> 6);
}
template <int D>
__device__ __forceinline__ void tma_state_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar,
                                               int row0) {
  tma_load_3d(dst, tm, bar, 0, row0, 0);
}
// The same tiles through plain 2-D maps, one request per 64-column panel.
template <int D>
__device__ __forceinline__ void tma_tok_tile_2d(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar,
                                                int x0, int tok0) {
#pragma unroll
  for (int pnl = 0; pnl < D / 64; ++pnl) tma_load_2d(dst + pnl * PANEL, tm, bar, x0 + pnl * 64, tok0);
}
template <int D>
__device__ __forceinline__ void tma_state_tile_2d(uint8_t* dst, const CUtensorMap* tm,
                                                  uint64_t* bar, int row0) {
#pragma unroll
  for (int pnl = 0; pnl < D / 64; ++pnl) tma_load_2d(dst + pnl * D * 128, tm, bar, pnl * 64, row0);
}
// Wait for a tile group that is loaded once per CTA (phase 0).  Bounded: when a wait anywhere
// in the grid has run out, the status word is set and every later wait returns at once.
// The status word lives in global memory: it is read only once the barrier has not flipped
// after a few polls (a tile that has already landed costs no global round trip).
__device__ __forceinline__ void tile_wait(uint64_t* bar, int* status) {
#pragma unroll 1
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, 0)) return;
  if (status && *reinterpret_cast<volatile int*>(status)) return;
  if (!mbar_wait(bar, 0) && status) atomicExch(status, EFLA_WAIT_STATUS);
}
// one row tile: acc[NT][4] += A[m0.., :] * B[.., n0..] over swizzled tiles
template <int NT, int K, bool A_T, bool B_T>
__device__ __forceinline__ void wg(float (*acc)[4], const SwzTile& A, int m0, const SwzTile& B,
                                   int n0) {
  warp_gemm_swz<1, NT, K, A_T, B_T>(reinterpret_cast<float (*)[NT][4]>(acc), A, m0, B, n0);
}

// X = (I + diag(al) G)^-1 for a strictly-lower 64x64 G (fp32, leading dimension GLD), with all
// NTHR threads of the CTA and the working set in shared memory (compact rolled loops: this
// code runs once per CTA, so its size matters more than its instruction count).
//   1. the four 16x16 diagonal blocks by forward substitution (one column per thread of the
//      first two warps: 16 dependent steps);
//   2. inside each 32x32 diagonal block, X21 = -X22 (A21 X11) as two fp32 block products;
//   3. the same at the 64 level with 32x32 blocks.
// Xf receives X on and below the diagonal; everything above the diagonal is scratch.  Xf may
// be Gs itself (G is then destroyed).  Starts and ends on a CTA barrier.
//
// C[i][j0..j0+3] = sign * rs[i] * sum_kk A[i][kk] * B[kk][j0..], for `nblk` independent N x N
// blocks whose operands sit `step` elements apart.
template <int NTHR, int N>
__device__ __forceinline__ void solve_block_prod(const float* A, const float* B, float* C,
                                                 const float* rs, float sign, int nblk,
                                                 int step) {
  constexpr int Q = N / 4;
  for (int o = threadIdx.x; o < nblk * N * Q; o += NTHR) {
    const int blk = o / (N * Q), rem = o - blk * N * Q, i = rem / Q, j0 = (rem - i * Q) * 4;
    const float* a = A + blk * step + i * GLD;
    const float* bb = B + blk * step + j0;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int kk = 0; kk < N; ++kk) {
      const float av = a[kk];
      const float4 bv = *reinterpret_cast<const float4*>(bb + kk * GLD);
      acc.x += av * bv.x; acc.y += av * bv.y; acc.z += av * bv.z; acc.w += av * bv.w;
    }
    const float f = rs ? sign * rs[blk * (step / (GLD + 1)) + i] : sign;
    *reinterpret_cast<float4*>(C + blk * step + i * GLD + j0) =
        make_float4(f * acc.x, f * acc.y, f * acc.z, f * acc.w);
  }
}

template <int NTHR>
__device__ __forceinline__ void solve_blocked(const float* Gs, const float* __restrict__ al,
                                              float* Xf) {
  // 1. diagonal 16x16 blocks: thread (blk, cl) owns column cl of block blk.  Right-looking
  //    substitution with the column in registers: once x_j is known, every later row's partial
  //    sum takes its G[i][j] x_j term, so a step's critical path is one multiply and one FMA
  //    and no load depends on a value computed here.
  if (threadIdx.x < CH) {
    const int blk = threadIdx.x >> 4, cl = threadIdx.x & 15, o = 16 * blk;
    const float* gblk = Gs + o * GLD + o;
    float sum[16], x[16], av[16], gcur[16], gnext[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      sum[i] = 0.f;
      av[i] = al[o + i];
      gcur[i] = i > 0 ? gblk[i * GLD] : 0.f;
      gnext[i] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      // column j + 1 of G is requested before column j is consumed: no load sits on the
      // x_j -> sum -> x_{j+1} chain
#pragma unroll
      for (int i = j + 2; i < 16; ++i) gnext[i] = gblk[i * GLD + j + 1];
      x[j] = (j == cl) ? 1.f : (j < cl ? 0.f : -av[j] * sum[j]);
#pragma unroll
      for (int i = j + 1; i < 16; ++i) sum[i] += gcur[i] * x[j];
#pragma unroll
      for (int i = j + 2; i < 16; ++i) gcur[i] = gnext[i];
    }
    __syncwarp();  // all of G's block has been read before X replaces it (Xf may be Gs)
    float* xcol = Xf + o * GLD + o + cl;
#pragma unroll
    for (int j = 0; j < 16; ++j) xcol[j * GLD] = x[j];
  }
  __syncthreads();
  // 2. 32x32 diagonal blocks (two of them, 32 * (GLD + 1) elements apart)
  constexpr int S32 = 32 * (GLD + 1);
  //    T = a .* (G21 X11) -> upper-right 16x16 of the block (scratch)
  solve_block_prod<NTHR, 16>(Gs + 16 * GLD, Xf, Xf + 16, al + 16, 1.f, 2, S32);
  __syncthreads();
  //    X21 = -X22 T
  solve_block_prod<NTHR, 16>(Xf + 16 * GLD + 16, Xf + 16, Xf + 16 * GLD, nullptr, -1.f, 2, S32);
  __syncthreads();
  //    X11 of the 64 level must be lower triangular: clear the scratch
  for (int o = threadIdx.x; o < 2 * 16 * 16; o += NTHR) {
    const int blk = o >> 8, i = (o >> 4) & 15, j = o & 15;
    Xf[blk * S32 + i * GLD + 16 + j] = 0.f;
  }
  __syncthreads();
  // 3. 64 level: T = a .* (G21 X11) -> upper-right 32x32 (scratch);  X21 = -X22 T
  solve_block_prod<NTHR, 32>(Gs + 32 * GLD, Xf, Xf + 32, al + 32, 1.f, 1, 0);
  __syncthreads();
  solve_block_prod<NTHR, 32>(Xf + 32 * GLD + 32, Xf + 32, Xf + 32 * GLD, nullptr, -1.f, 1, 0);
  __syncthreads();
}

// ============================================================ forward: W, U
template <int D>
__global__ void __launch_bounds__(128)
efla_wy_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
               const float* __restrict__ alpha, bf16* __restrict__ w, bf16* __restrict__ u,
               bf16* __restrict__ xinv, int T, int H, int* status) {
  constexpr int TILE = (D / 64) * PANEL;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* Ks = smem;
  uint8_t* Vs = Ks + TILE;
  uint8_t* Ts = Vs + TILE;
  float* Gs = reinterpret_cast<float*>(Ts + PANEL);
  float* al = Gs + CH * GLD;
  uint64_t* bars = reinterpret_cast<uint64_t*>(al + CH);

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int tok0 = b * T + blockIdx.x * CH;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  // one thread per tile requests it (a TMA instruction is slow to issue; spread them)
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bars[0], TILE);
    tma_tok_tile<D>(Ks, &tm_k, &bars[0], h * D, tok0);
  } else if (threadIdx.x == 32) {
    mbar_arrive_expect_tx(&bars[1], TILE);
    tma_tok_tile<D>(Vs, &tm_v, &bars[1], h * D, tok0);
  }
  // alpha is requested now and parked in shared memory only when the solve needs it, so its
  // global latency hides behind the K tile and the Gram product
  const float my_al =
      threadIdx.x < CH ? alpha[(static_cast<long long>(tok0) + threadIdx.x) * H + h] : 0.f;
  tile_wait(&bars[0], status);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const SwzTile Kt = swz_tile(Ks, CH), Vt = swz_tile(Vs, CH), Tt = swz_tile(Ts, CH);
  {
    float acc[8][4];
    zero_acc<8>(acc);
    wg<8, D, false, false>(acc, Kt, 16 * warp, Kt, 0);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = 16 * warp + g + (e >> 1) * 8, col = nt * 8 + 2 * tg + (e & 1);
        Gs[row * GLD + col] = col < row ? acc[nt][e] : 0.f;
      }
  }
  if (threadIdx.x < CH) al[threadIdx.x] = my_al;
  __syncthreads();
  solve_blocked<128>(Gs, al, Gs);
  // T = X diag(a) feeds the two products below; X itself (bf16) is kept for the backward pass
  bf16* xg = xinv + (static_cast<long long>(bh) * (T / CH) + blockIdx.x) * CH * CH;
#pragma unroll
  for (int it = 0; it < CH * CH / 4 / 128; ++it) {
    const int e = threadIdx.x + it * 128, i = e >> 4, c = (e & 15) * 4;
    const float4 xr = *reinterpret_cast<const float4*>(Gs + i * GLD + c);
    const float4 ar = *reinterpret_cast<const float4*>(al + c);
    const float x0 = c <= i ? xr.x : 0.f, x1 = c + 1 <= i ? xr.y : 0.f;
    const float x2 = c + 2 <= i ? xr.z : 0.f, x3 = c + 3 <= i ? xr.w : 0.f;
    sts_bf162(Tt.at(i, c), x0 * ar.x, x1 * ar.y);
    sts_bf162(Tt.at(i, c + 2), x2 * ar.z, x3 * ar.w);
    uint2 xo;
    *reinterpret_cast<bf162*>(&xo.x) = __floats2bfloat162_rn(x0, x1);
    *reinterpret_cast<bf162*>(&xo.y) = __floats2bfloat162_rn(x2, x3);
    *reinterpret_cast<uint2*>(xg + i * CH + c) = xo;
  }
  __syncthreads();
  const long long orow = (static_cast<long long>(tok0) + 16 * warp) * H + h;  // row of (B*T*H, D)
  {
    float acc[D / 8][4];
    zero_acc<D / 8>(acc);
    wg<D / 8, CH, false, true>(acc, Tt, 16 * warp, Kt, 0);
    frag_store_bf16<D / 8>(w + orow * D, static_cast<long long>(H) * D, acc);
  }
  tile_wait(&bars[1], status);
  {
    float acc[D / 8][4];
    zero_acc<D / 8>(acc);
    wg<D / 8, CH, false, true>(acc, Tt, 16 * warp, Vt, 0);
    frag_store_bf16<D / 8>(u + orow * D, static_cast<long long>(H) * D, acc);
  }
}

// ==================================================== forward: state recurrence
// One CTA per (b,h) and 64-column slice of the value dimension: eight compute warps (warp
// (r, half) owns token rows 16r.. of the chunk products and 32 of the slice's columns) and
// one copy warp.  One thread of the copy warp moves every tile with TMA (tensor-map loads on
// mbarriers into 128-byte-swizzled tiles, tensor-map stores in bulk groups): W and K of a
// chunk are double-buffered and requested two chunks ahead, so the serial chain per chunk is
// W S -> U' -> K^T U' with no global load or store instruction in the compute warps.  Every
// wait is bounded; the first one that runs out sets the status word and a flag that turns all
// later waits into no-ops, so the kernel still runs to its end.
constexpr int SER_THREADS = 288;  // 8 compute warps + 1 copy warp

struct SerialSync {
  uint64_t full[2], empty[2], full_u, ready_s, ready_u, st_free;
  volatile uint32_t dead;
  uint32_t pad;
};

__device__ __forceinline__ void compute_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}
__device__ __forceinline__ void ser_wait(SerialSync* sy, uint64_t* bar, uint32_t parity,
                                         int* status) {
  if (sy->dead) return;
  if (!mbar_wait(bar, parity)) {
    sy->dead = 1;
    if (status) atomicExch(status, EFLA_WAIT_STATUS);
  }
}
__device__ __forceinline__ void serial_sync_init(SerialSync* sy) {
  mbar_init(&sy->full[0], 1);
  mbar_init(&sy->full[1], 1);
  mbar_init(&sy->empty[0], 8);
  mbar_init(&sy->empty[1], 8);
  mbar_init(&sy->full_u, 1);
  mbar_init(&sy->ready_s, 1);
  mbar_init(&sy->ready_u, 1);
  mbar_init(&sy->st_free, 1);
  sy->dead = 0;
  fence_mbar_init();
}

// Token-major tensors (k, w, u, up, ...) are mapped as matrices [B*T][H*D] with the token
// stride as leading dimension; the state snapshots as [B*H*n*D][D].
template <int D>
__global__ void __launch_bounds__(SER_THREADS, 2)
efla_state_fwd_kernel(const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_u,
                      const __grid_constant__ CUtensorMap tm_up,
                      const __grid_constant__ CUtensorMap tm_states,
                      const float* __restrict__ s0, float* __restrict__ s_final,
                      float* __restrict__ p_final, const unsigned char* __restrict__ resets, int T,
                      int H, int* status) {
  constexpr int NT = 4, MT = D / 64, NSL = D / BV, TILE = (D / 64) * PANEL;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* Wb = smem;                 // [2][TILE]
  uint8_t* Kb = Wb + 2 * TILE;        // [2][TILE]
  uint8_t* Us = Kb + 2 * TILE;        // [PANEL]
  uint8_t* Ss = Us + PANEL;           // [D rows x 128 B]
  uint8_t* Ups = Ss + D * 128;        // [PANEL]
  SerialSync* sy = reinterpret_cast<SerialSync*>(Ups + PANEL);

  // With p_final the grid has twice the column slices: the second half runs the homogeneous
  // recurrence (U = 0) on the identity, i.e. the span's transfer matrix P = prod (I - K^T W),
  // which context parallelism needs next to the zero-state response.
  const bool ident = blockIdx.x >= NSL;
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, v0 = (blockIdx.x % NSL) * BV;
  const int n = T / CH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) serial_sync_init(sy);
  __syncthreads();

  if (warp == 8) {
    if (lane != 0) return;
    // ------------------------------------------------------------------ copy thread
    auto load_wk = [&](int c) {
      const int st = c & 1, tok0 = b * T + c * CH;
      mbar_arrive_expect_tx(&sy->full[st], 2 * TILE);
      tma_tok_tile<D>(Wb + st * TILE, &tm_w, &sy->full[st], h * D, tok0);
      tma_tok_tile<D>(Kb + st * TILE, &tm_k, &sy->full[st], h * D, tok0);
    };
    auto load_u = [&](int c) {
      mbar_arrive_expect_tx(&sy->full_u, PANEL);
      tma_load_2d(Us, &tm_u, &sy->full_u, h * D + v0, b * T + c * CH);
    };
    load_wk(0);
    if (!ident) load_u(0);
    if (n > 1) load_wk(1);
    for (int c = 0; c < n; ++c) {
      if (!ident) {
        ser_wait(sy, &sy->ready_s, c & 1, status);
        tma_store_2d(&tm_states, Ss, v0, (bh * n + c) * D);
        ser_wait(sy, &sy->ready_u, c & 1, status);
        tma_store_2d(&tm_up, Ups, h * D + v0, b * T + c * CH);
        bulk_commit();
        if (c + 1 < n) load_u(c + 1);  // the U tile is free once chunk c's U' exists
        bulk_wait_read<0>();
        mbar_arrive(&sy->st_free);
      }
      if (c + 2 < n) {
        ser_wait(sy, &sy->empty[c & 1], (c >> 1) & 1, status);
        load_wk(c + 2);
      }
    }
    bulk_wait<0>();
    return;
  }

  // -------------------------------------------------------------------- compute warps
  const int g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, half = warp >> 2, cw = 32 * half;
  float sacc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + cw + nt * 8 + 2 * tg + (e & 1);
        sacc[mt][nt][e] = ident ? (row == col ? 1.f : 0.f)
                                : (s0 ? s0[(static_cast<long long>(bh) * D + row) * D + col] : 0.f);
      }
  const SwzTile St = swz_tile(Ss, D), Ut = swz_tile(Us, CH), Upt = swz_tile(Ups, CH);
  // resets[b][c] != 0: chunk c starts a new document, the state entering it is zero (the flag
  // of the next chunk is fetched a step ahead, off the serial chain)
  unsigned char rz = resets ? resets[b * n] : 0;

  for (int c = 0; c < n; ++c) {
    const SwzTile Wt = swz_tile(Wb + (c & 1) * TILE, CH), Kt = swz_tile(Kb + (c & 1) * TILE, CH);
    if (rz) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) zero_acc<NT>(sacc[mt]);
    }
    if (resets && c + 1 < n) rz = resets[b * n + c + 1];
    // snapshot of the state entering chunk c: bf16 MMA operand + saved for O and backward
    if (!ident && c > 0) ser_wait(sy, &sy->st_free, (c - 1) & 1, status);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) frag_store_swz<NT>(St, r * 16 * MT + mt * 16, cw, sacc[mt]);
    if (!ident) fence_proxy_async_smem();
    compute_bar_sync();
    if (!ident && threadIdx.x == 0) mbar_arrive(&sy->ready_s);
    ser_wait(sy, &sy->full[c & 1], (c >> 1) & 1, status);
    {
      float acc[1][NT][4];
      zero_acc<NT>(acc[0]);
      warp_gemm_swz<1, NT, D, false, true>(acc, Wt, 16 * r, St, cw);
      if (!ident) ser_wait(sy, &sy->full_u, c & 1, status);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int row = 16 * r + g + hf * 8, col = cw + nt * 8 + 2 * tg;
          const float2 uu = ident ? make_float2(0.f, 0.f) : lds_bf162(Ut.at(row, col));
          sts_bf162(Upt.at(row, col), uu.x - acc[0][nt][2 * hf], uu.y - acc[0][nt][2 * hf + 1]);
        }
    }
    if (!ident) fence_proxy_async_smem();
    compute_bar_sync();
    if (!ident && threadIdx.x == 0) mbar_arrive(&sy->ready_u);
    warp_gemm_swz<MT, NT, CH, true, true>(sacc, Kt, r * 16 * MT, Upt, cw);
    __syncwarp();
    if (lane == 0) mbar_arrive(&sy->empty[c & 1]);
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + cw + nt * 8 + 2 * tg + (e & 1);
        (ident ? p_final : s_final)[(static_cast<long long>(bh) * D + row) * D + col] =
            sacc[mt][nt][e];
      }
}

// ================================================================ forward: O
template <int D>
__global__ void __launch_bounds__(256, 2)
efla_out_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_up,
                const __grid_constant__ CUtensorMap tm_states, bf16* __restrict__ o, int T, int H,
                int* status) {
  constexpr int NT = D / 16, TILE = (D / 64) * PANEL, STILE = (D / 64) * D * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + TILE;
  uint8_t* Ups = Ks + TILE;
  uint8_t* Sb = Ups + TILE;
  uint8_t* Ps = Sb + STILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + PANEL);

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, n = T / CH;
  const int tok0 = b * T + blockIdx.x * CH;
  const long long HD = static_cast<long long>(H) * D;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 2);
    mbar_init(&bars[1], 2);
    fence_mbar_init();
  }
  __syncthreads();
  // one thread per tile requests it (a TMA instruction is slow to issue; spread them)
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bars[0], TILE);
    tma_tok_tile<D>(Qs, &tm_q, &bars[0], h * D, tok0);
  } else if (threadIdx.x == 32) {
    mbar_arrive_expect_tx(&bars[0], TILE);
    tma_tok_tile<D>(Ks, &tm_k, &bars[0], h * D, tok0);
  } else if (threadIdx.x == 64) {
    mbar_arrive_expect_tx(&bars[1], TILE);
    tma_tok_tile<D>(Ups, &tm_up, &bars[1], h * D, tok0);
  } else if (threadIdx.x == 96) {
    mbar_arrive_expect_tx(&bars[1], STILE);
    tma_state_tile<D>(Sb, &tm_states, &bars[1], (bh * n + blockIdx.x) * D);
  }
  tile_wait(&bars[0], status);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, half = warp >> 2;
  const SwzTile Qt = swz_tile(Qs, CH), Kt = swz_tile(Ks, CH), Upt = swz_tile(Ups, CH),
                St = swz_tile(Sb, D), Pt = swz_tile(Ps, CH);
  {
    float acc[4][4];
    zero_acc<4>(acc);
    wg<4, D, false, false>(acc, Qt, 16 * r, Kt, 32 * half);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = 32 * half + nt * 8 + 2 * tg;
        sts_bf162(Pt.at(row, col), col <= row ? acc[nt][2 * hf] : 0.f,
                  col + 1 <= row ? acc[nt][2 * hf + 1] : 0.f);
      }
  }
  tile_wait(&bars[1], status);
  __syncthreads();
  const int c0 = (D / 2) * half;
  float acc[NT][4];
  zero_acc<NT>(acc);
  wg<NT, D, false, true>(acc, Qt, 16 * r, St, c0);
  wg<NT, CH, false, true>(acc, Pt, 16 * r, Upt, c0);
  frag_store_bf16<NT>(o + (static_cast<long long>(tok0) + 16 * r) * HD + h * D + c0, HD, acc);
}

// ===================================================== forward: O on tcgen05 (D = 128)
// Two adjacent chunks per CTA, so that every product has a 128-row operand for the 5th-gen
// tensor core (accumulators in TMEM, operands read by the MMA unit straight from the TMA
// tiles):
//   P   (128 x 128) = [Q1;Q2] [K1;K2]^T        only the two 64x64 diagonal blocks are used
//   O_i^T (128 x 64) = S_i^T Q_i^T + U'_i^T P_i^T     (M = value dim, N = the chunk's tokens)
// The transposed form makes the value dimension the 128-lane M of the MMA: S_i and U'_i are
// read as M-major operands exactly as TMA lays them out, Q_i and the masked P_i as K-major
// ones.  128 threads = the 128 TMEM lanes; thread 0 also issues the TMA requests and MMAs.
constexpr int OUT_TC_THREADS = 128;
constexpr int OUT_TC_SMEM = 2 * 32768 /*Q,K*/ + 2 * 16384 /*U'*/ + 2 * 32768 /*S*/ + 2 * PANEL /*P*/ +
                            64 /*barriers + TMEM slot*/ + 1024;

__global__ void __launch_bounds__(OUT_TC_THREADS, 1)
efla_out_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_up,
                   const __grid_constant__ CUtensorMap tm_states, bf16* __restrict__ o, int T,
                   int H, int* status) {
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* Qs = smem;                 // 128 tokens x 128: two panels of 128 rows x 128 B
  uint8_t* Ks = Qs + 32768;
  uint8_t* Ups = Ks + 32768;          // per chunk: 64 tokens x 128 (two 64-row panels)
  uint8_t* Sb = Ups + 2 * 16384;      // per chunk: 128 x 128 (two 128-row panels)
  uint8_t* Ps = Sb + 2 * 32768;       // per chunk: 64 x 64, one panel
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + 2 * PANEL);  // 0,1: TMA; 2,3,4: MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, n = T / CH;
  const int c0 = 2 * blockIdx.x;                 // first chunk of the pair
  const int tok0 = b * T + c0 * CH;
  const long long HD = static_cast<long long>(H) * D;
  const int warp = threadIdx.x >> 5;
  // bounded wait that gives up at once when any wait of the grid has already run out
  auto waitb = [&](uint64_t* bar) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, 0)) return true;
    if (status && *reinterpret_cast<volatile int*>(status)) return false;
    return mbar_wait(bar, 0);
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bars[0], 2 * 32768);
#pragma unroll
    for (int pnl = 0; pnl < 2; ++pnl)
#pragma unroll
      for (int rh = 0; rh < 2; ++rh) {
        tma_load_2d(Qs + pnl * 16384 + rh * 8192, &tm_q, &bars[0], h * D + pnl * 64, tok0 + rh * 64);
        tma_load_2d(Ks + pnl * 16384 + rh * 8192, &tm_k, &bars[0], h * D + pnl * 64, tok0 + rh * 64);
      }
    mbar_arrive_expect_tx(&bars[1], 2 * 16384 + 2 * 32768);
#pragma unroll
    for (int ci = 0; ci < 2; ++ci) {
      tma_tok_tile_2d<D>(Ups + ci * 16384, &tm_up, &bars[1], h * D, tok0 + ci * CH);
      tma_state_tile_2d<D>(Sb + ci * 32768, &tm_states, &bars[1], (bh * n + c0 + ci) * D);
    }
    // P = Q K^T for the pair
    if (!waitb(&bars[0])) ok = false;
    tc_fence_after();
    if (ok) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
      const uint32_t qa = smem_u32(Qs), ka = smem_u32(Ks);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        umma_f16(tmem, umma_smem_desc(qa + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                 umma_smem_desc(ka + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), idesc, k ? 1u : 0u);
      umma_commit(&bars[2]);
    }
    // O_i^T = S_i^T Q_i^T (columns 128 + 64 i of TMEM)
    if (ok && !waitb(&bars[1])) ok = false;
    tc_fence_after();
    if (ok) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 1, 0);
      const uint32_t qa = smem_u32(Qs);
#pragma unroll
      for (int ci = 0; ci < 2; ++ci) {
        const uint32_t sa = smem_u32(Sb + ci * 32768);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16(tmem + 128 + 64 * ci, umma_smem_desc(sa + k * 2048, 16384, 1024),
                   umma_smem_desc(qa + (k >> 2) * 16384 + ci * 8192 + (k & 3) * 32, 16, 1024), idesc,
                   k ? 1u : 0u);
      }
      umma_commit(&bars[3]);
    }
    if (!ok && status) atomicExch(status, EFLA_WAIT_STATUS);
  }
  __syncwarp();

  // masked P -> bf16 K-major panels (thread = one token row of the pair)
  {
    const int ci = warp >> 1, rl = threadIdx.x & 63;
    const bool got = waitb(&bars[2]);
    tc_fence_after();
    uint8_t* prow = Ps + ci * PANEL + rl * 128;
#pragma unroll
    for (int hc = 0; hc < 2; ++hc) {
      uint32_t v[32];
      tmem_ld_32x32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + 64 * ci + hc * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 o4;
        bf162* oh = reinterpret_cast<bf162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = hc * 32 + q4 * 8 + 2 * j;
          oh[j] = __floats2bfloat162_rn(got && col <= rl ? __uint_as_float(v[q4 * 8 + 2 * j]) : 0.f,
                                        got && col + 1 <= rl ? __uint_as_float(v[q4 * 8 + 2 * j + 1])
                                                             : 0.f);
        }
        const int chunk = hc * 4 + q4;
        *reinterpret_cast<uint4*>(prow + ((chunk ^ (rl & 7)) << 4)) = o4;
      }
    }
  }
  fence_proxy_async_smem();  // the MMA unit reads P through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (threadIdx.x == 0) {
    // O_i^T += U'_i^T P_i^T
    bool ok2 = waitb(&bars[3]);
    tc_fence_after();
    if (ok2) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 1, 0);
#pragma unroll
      for (int ci = 0; ci < 2; ++ci) {
        const uint32_t ua = smem_u32(Ups + ci * 16384), pa = smem_u32(Ps + ci * PANEL);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem + 128 + 64 * ci, umma_smem_desc(ua + k * 2048, 8192, 1024),
                   umma_smem_desc(pa + k * 32, 16, 1024), idesc, 1u);
      }
      umma_commit(&bars[4]);
    } else if (status) {
      atomicExch(status, EFLA_WAIT_STATUS);
    }
  }
  __syncwarp();

  // O^T (lane = value index) -> staging [token][value] in the dead Q tile -> coalesced stores
  {
    const bool got = waitb(&bars[4]);
    tc_fence_after();
    bf16* stage = reinterpret_cast<bf16*>(Qs);
#pragma unroll 1
    for (int cc = 0; cc < 4; ++cc) {  // 4 x 32 tokens
      uint32_t v[32];
      tmem_ld_32x32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + 128 + cc * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        stage[(cc * 32 + j) * D + threadIdx.x] = __float2bfloat16(got ? __uint_as_float(v[j]) : 0.f);
    }
  }
  tc_fence_before();
  __syncthreads();
  {
    const uint4* stage = reinterpret_cast<const uint4*>(Qs);
    for (int i = threadIdx.x; i < 128 * 16; i += OUT_TC_THREADS) {
      const int row = i >> 4, cu = i & 15;
      *reinterpret_cast<uint4*>(o + (static_cast<long long>(tok0) + row) * HD + h * D + cu * 8) =
          stage[i];
    }
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ============================================== backward: dQ and D = P^T dO
template <int D>
__global__ void __launch_bounds__(256, 2)
efla_bwd_local_kernel(const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_up,
                      const __grid_constant__ CUtensorMap tm_dO,
                      const __grid_constant__ CUtensorMap tm_states, bf16* __restrict__ dq,
                      bf16* __restrict__ dloc, int T, int H, long long dqs, int* status) {
  constexpr int NT = D / 16, TILE = (D / 64) * PANEL, STILE = (D / 64) * D * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + TILE;
  uint8_t* Ups = Ks + TILE;
  uint8_t* dOs = Ups + TILE;
  uint8_t* Sb = dOs + TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(Sb + STILE);
  uint8_t* Ps = Qs;    // P and dP replace Q and U' once both products are in registers
  uint8_t* dPs = Ups;

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, n = T / CH;
  const int tok0 = b * T + blockIdx.x * CH;
  const long long HD = static_cast<long long>(H) * D;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 4);
    mbar_init(&bars[1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  // one thread per tile requests it (a TMA instruction is slow to issue; spread them)
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bars[0], TILE);
    tma_tok_tile<D>(Qs, &tm_q, &bars[0], h * D, tok0);
  } else if (threadIdx.x == 32) {
    mbar_arrive_expect_tx(&bars[0], TILE);
    tma_tok_tile<D>(Ks, &tm_k, &bars[0], h * D, tok0);
  } else if (threadIdx.x == 64) {
    mbar_arrive_expect_tx(&bars[0], TILE);
    tma_tok_tile<D>(Ups, &tm_up, &bars[0], h * D, tok0);
  } else if (threadIdx.x == 96) {
    mbar_arrive_expect_tx(&bars[0], TILE);
    tma_tok_tile<D>(dOs, &tm_dO, &bars[0], h * D, tok0);
  } else if (threadIdx.x == 128) {
    mbar_arrive_expect_tx(&bars[1], STILE);
    tma_state_tile<D>(Sb, &tm_states, &bars[1], (bh * n + blockIdx.x) * D);
  }
  tile_wait(&bars[0], status);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, half = warp >> 2;
  const SwzTile Qt = swz_tile(Qs, CH), Kt = swz_tile(Ks, CH), Upt = swz_tile(Ups, CH),
                dOt = swz_tile(dOs, CH), St = swz_tile(Sb, D), Pt = swz_tile(Ps, CH),
                dPt = swz_tile(dPs, CH);
  {
    float accp[4][4], accd[4][4];
    zero_acc<4>(accp);
    zero_acc<4>(accd);
    wg<4, D, false, false>(accp, Qt, 16 * r, Kt, 32 * half);
    wg<4, D, false, false>(accd, dOt, 16 * r, Upt, 32 * half);
    __syncthreads();  // all warps are done with Q and U'
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = 32 * half + nt * 8 + 2 * tg;
        const bool k0 = col <= row, k1 = col + 1 <= row;
        sts_bf162(Pt.at(row, col), k0 ? accp[nt][2 * hf] : 0.f, k1 ? accp[nt][2 * hf + 1] : 0.f);
        sts_bf162(dPt.at(row, col), k0 ? accd[nt][2 * hf] : 0.f, k1 ? accd[nt][2 * hf + 1] : 0.f);
      }
  }
  tile_wait(&bars[1], status);
  __syncthreads();
  const int c0 = (D / 2) * half;
  {
    float acc[NT][4];
    zero_acc<NT>(acc);
    wg<NT, D, false, false>(acc, dOt, 16 * r, St, c0);
    wg<NT, CH, false, true>(acc, dPt, 16 * r, Kt, c0);
    frag_store_bf16<NT>(dq + (static_cast<long long>(tok0) + 16 * r) * dqs + h * D + c0, dqs, acc);
  }
  {
    float acc[NT][4];
    zero_acc<NT>(acc);
    wg<NT, CH, true, true>(acc, Pt, 16 * r, dOt, c0);
    frag_store_bf16<NT>(dloc + (static_cast<long long>(tok0) + 16 * r) * HD + h * D + c0, HD, acc);
  }
}

// ================================================ backward: reverse recurrence
// Same structure as the forward recurrence (eight compute warps + one copy warp), walking the
// chunks from the last to the first.  `dup` receives the NEGATED dU' (the form the recurrence
// consumes as an MMA operand); efla_bwd_final_kernel flips the sign back.
template <int D>
__global__ void __launch_bounds__(SER_THREADS, 1)
efla_state_bwd_kernel(const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_dO,
                      const __grid_constant__ CUtensorMap tm_dloc,
                      const __grid_constant__ CUtensorMap tm_dup,
                      const __grid_constant__ CUtensorMap tm_dstates,
                      const float* __restrict__ ds_final, float* __restrict__ ds0,
                      const unsigned char* __restrict__ resets, int T, int H, int* status) {
  constexpr int NT = 4, MT = D / 64, TILE = (D / 64) * PANEL;
  constexpr int STAGE = 3 * TILE + 2 * PANEL;  // K | Q | W | Dl | dO
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* dSs = smem + 2 * STAGE;   // [D rows x 128 B]
  uint8_t* dUps = dSs + D * 128;     // [PANEL]
  SerialSync* sy = reinterpret_cast<SerialSync*>(dUps + PANEL);

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, v0 = blockIdx.x * BV;
  const int n = T / CH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) serial_sync_init(sy);
  __syncthreads();

  if (warp == 8) {
    if (lane != 0) return;
    // step i = n-1-c processes chunk c; its tiles live in stage i & 1
    auto load = [&](int i) {
      const int tok0 = b * T + (n - 1 - i) * CH;
      uint8_t* st = smem + (i & 1) * STAGE;
      uint64_t* bar = &sy->full[i & 1];
      mbar_arrive_expect_tx(bar, STAGE);
      tma_tok_tile<D>(st, &tm_k, bar, h * D, tok0);
      tma_tok_tile<D>(st + TILE, &tm_q, bar, h * D, tok0);
      tma_tok_tile<D>(st + 2 * TILE, &tm_w, bar, h * D, tok0);
      tma_load_2d(st + 3 * TILE, &tm_dloc, bar, h * D + v0, tok0);
      tma_load_2d(st + 3 * TILE + PANEL, &tm_dO, bar, h * D + v0, tok0);
    };
    load(0);
    if (n > 1) load(1);
    for (int i = 0; i < n; ++i) {
      const int c = n - 1 - i;
      ser_wait(sy, &sy->ready_s, i & 1, status);
      tma_store_2d(&tm_dstates, dSs, v0, (bh * n + c) * D);
      ser_wait(sy, &sy->ready_u, i & 1, status);
      tma_store_2d(&tm_dup, dUps, h * D + v0, b * T + c * CH);
      bulk_commit();
      bulk_wait_read<0>();
      mbar_arrive(&sy->st_free);
      if (i + 2 < n) {
        ser_wait(sy, &sy->empty[i & 1], (i >> 1) & 1, status);
        load(i + 2);
      }
    }
    bulk_wait<0>();
    return;
  }

  const int g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, half = warp >> 2, cw = 32 * half;
  float dacc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + cw + nt * 8 + 2 * tg + (e & 1);
        dacc[mt][nt][e] =
            ds_final ? ds_final[(static_cast<long long>(bh) * D + row) * D + col] : 0.f;
      }
  const SwzTile dSt = swz_tile(dSs, D), dUpt = swz_tile(dUps, CH);
  // a chunk that starts a new document passes no gradient to the chunk before it
  unsigned char rz = resets ? resets[b * n + n - 1] : 0;

  for (int i = 0; i < n; ++i) {
    uint8_t* st = smem + (i & 1) * STAGE;
    const SwzTile Kt = swz_tile(st, CH), Qt = swz_tile(st + TILE, CH),
                  Wt = swz_tile(st + 2 * TILE, CH), Dlt = swz_tile(st + 3 * TILE, CH),
                  dOt = swz_tile(st + 3 * TILE + PANEL, CH);
    if (i > 0) ser_wait(sy, &sy->st_free, (i - 1) & 1, status);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) frag_store_swz<NT>(dSt, r * 16 * MT + mt * 16, cw, dacc[mt]);
    fence_proxy_async_smem();
    compute_bar_sync();
    if (threadIdx.x == 0) mbar_arrive(&sy->ready_s);
    ser_wait(sy, &sy->full[i & 1], (i >> 1) & 1, status);
    {
      float acc[1][NT][4];
      zero_acc<NT>(acc[0]);
      warp_gemm_swz_2chain<NT, D, false, true>(acc[0], Kt, 16 * r, dSt, cw);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int row = 16 * r + g + hf * 8, col = cw + nt * 8 + 2 * tg;
          const float2 dl = lds_bf162(Dlt.at(row, col));
          // the recurrence subtracts W^T dU': the negated copy is the MMA operand
          sts_bf162(dUpt.at(row, col), -(dl.x + acc[0][nt][2 * hf]),
                    -(dl.y + acc[0][nt][2 * hf + 1]));
        }
    }
    fence_proxy_async_smem();
    compute_bar_sync();
    if (threadIdx.x == 0) mbar_arrive(&sy->ready_u);
    warp_gemm_swz<MT, NT, CH, true, true>(dacc, Qt, r * 16 * MT, dOt, cw);
    warp_gemm_swz<MT, NT, CH, true, true>(dacc, Wt, r * 16 * MT, dUpt, cw);
    __syncwarp();
    if (lane == 0) mbar_arrive(&sy->empty[i & 1]);
    if (rz) {  // also for chunk 0: a reset there makes the initial state irrelevant
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) zero_acc<NT>(dacc[mt]);
    }
    if (resets && i + 1 < n) rz = resets[b * n + n - 2 - i];
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r * 16 * MT + mt * 16 + g + (e >> 1) * 8;
        const int col = v0 + cw + nt * 8 + 2 * tg + (e & 1);
        ds0[(static_cast<long long>(bh) * D + row) * D + col] = dacc[mt][nt][e];
      }
}

// ================================================= backward: dK, dV, d(alpha)
// CG column groups of warps: a CTA has 4 x CG warps, warp (r, cg) owns the 16 rows 16 r of a
// product and the columns [cg * W / CG, (cg + 1) * W / CG) of its W-wide result.
template <int D, int CG>
__global__ void __launch_bounds__(128 * CG, 1)
efla_bwd_final_kernel(const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_up,
                      const __grid_constant__ CUtensorMap tm_dO,
                      const __grid_constant__ CUtensorMap tm_dup,
                      const __grid_constant__ CUtensorMap tm_states,
                      const __grid_constant__ CUtensorMap tm_dstates,
                      const __grid_constant__ CUtensorMap tm_xinv,
                      const __grid_constant__ CUtensorMap tm_v, const float* __restrict__ alpha,
                      bf16* __restrict__ dk, bf16* __restrict__ dv, float* __restrict__ dalpha,
                      int T, int H, long long dks, long long dvs, int* status) {
  constexpr int NT = D / (8 * CG), CW = CH / CG, CN = CW / 8;  // per warp: NT tiles of D, CN of CH
  constexpr int TILE = (D / 64) * PANEL, STILE = (D / 64) * D * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + TILE;
  uint8_t* Ups = Ks + TILE;
  uint8_t* dOs = Ups + TILE;
  uint8_t* Zs = dOs + TILE;    // holds -dU' first, then Z
  uint8_t* Sb = Zs + TILE;     // S_in
  uint8_t* dSb = Sb + STILE;   // dS_out
  uint8_t* Xs = dSb + STILE;   // X = (I + diag(a) G)^-1 as the forward pass saved it
  uint8_t* dGs = Xs + PANEL;
  uint8_t* dPs = dGs + PANEL;
  uint8_t* Vs = dPs + PANEL;   // V, for R = V - K S_in
  float* Gs = reinterpret_cast<float*>(Vs + TILE);
  float* al = Gs + CH * GLD;
  float* dal = al + CH;
  uint64_t* bars = reinterpret_cast<uint64_t*>(dal + CH);

  const int bh = blockIdx.y, b = bh / H, h = bh - b * H, n = T / CH;
  const int tok0 = b * T + blockIdx.x * CH;
  const int srow = (bh * n + blockIdx.x) * D;
  // every tile is requested up front, in the order the steps below need them
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 4);
    mbar_init(&bars[2], 2);
    mbar_init(&bars[3], 1);
    mbar_init(&bars[4], 1);
    fence_mbar_init();
  }
  __syncthreads();
  // one thread per tile requests it (a TMA instruction is slow to issue; spread them)
  switch (threadIdx.x) {
    case 0:
      mbar_arrive_expect_tx(&bars[0], TILE);
      tma_tok_tile<D>(Ks, &tm_k, &bars[0], h * D, tok0);
      break;
    case 32:
      mbar_arrive_expect_tx(&bars[1], PANEL);
      tma_load_2d(Xs, &tm_xinv, &bars[1], 0, (bh * n + blockIdx.x) * CH);
      break;
    case 64:
      mbar_arrive_expect_tx(&bars[1], TILE);
      tma_tok_tile<D>(Zs, &tm_dup, &bars[1], h * D, tok0);
      break;
    case 96:
      mbar_arrive_expect_tx(&bars[1], STILE);
      tma_state_tile<D>(Sb, &tm_states, &bars[1], srow);
      break;
    case 128:
      mbar_arrive_expect_tx(&bars[2], TILE);
      tma_tok_tile<D>(Ups, &tm_up, &bars[2], h * D, tok0);
      break;
    case 160:
      mbar_arrive_expect_tx(&bars[2], TILE);
      tma_tok_tile<D>(dOs, &tm_dO, &bars[2], h * D, tok0);
      break;
    case 192:
      mbar_arrive_expect_tx(&bars[3], TILE);
      tma_tok_tile<D>(Qs, &tm_q, &bars[3], h * D, tok0);
      break;
    case 224:
      mbar_arrive_expect_tx(&bars[4], STILE);
      tma_state_tile<D>(dSb, &tm_dstates, &bars[4], srow);
      break;
    case 16:
      mbar_arrive_expect_tx(&bars[1], TILE);
      tma_tok_tile<D>(Vs, &tm_v, &bars[1], h * D, tok0);
      break;
    default:
      break;
  }
  // alpha is requested now, parked in shared memory after the Gram product (first use: step 3)
  const float my_al =
      threadIdx.x < CH ? alpha[(static_cast<long long>(tok0) + threadIdx.x) * H + h] : 0.f;
#if CEO_BF_PREFETCH
  // One CTA fits an SM, so nothing overlaps the arrival of a CTA's first tiles.  CTAs are
  // handed out in linear order: the one that follows this one on this SM is about gridDim
  // CTAs-in-flight further on; its tiles are pulled into L2 now.
  {
    const long long lin = static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x + BF_AHEAD;
    if (lin < static_cast<long long>(gridDim.x) * gridDim.y) {
      const int nx = static_cast<int>(lin % gridDim.x), nbh = static_cast<int>(lin / gridDim.x);
      const int nb = nbh / H, nh = nbh - nb * H;
      const int ntok0 = nb * T + nx * CH, nsrow = (nbh * n + nx) * D;
      switch (threadIdx.x) {
        case 1: tma_prefetch_3d(&tm_k, 0, ntok0, (nh * D) >> 6); break;
        case 33: tma_prefetch_2d(&tm_xinv, 0, (nbh * n + nx) * CH); break;
        case 65: tma_prefetch_3d(&tm_dup, 0, ntok0, (nh * D) >> 6); break;
        case 97: tma_prefetch_3d(&tm_states, 0, nsrow, 0); break;
        case 129: tma_prefetch_3d(&tm_up, 0, ntok0, (nh * D) >> 6); break;
        case 161: tma_prefetch_3d(&tm_dO, 0, ntok0, (nh * D) >> 6); break;
        case 193: tma_prefetch_3d(&tm_q, 0, ntok0, (nh * D) >> 6); break;
        case 225: tma_prefetch_3d(&tm_dstates, 0, nsrow, 0); break;
        case 17: tma_prefetch_3d(&tm_v, 0, ntok0, (nh * D) >> 6); break;
        default: break;
      }
    }
  }
#endif
  tile_wait(&bars[0], status);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int r = warp & 3, cg = warp >> 2;
  const int c0 = (D / CG) * cg;
  const SwzTile Qt = swz_tile(Qs, CH), Kt = swz_tile(Ks, CH), Upt = swz_tile(Ups, CH),
                dOt = swz_tile(dOs, CH), Zt = swz_tile(Zs, CH), St = swz_tile(Sb, D),
                dSt = swz_tile(dSb, D), Xt = swz_tile(Xs, CH), dGt = swz_tile(dGs, CH),
                dPt = swz_tile(dPs, CH), Vt = swz_tile(Vs, CH);

  // 1. G = K K^T, strictly lower part, fp32 (step 4 needs it for d(alpha))
  {
    float acc[CN][4];
    zero_acc<CN>(acc);
    wg<CN, D, false, false>(acc, Kt, 16 * r, Kt, CW * cg);
#pragma unroll
    for (int nt = 0; nt < CN; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = 16 * r + g + (e >> 1) * 8, col = CW * cg + nt * 8 + 2 * tg + (e & 1);
        Gs[row * GLD + col] = col < row ? acc[nt][e] : 0.f;
      }
  }
  if (threadIdx.x < CH) {
    al[threadIdx.x] = my_al;
    dal[threadIdx.x] = 0.f;
  }
  __syncthreads();
  tile_wait(&bars[1], status);
  // 3. Z = X^T dU' ; R = V - K S_in ; dV = a Z ; d(alpha) += Z . R
  float zacc[NT][4];
  zero_acc<NT>(zacc);
  wg<NT, CH, true, true>(zacc, Xt, 16 * r, Zt, c0);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)  // `dup` holds -dU'
#pragma unroll
    for (int e = 0; e < 4; ++e) zacc[nt][e] = -zacc[nt][e];
  {
    float racc[NT][4];
    zero_acc<NT>(racc);
    wg<NT, D, false, true>(racc, Kt, 16 * r, St, c0);
    float p[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = c0 + nt * 8 + 2 * tg;
        const long long tok = static_cast<long long>(tok0) + row;
        const float2 vv = lds_bf162(Vt.at(row, col));
        p[hf] += zacc[nt][2 * hf] * (vv.x - racc[nt][2 * hf]) +
                 zacc[nt][2 * hf + 1] * (vv.y - racc[nt][2 * hf + 1]);
        const float a = al[row];
        *reinterpret_cast<bf162*>(dv + tok * dvs + h * D + col) =
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
  __syncthreads();  // every warp is done reading dU' out of Zs and X out of the first panel
  frag_store_swz<NT>(Zt, 16 * r, c0, zacc);
  tile_wait(&bars[2], status);
  __syncthreads();
  // 4. dA = -strict_tril(Z U'^T) ; d(alpha) += dA . G ; dG = a dA ;  dP = tril(dO U'^T)
  {
    float acc[CN][4];
    zero_acc<CN>(acc);
    wg<CN, D, false, false>(acc, Zt, 16 * r, Upt, CW * cg);
    float p[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < CN; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = CW * cg + nt * 8 + 2 * tg;
        const float a = al[row];
        const float d0 = col < row ? -acc[nt][2 * hf] : 0.f;
        const float d1 = col + 1 < row ? -acc[nt][2 * hf + 1] : 0.f;
        p[hf] += d0 * Gs[row * GLD + col] + d1 * Gs[row * GLD + col + 1];
        sts_bf162(dGt.at(row, col), a * d0, a * d1);
      }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float s = p[hf];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (tg == 0) atomicAdd(&dal[16 * r + g + hf * 8], s);
    }
    zero_acc<CN>(acc);
    wg<CN, D, false, false>(acc, dOt, 16 * r, Upt, CW * cg);
#pragma unroll
    for (int nt = 0; nt < CN; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * r + g + hf * 8, col = CW * cg + nt * 8 + 2 * tg;
        sts_bf162(dPt.at(row, col), col <= row ? acc[nt][2 * hf] : 0.f,
                  col + 1 <= row ? acc[nt][2 * hf + 1] : 0.f);
      }
  }
  tile_wait(&bars[3], status);
  __syncthreads();
  // 5. dK = -a (Z S_in^T) + dG K + dG^T K + dP^T Q + U' dS_out^T
  float kacc[NT][4];
  zero_acc<NT>(kacc);
  wg<NT, D, false, false>(kacc, Zt, 16 * r, St, c0);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) kacc[nt][e] *= -al[16 * r + g + (e >> 1) * 8];
  wg<NT, CH, false, true>(kacc, dGt, 16 * r, Kt, c0);
  wg<NT, CH, true, true>(kacc, dGt, 16 * r, Kt, c0);
  wg<NT, CH, true, true>(kacc, dPt, 16 * r, Qt, c0);
  tile_wait(&bars[4], status);
  wg<NT, D, false, false>(kacc, Upt, 16 * r, dSt, c0);
  frag_store_bf16<NT>(dk + (static_cast<long long>(tok0) + 16 * r) * dks + h * D + c0, dks, kacc);
  if (threadIdx.x < CH)
    dalpha[(static_cast<long long>(tok0) + threadIdx.x) * H + h] = dal[threadIdx.x];
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

// D / 8 lanes share one (token, head) row, eight elements (one 16-byte access) each, so a
// warp covers 32 / (D / 8) rows at a time.
template <int LPR>
__device__ __forceinline__ float group_reduce_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// A warp takes U * RPW consecutive (token, head) rows per iteration and requests all of their
// 16-byte pieces before it uses any (2 U loads in flight per lane forward, 4 U backward): with
// one row group in flight per warp these kernels ran at half the memory bandwidth.
// rows * H < 2^31 (checked on the host), so row ids divide as 32-bit integers.
template <int D>
__global__ void __launch_bounds__(256)
efla_prep_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                     const float* __restrict__ beta, int beta_scalar, bf16* __restrict__ qn,
                     bf16* __restrict__ kn, float* __restrict__ rq, float* __restrict__ rk,
                     float* __restrict__ alpha, long long rows, int H, long long qs, long long ks,
                     int normalize) {
  constexpr int LPR = D / 8, RPW = 32 / LPR, U = 4;
  const int lane = threadIdx.x & 31, sub = lane % LPR, rw = lane / LPR;
  const unsigned wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned nw = (gridDim.x * blockDim.x) >> 5;
  const unsigned total = static_cast<unsigned>(rows * H);
  for (unsigned id0 = wid * (RPW * U); id0 < total; id0 += nw * (RPW * U)) {
    uint4 qp[U], kp[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned id = id0 + u * RPW + rw;
      const unsigned idc = id < total ? id : 0;
      const unsigned tok = idc / static_cast<unsigned>(H), h = idc - tok * H;
      qp[u] = *reinterpret_cast<const uint4*>(q + tok * qs + h * D + sub * 8);
      kp[u] = *reinterpret_cast<const uint4*>(k + tok * ks + h * D + sub * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned id = id0 + u * RPW + rw;
      float qv[8], kv[8];
      unpack8(qp[u], qv);
      unpack8(kp[u], kv);
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sq += qv[e] * qv[e];
        sk += kv[e] * kv[e];
      }
      sq = group_reduce_sum<LPR>(sq);
      sk = group_reduce_sum<LPR>(sk);
      const float iq = normalize ? rsqrtf(sq + 1e-6f) : 1.f;
      const float ik = normalize ? rsqrtf(sk + 1e-6f) : 1.f;
      if (id >= total) continue;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        qv[e] *= iq;
        kv[e] *= ik;
      }
      *reinterpret_cast<uint4*>(qn + static_cast<long long>(id) * D + sub * 8) = pack8(qv);
      *reinterpret_cast<uint4*>(kn + static_cast<long long>(id) * D + sub * 8) = pack8(kv);
      if (sub == 0) {
        const float b = beta_scalar ? beta[0] : beta[id];
        rq[id] = iq;
        rk[id] = ik;
        alpha[id] = normalize ? -expm1f(-b) : efla_coeff(b, sk);
      }
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
  constexpr int LPR = D / 8, RPW = 32 / LPR, U = 2;
  const int lane = threadIdx.x & 31, sub = lane % LPR, rw = lane / LPR;
  const unsigned wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned nw = (gridDim.x * blockDim.x) >> 5;
  const unsigned total = static_cast<unsigned>(rows * H);
  for (unsigned id0 = wid * (RPW * U); id0 < total; id0 += nw * (RPW * U)) {
    uint4 qp[U], kp[U], gqp[U], gkp[U];
    float bb[U], daa[U], iqq[U], ikk[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned id = id0 + u * RPW + rw;
      const unsigned idc = id < total ? id : 0;
      const long long o = static_cast<long long>(idc) * D + sub * 8;
      qp[u] = *reinterpret_cast<const uint4*>(qn + o);
      kp[u] = *reinterpret_cast<const uint4*>(kn + o);
      gqp[u] = *reinterpret_cast<const uint4*>(dqn + o);
      gkp[u] = *reinterpret_cast<const uint4*>(dkn + o);
      bb[u] = beta_scalar ? beta[0] : beta[idc];
      daa[u] = dalpha[idc];
      iqq[u] = rq[idc];
      ikk[u] = rk[idc];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned id = id0 + u * RPW + rw;
      float qv[8], kv[8], gq[8], gk[8];
      unpack8(qp[u], qv);
      unpack8(kp[u], kv);
      unpack8(gqp[u], gq);
      unpack8(gkp[u], gk);
      float dq_dot = 0.f, dk_dot = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dq_dot += qv[e] * gq[e];
        dk_dot += kv[e] * gk[e];
        sk += kv[e] * kv[e];
      }
      dq_dot = group_reduce_sum<LPR>(dq_dot);
      dk_dot = group_reduce_sum<LPR>(dk_dot);
      sk = group_reduce_sum<LPR>(sk);
      if (id >= total) continue;
      const float b = bb[u], da = daa[u];
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
      const float iq = iqq[u], ik = ikk[u];
      float oq[8], ok[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (normalize) {
          oq[e] = iq * (gq[e] - qv[e] * dq_dot);
          ok[e] = ik * (gk[e] - kv[e] * dk_dot);
        } else {
          oq[e] = gq[e];
          ok[e] = gk[e] + kcoef * kv[e];
        }
      }
      const unsigned tok = id / static_cast<unsigned>(H), h = id - tok * H;
      *reinterpret_cast<uint4*>(dq + tok * dqs + h * D + sub * 8) = pack8(oq);
      *reinterpret_cast<uint4*>(dk + tok * dks + h * D + sub * 8) = pack8(ok);
      if (sub == 0) dbeta[id] = db;
    }
  }
}

// ------------------------------------------------------------------ host side
constexpr int BAR_BYTES = 64;  // up to eight mbarriers
template <int D> constexpr int tile_bytes() { return (D / 64) * PANEL; }
template <int D> constexpr int stile_bytes() { return (D / 64) * D * 128; }
template <int D> constexpr int smem_wy() { return 2 * tile_bytes<D>() + PANEL + CH * GLD * 4 + CH * 4 + BAR_BYTES + 1024; }
template <int D> constexpr int smem_state_fwd() { return 4 * tile_bytes<D>() + 2 * PANEL + D * 128 + static_cast<int>(sizeof(SerialSync)) + 1024; }
template <int D> constexpr int smem_out() { return 3 * tile_bytes<D>() + stile_bytes<D>() + PANEL + BAR_BYTES + 1024; }
template <int D> constexpr int smem_bwd_local() { return 4 * tile_bytes<D>() + stile_bytes<D>() + BAR_BYTES + 1024; }
template <int D> constexpr int smem_state_bwd() { return 2 * (3 * tile_bytes<D>() + 2 * PANEL) + D * 128 + PANEL + static_cast<int>(sizeof(SerialSync)) + 1024; }
template <int D> constexpr int smem_bwd_final() { return 6 * tile_bytes<D>() + 2 * stile_bytes<D>() + 3 * PANEL + CH * GLD * 4 + 2 * CH * 4 + BAR_BYTES + 1024; }

template <typename Kern>
static cudaError_t set_smem(Kern kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}
template <int D>
static cudaError_t efla_configure() {
  static bool cfg = false;
  if (cfg) return cudaSuccess;
  cudaError_t e;
  if ((e = set_smem(efla_wy_kernel<D>, smem_wy<D>())) != cudaSuccess) return e;
  if ((e = set_smem(efla_state_fwd_kernel<D>, smem_state_fwd<D>())) != cudaSuccess) return e;
  if ((e = set_smem(efla_out_kernel<D>, smem_out<D>())) != cudaSuccess) return e;
  if (D == 128 && (e = set_smem(efla_out_tc_kernel, OUT_TC_SMEM)) != cudaSuccess) return e;
  if ((e = set_smem(efla_bwd_local_kernel<D>, smem_bwd_local<D>())) != cudaSuccess) return e;
  if ((e = set_smem(efla_state_bwd_kernel<D>, smem_state_bwd<D>())) != cudaSuccess) return e;
  if ((e = set_smem(efla_bwd_final_kernel<D, BF_CG>, smem_bwd_final<D>())) != cudaSuccess) return e;
  cfg = true;
  return cudaSuccess;
}

// 1: the output kernel runs on tcgen05 (efla_out_tc_kernel) where the shape allows.  Off by
// default: with one CTA per SM its TMA latency is exposed and it measures slower than the
// warp-MMA kernel (58 us against 41 us for 8192 tokens, H = 16, d = 128).
static int g_out_tcgen05 = 0;

// Every tensor a stage touches through TMA, by the slot numbers of ceo_efla_stage.
struct EflaTensors {
  const void* p[25];
  long long stride[6];  // q, k, v, dq, dk, dv
};
enum { I_Q = 0, I_K, I_V, I_ALPHA, I_W, I_U, I_UP, I_STATES, I_O, I_S0, I_SFINAL, I_DO, I_DLOC,
       I_DUP, I_DSTATES, I_DSFINAL, I_DS0, I_DQ, I_DK, I_DV, I_DALPHA, I_PFINAL, I_STATUS, I_XINV, I_RESETS };

template <int D>
static int efla_run_stage(int stage, const EflaTensors& t, int B, int T, int H, cudaStream_t st) {
  if (efla_configure<D>() != cudaSuccess) return static_cast<int>(cudaGetLastError());
  const int n = T / CH;
  const long long tokens = static_cast<long long>(B) * T, HD = static_cast<long long>(H) * D;
  const long long srows = static_cast<long long>(B) * H * n * D;
  if (tokens > 0x7fffffffll || srows > 0x7fffffffll) return -5;
  auto b16 = [&](int i) { return static_cast<bf16*>(const_cast<void*>(t.p[i])); };
  auto f32 = [&](int i) { return static_cast<float*>(const_cast<void*>(t.p[i])); };
  int* status = static_cast<int*>(const_cast<void*>(t.p[I_STATUS]));
  // token-major map of slot i (leading dimension: its token stride), state map of slot i
  auto tok = [&](CUtensorMap* tm, int i, long long stride) {
    if (!t.p[i] || (reinterpret_cast<uintptr_t>(t.p[i]) & 15) || (stride & 7)) return -2;
    return encode_tmap_2d_bf16(tm, t.p[i], static_cast<uint64_t>(HD), tokens, stride, CH) ? -3 : 0;
  };
  auto sta = [&](CUtensorMap* tm, int i) {
    if (!t.p[i] || (reinterpret_cast<uintptr_t>(t.p[i]) & 15)) return -2;
    return encode_tmap_2d_bf16(tm, t.p[i], D, srows, D, D) ? -3 : 0;
  };
  // panel maps: one request per whole 64 x D token tile / D x D state
  auto tokp = [&](CUtensorMap* tm, int i, long long stride) {
    if (!t.p[i] || (reinterpret_cast<uintptr_t>(t.p[i]) & 15) || (stride & 7)) return -2;
    return encode_tmap_panels_bf16(tm, t.p[i], static_cast<uint64_t>(HD), tokens, stride, CH,
                                   D / 64) ? -3 : 0;
  };
  auto stap = [&](CUtensorMap* tm, int i) {
    if (!t.p[i] || (reinterpret_cast<uintptr_t>(t.p[i]) & 15)) return -2;
    return encode_tmap_panels_bf16(tm, t.p[i], D, srows, D, D, D / 64) ? -3 : 0;
  };
  const dim3 gpar(n, B * H);
  CUtensorMap m[9];
  int rc = 0;
#define MAP(call) if ((rc = (call)) != 0) return rc
  switch (stage) {
    case 0:
      MAP(tokp(&m[0], I_K, t.stride[1]));
      MAP(tokp(&m[1], I_V, t.stride[2]));
      if (!t.p[I_XINV]) return -5;
      efla_wy_kernel<D><<<gpar, 128, smem_wy<D>(), st>>>(m[0], m[1], f32(I_ALPHA), b16(I_W),
                                                         b16(I_U), b16(I_XINV), T, H, status);
      break;
    case 1:
      MAP(tokp(&m[0], I_K, t.stride[1]));
      MAP(tokp(&m[1], I_W, HD));
      MAP(tok(&m[2], I_U, HD));
      MAP(tok(&m[3], I_UP, HD));
      MAP(sta(&m[4], I_STATES));
      efla_state_fwd_kernel<D><<<dim3(t.p[I_PFINAL] ? 2 * (D / BV) : D / BV, B * H), SER_THREADS,
                                 smem_state_fwd<D>(), st>>>(
          m[0], m[1], m[2], m[3], m[4], f32(I_S0), f32(I_SFINAL), f32(I_PFINAL),
          static_cast<const unsigned char*>(t.p[I_RESETS]), T, H, status);
      break;
    case 2:
      if (g_out_tcgen05 && D == 128 && (n & 1) == 0) {  // chunk pairs on the tcgen05 path
        MAP(tok(&m[0], I_Q, t.stride[0]));
        MAP(tok(&m[1], I_K, t.stride[1]));
        MAP(tok(&m[2], I_UP, HD));
        MAP(sta(&m[3], I_STATES));
        efla_out_tc_kernel<<<dim3(n / 2, B * H), OUT_TC_THREADS, OUT_TC_SMEM, st>>>(
            m[0], m[1], m[2], m[3], b16(I_O), T, H, status);
      } else {
        MAP(tokp(&m[0], I_Q, t.stride[0]));
        MAP(tokp(&m[1], I_K, t.stride[1]));
        MAP(tokp(&m[2], I_UP, HD));
        MAP(stap(&m[3], I_STATES));
        efla_out_kernel<D><<<gpar, 256, smem_out<D>(), st>>>(m[0], m[1], m[2], m[3], b16(I_O), T,
                                                             H, status);
      }
      break;
    case 3:
      MAP(tokp(&m[0], I_Q, t.stride[0]));
      MAP(tokp(&m[1], I_K, t.stride[1]));
      MAP(tokp(&m[2], I_UP, HD));
      MAP(tokp(&m[3], I_DO, HD));
      MAP(stap(&m[4], I_STATES));
      efla_bwd_local_kernel<D><<<gpar, 256, smem_bwd_local<D>(), st>>>(
          m[0], m[1], m[2], m[3], m[4], b16(I_DQ), b16(I_DLOC), T, H, t.stride[3], status);
      break;
    case 4:
      MAP(tokp(&m[0], I_Q, t.stride[0]));
      MAP(tokp(&m[1], I_K, t.stride[1]));
      MAP(tokp(&m[2], I_W, HD));
      MAP(tok(&m[3], I_DO, HD));
      MAP(tok(&m[4], I_DLOC, HD));
      MAP(tok(&m[5], I_DUP, HD));
      MAP(sta(&m[6], I_DSTATES));
      efla_state_bwd_kernel<D><<<dim3(D / BV, B * H), SER_THREADS, smem_state_bwd<D>(), st>>>(
          m[0], m[1], m[2], m[3], m[4], m[5], m[6], f32(I_DSFINAL), f32(I_DS0),
          static_cast<const unsigned char*>(t.p[I_RESETS]), T, H, status);
      break;
    case 5:
      MAP(tokp(&m[0], I_Q, t.stride[0]));
      MAP(tokp(&m[1], I_K, t.stride[1]));
      MAP(tokp(&m[2], I_UP, HD));
      MAP(tokp(&m[3], I_DO, HD));
      MAP(tokp(&m[4], I_DUP, HD));
      MAP(stap(&m[5], I_STATES));
      MAP(stap(&m[6], I_DSTATES));
      if (!t.p[I_XINV] || (reinterpret_cast<uintptr_t>(t.p[I_XINV]) & 15)) return -2;
      MAP(encode_tmap_2d_bf16(&m[7], t.p[I_XINV], CH, static_cast<uint64_t>(B) * H * n * CH, CH, CH)
              ? -3 : 0);
      MAP(tokp(&m[8], I_V, t.stride[2]));
      efla_bwd_final_kernel<D, BF_CG><<<gpar, 128 * BF_CG, smem_bwd_final<D>(), st>>>(
          m[0], m[1], m[2], m[3], m[4], m[5], m[6], m[7], m[8], f32(I_ALPHA), b16(I_DK), b16(I_DV),
          f32(I_DALPHA), T, H, t.stride[4], t.stride[5], status);
      break;
    default:
      return -5;
  }
#undef MAP
  return static_cast<int>(cudaGetLastError());
}

static bool efla_args_ok(int B, int T, int H, int D, long long qs, long long ks, long long vs) {
  return B > 0 && T > 0 && H > 0 && (T % CH) == 0 && (D == 64 || D == 128) && (qs & 7) == 0 &&
         (ks & 7) == 0 && (vs & 7) == 0;
}

}  // namespace ceo
using namespace ceo;

extern "C" int ceo_efla_set_wait_limit(unsigned int iterations) {
  return ceo::set_wait_limit_override(iterations);
}

extern "C" int ceo_efla_set_tcgen05(int on) {
  ceo::g_out_tcgen05 = on != 0;
  return 0;
}

extern "C" int ceo_efla_fwd(const void* q, const void* k, const void* v, const float* alpha,
                            const float* s0, void* w, void* up, void* states, void* xinv, void* o,
                            float* s_final, const unsigned char* resets, int B, int T, int H,
                            int D, long long q_stride, long long k_stride, long long v_stride,
                            int* status, cudaStream_t stream) {
  if (!efla_args_ok(B, T, H, D, q_stride, k_stride, v_stride)) return -5;
  EflaTensors t = {};
  t.p[I_Q] = q; t.p[I_K] = k; t.p[I_V] = v; t.p[I_ALPHA] = alpha; t.p[I_W] = w;
  t.p[I_U] = o;  // U is staged in `o` (same shape, overwritten by the last kernel)
  t.p[I_UP] = up; t.p[I_STATES] = states; t.p[I_O] = o; t.p[I_S0] = s0; t.p[I_SFINAL] = s_final;
  t.p[I_STATUS] = status; t.p[I_XINV] = xinv; t.p[I_RESETS] = resets;
  t.stride[0] = q_stride; t.stride[1] = k_stride; t.stride[2] = v_stride;
  for (int stage = 0; stage < 3; ++stage) {
    const int rc = D == 64 ? efla_run_stage<64>(stage, t, B, T, H, stream)
                           : efla_run_stage<128>(stage, t, B, T, H, stream);
    if (rc) return rc;
  }
  return 0;
}

extern "C" int ceo_efla_bwd(const void* q, const void* k, const void* v, const float* alpha,
                            const void* w, const void* up, const void* states, const void* xinv,
                            const void* dO, const float* ds_final, void* dloc, void* dup,
                            void* dstates, void* dq,
                            void* dk, void* dv, float* dalpha, float* ds0,
                            const unsigned char* resets, int B, int T, int H,
                            int D, long long q_stride, long long k_stride, long long v_stride,
                            long long dq_stride, long long dk_stride, long long dv_stride,
                            int* status, cudaStream_t stream) {
  if (!efla_args_ok(B, T, H, D, q_stride, k_stride, v_stride)) return -5;
  if ((dq_stride | dk_stride | dv_stride) & 1) return -2;
  EflaTensors t = {};
  t.p[I_Q] = q; t.p[I_K] = k; t.p[I_V] = v; t.p[I_ALPHA] = alpha; t.p[I_W] = w; t.p[I_UP] = up;
  t.p[I_STATES] = states; t.p[I_DO] = dO; t.p[I_DSFINAL] = ds_final; t.p[I_DLOC] = dloc;
  t.p[I_DUP] = dup; t.p[I_DSTATES] = dstates; t.p[I_DQ] = dq; t.p[I_DK] = dk; t.p[I_DV] = dv;
  t.p[I_DALPHA] = dalpha; t.p[I_DS0] = ds0; t.p[I_STATUS] = status; t.p[I_XINV] = xinv;
  t.p[I_RESETS] = resets;
  t.stride[0] = q_stride; t.stride[1] = k_stride; t.stride[2] = v_stride;
  t.stride[3] = dq_stride; t.stride[4] = dk_stride; t.stride[5] = dv_stride;
  for (int stage = 3; stage < 6; ++stage) {
    const int rc = D == 64 ? efla_run_stage<64>(stage, t, B, T, H, stream)
                           : efla_run_stage<128>(stage, t, B, T, H, stream);
    if (rc) return rc;
  }
  return 0;
}

extern "C" int ceo_efla_prep_fwd(const void* q, const void* k, const float* beta, int beta_scalar,
                                 void* qn, void* kn, float* rq, float* rk, float* alpha,
                                 long long rows, int H, int D, long long q_stride,
                                 long long k_stride, int normalize, cudaStream_t stream) {
  if (rows <= 0 || H <= 0 || (D != 64 && D != 128) || rows * H >= (1LL << 31)) return -5;
  if (((q_stride | k_stride) & 7) ||
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
        reinterpret_cast<uintptr_t>(qn) | reinterpret_cast<uintptr_t>(kn)) & 15))
    return -2;  // rows move as 16-byte accesses
  const int grid = grid_for(rows * H, 8 * 4 * (D == 64 ? 4 : 2), 148 * 4);  // one resident wave
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
  if (rows <= 0 || H <= 0 || (D != 64 && D != 128) || rows * H >= (1LL << 31)) return -5;
  if (((dq_stride | dk_stride) & 7) ||
      ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
        reinterpret_cast<uintptr_t>(dqn) | reinterpret_cast<uintptr_t>(dkn) |
        reinterpret_cast<uintptr_t>(qn) | reinterpret_cast<uintptr_t>(kn)) & 15))
    return -2;  // rows move as 16-byte accesses
  const int grid = grid_for(rows * H, 8 * 2 * (D == 64 ? 4 : 2), 148 * 3);  // one resident wave
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
//       21 p_final (stage 1 only, optional: also computes the span's transfer matrix),
//       22 status word (int, optional) of the bounded waits,
//       23 xinv: bf16 (B,H,T/64,64,64), written by stage 0 and read by stage 5,
//       24 resets: bytes (B,T/64), optional; non-zero = the chunk starts from a zero state
// strides (elements per token): 0 q, 1 k, 2 v, 3 dq, 4 dk, 5 dv
// stage: 0 wy, 1 state_fwd, 2 out, 3 bwd_local, 4 state_bwd, 5 bwd_final
extern "C" int ceo_efla_stage(int stage, void* const* ptrs, const long long* strides, int B, int T,
                              int H, int D, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0 || (T % ceo::CH) || (D != 64 && D != 128)) return -5;
  ceo::EflaTensors t = {};
  for (int i = 0; i < 25; ++i) t.p[i] = ptrs[i];
  for (int i = 0; i < 6; ++i) {
    if (strides[i] & 7) return -2;
    t.stride[i] = strides[i];
  }
  return D == 64 ? ceo::efla_run_stage<64>(stage, t, B, T, H, stream)
                 : ceo::efla_run_stage<128>(stage, t, B, T, H, stream);
}
