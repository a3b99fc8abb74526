// Warp-level bf16 tensor-core tiles out of shared memory (ldmatrix + mma.sync
// m16n8k16, fp32 accumulate) for the small per-chunk products of the EFLA kernels
// (64x64x128 and the like), where one warp owns 16 or 32 output rows.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace ceo {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// ---- products over tiles in the layout TMA writes with 128-byte swizzle ------------------
// A tile of R rows x C columns (bf16) is stored as C/64 panels of R rows x 128 bytes; inside a
// panel the 16-byte chunk j of row r sits at chunk (j ^ (r & 7)).  Panels start on 1024-byte
// boundaries.  ldmatrix rows are whole chunks, so fragments load conflict-free.
struct SwzTile {
  uint32_t base;         // shared-space address of the tile
  uint32_t panel_bytes;  // rows * 128
  __device__ __forceinline__ uint32_t at(int row, int col) const {
    return base + (col >> 6) * panel_bytes + row * 128 +
           (((((col >> 3) & 7) ^ (row & 7))) << 4) + (col & 7) * 2;
  }
};
__device__ __forceinline__ SwzTile swz_tile(const void* p, int rows) {
  SwzTile t;
  t.base = smem_addr(p);
  t.panel_bytes = rows * 128;
  return t;
}
__device__ __forceinline__ void sts_bf162(uint32_t addr, float x, float y) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(*reinterpret_cast<const uint32_t*>(&v))
               : "memory");
}
__device__ __forceinline__ float2 lds_bf162(uint32_t addr) {
  uint32_t u;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(u) : "r"(addr));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
}

// acc[MT][NT][4] += A (16*MT x K) * B (K x 8*NT) with A rows m0.. and B columns n0.. of
// swizzled tiles.
//   A_T = false: A tile stored [m][k];  true: stored [k][m]
//   B_T = false: B tile stored [n][k];  true: stored [k][n]
// Accumulator layout (g = lane/4, t = lane%4): acc[mt][nt][0..1] -> row 16*mt+g, cols
// nt*8+2t, +1; acc[mt][nt][2..3] -> row 16*mt+g+8, same cols.
// The MT row tiles share every B fragment, and the fragments of k-step i+1 are requested
// before the MMAs of k-step i are issued (two register sets), so ldmatrix latency overlaps
// the tensor work; the asm statements are volatile, hence emitted in exactly this order.
template <int MT, int NT, bool A_T, bool B_T>
__device__ __forceinline__ void warp_frags_swz(uint32_t (*a)[4], uint32_t (*b)[4],
                                               const SwzTile& A, int m0, const SwzTile& B, int n0,
                                               int k0) {
  const int lane = threadIdx.x & 31;
  const int l7 = lane & 7, b3 = (lane >> 3) & 1, b4 = lane >> 4;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    if (!A_T)
      ldsm_x4(a[mt], A.at(m0 + mt * 16 + l7 + b3 * 8, k0 + b4 * 8));
    else
      ldsm_x4_t(a[mt], A.at(k0 + l7 + b4 * 8, m0 + mt * 16 + b3 * 8));
  }
#pragma unroll
  for (int nt = 0; nt < NT; nt += 2) {
    if (!B_T)
      ldsm_x4(b[nt / 2], B.at(n0 + nt * 8 + l7 + b4 * 8, k0 + b3 * 8));
    else
      ldsm_x4_t(b[nt / 2], B.at(k0 + l7 + b3 * 8, n0 + nt * 8 + b4 * 8));
  }
}
template <int MT, int NT, int K, bool A_T, bool B_T>
__device__ __forceinline__ void warp_gemm_swz(float (*acc)[NT][4], const SwzTile& A, int m0,
                                              const SwzTile& B, int n0) {
  static_assert(NT % 2 == 0 && K % 16 == 0, "tile shape");
  constexpr bool PIPE = (4 * MT + 2 * NT) <= 24;
  constexpr int NB = PIPE ? 2 : 1;
  uint32_t a[NB][MT][4], b[NB][NT / 2][4];
  if (PIPE) warp_frags_swz<MT, NT, A_T, B_T>(a[0], b[0], A, m0, B, n0, 0);
#pragma unroll
  for (int k0 = 0; k0 < K; k0 += 16) {
    const int cur = PIPE ? (k0 / 16) & 1 : 0;
    if (!PIPE) warp_frags_swz<MT, NT, A_T, B_T>(a[0], b[0], A, m0, B, n0, k0);
    if (PIPE && k0 + 16 < K)
      warp_frags_swz<MT, NT, A_T, B_T>(a[cur ^ 1], b[cur ^ 1], A, m0, B, n0, k0 + 16);
#pragma unroll
    for (int nt = 0; nt < NT; nt += 2)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma16816(acc[mt][nt], a[cur][mt], b[cur][nt / 2]);
        mma16816(acc[mt][nt + 1], a[cur][mt], b[cur][nt / 2] + 2);
      }
  }
}
// Same product with the k-steps dealt alternately to two accumulator sets that are summed at
// the end: for a single row tile with a long K the dependent MMA chain is what bounds the
// time, and this halves it (used on the serial critical path of the state recurrences).
template <int NT, int K, bool A_T, bool B_T>
__device__ __forceinline__ void warp_gemm_swz_2chain(float (*acc)[4], const SwzTile& A, int m0,
                                                     const SwzTile& B, int n0) {
  static_assert(NT % 2 == 0 && K % 32 == 0, "tile shape");
  float acc2[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc2[i][0] = acc2[i][1] = acc2[i][2] = acc2[i][3] = 0.f;
  uint32_t a[2][1][4], b[2][NT / 2][4];
  warp_frags_swz<1, NT, A_T, B_T>(a[0], b[0], A, m0, B, n0, 0);
#pragma unroll
  for (int k0 = 0; k0 < K; k0 += 16) {
    const int cur = (k0 / 16) & 1;
    if (k0 + 16 < K) warp_frags_swz<1, NT, A_T, B_T>(a[cur ^ 1], b[cur ^ 1], A, m0, B, n0, k0 + 16);
    float (*dst)[4] = cur ? acc2 : acc;
#pragma unroll
    for (int nt = 0; nt < NT; nt += 2) {
      mma16816(dst[nt], a[cur][0], b[cur][nt / 2]);
      mma16816(dst[nt + 1], a[cur][0], b[cur][nt / 2] + 2);
    }
  }
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] += acc2[i][e];
}

// Stores a 16 x 8*NT accumulator tile as bf16 at rows m0.., columns n0.. of a swizzled tile.
template <int NT>
__device__ __forceinline__ void frag_store_swz(const SwzTile& t, int m0, int n0,
                                               float (*acc)[4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    sts_bf162(t.at(m0 + g, n0 + nt * 8 + 2 * tg), acc[nt][0], acc[nt][1]);
    sts_bf162(t.at(m0 + g + 8, n0 + nt * 8 + 2 * tg), acc[nt][2], acc[nt][3]);
  }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (*acc)[4]) {
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
}

}  // namespace ceo
