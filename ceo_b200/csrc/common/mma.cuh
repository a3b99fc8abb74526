// Warp-level bf16 tensor-core tiles out of shared memory (ldmatrix + mma.sync
// m16n8k16, fp32 accumulate) for the small per-chunk products of the EFLA kernels
// (64x64x128 and the like), where one warp owns 16 output rows.
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

// acc[NT][4] += A (16 x K) * B (K x 8*NT), operands in shared memory (bf16).
//   A_T = false: A stored [m][k] with leading dimension lda; `A` points at (m0, 0)
//   A_T = true : A stored [k][m];                            `A` points at (0, m0)
//   B_T = false: B stored [n][k] with leading dimension ldb; `B` points at (n0, 0)
//   B_T = true : B stored [k][n];                            `B` points at (0, n0)
// Rows of both tiles must start on 16-byte boundaries (lda, ldb multiples of 8).
// Accumulator layout (g = lane/4, t = lane%4): acc[nt][0..1] -> row g, cols nt*8+2t, +1;
// acc[nt][2..3] -> row g+8, same cols.
template <int NT, int K, bool A_T, bool B_T>
__device__ __forceinline__ void warp_gemm(float (*acc)[4], const __nv_bfloat16* A, int lda,
                                          const __nv_bfloat16* B, int ldb) {
  static_assert(NT % 2 == 0 && K % 16 == 0, "tile shape");
  const int lane = threadIdx.x & 31;
  const int l7 = lane & 7, b3 = (lane >> 3) & 1, b4 = lane >> 4;
#pragma unroll
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t a[4];
    if (!A_T)
      ldsm_x4(a, smem_addr(A + (l7 + b3 * 8) * lda + k0 + b4 * 8));
    else
      ldsm_x4_t(a, smem_addr(A + (k0 + l7 + b4 * 8) * lda + b3 * 8));
#pragma unroll
    for (int nt = 0; nt < NT; nt += 2) {
      uint32_t b[4];
      if (!B_T)
        ldsm_x4(b, smem_addr(B + (nt * 8 + l7 + b4 * 8) * ldb + k0 + b3 * 8));
      else
        ldsm_x4_t(b, smem_addr(B + (k0 + l7 + b3 * 8) * ldb + nt * 8 + b4 * 8));
      mma16816(acc[nt], a, b);
      mma16816(acc[nt + 1], a, b + 2);
    }
  }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (*acc)[4]) {
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
}

// cp.async 16-byte copy, global -> shared
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(smem_dst)), "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

}  // namespace ceo
