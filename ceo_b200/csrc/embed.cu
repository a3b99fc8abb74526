// Embedding gather (forward) and scatter-add into an fp32 gradient (backward),
// plus generic row gather / scatter utilities.  The reference declares
// embedding_forward_cuda (kernels/cuda/include/kernels.h:366) without a source and
// gathers rows on the CPU (src/nn/layers.zig:659-686).
#include "common/util.cuh"
#include "common/check.cuh"
#include "include/ceo_kernels.h"

CEO_BOUNDS_TU(embed)

namespace ceo {

// One warp per token row; ids outside [0, vocab) produce a zero row and bump *oob.
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids,
                                     const bf16* __restrict__ table, bf16* __restrict__ out,
                                     long long n, int D, long long vocab, int* oob) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int nv = D >> 3;
  for (long long r = w; r < n; r += nw) {
    const long long id = ids[r];
    uint4* o = reinterpret_cast<uint4*>(out + r * D);
    if (id < 0 || id >= vocab) {
      if (lane == 0 && oob) atomicAdd(oob, 1);
      for (int c = lane; c < nv; c += 32) o[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(table);
    for (int c = lane; c < nv; c += 32)
      reinterpret_cast<uint4*>(out)[CEO_IDX(r * nv + c, n * nv, 301)] =
          s[CEO_IDX(id * nv + c, vocab * nv, 302)];
  }
}

// dtable[ids[r]] += dy[r]  (fp32 accumulation with vector reductions)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids,
                                     const bf16* __restrict__ dy, float* __restrict__ dtable,
                                     long long n, int D, long long vocab) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int nv = D >> 3;
  for (long long r = w; r < n; r += nw) {
    const long long id = ids[r];
    if (id < 0 || id >= vocab) continue;
    const uint4* s = reinterpret_cast<const uint4*>(dy + r * D);
    float* d = dtable + id * D;
    for (int c = lane; c < nv; c += 32) {
      float f[8];
      unpack8(s[c], f);
      float* p = d + c * 8;
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(f[0]), "f"(f[1]),
                   "f"(f[2]), "f"(f[3])
                   : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + 4), "f"(f[4]),
                   "f"(f[5]), "f"(f[6]), "f"(f[7])
                   : "memory");
    }
  }
}

}  // namespace ceo
using namespace ceo;

extern "C" int ceo_embedding_fwd(const long long* ids, const void* table, void* out, long long n,
                                 int D, long long vocab, int* oob_count, cudaStream_t stream) {
  if (n <= 0 || D <= 0 || (D & 7)) return -5;
  embedding_fwd_kernel<<<grid_for(n, 8, 148 * 32), 256, 0, stream>>>(
      ids, static_cast<const bf16*>(table), static_cast<bf16*>(out), n, D, vocab, oob_count);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_embedding_bwd(const long long* ids, const void* dy, float* dtable, long long n,
                                 int D, long long vocab, cudaStream_t stream) {
  if (n <= 0 || D <= 0 || (D & 7)) return -5;
  embedding_bwd_kernel<<<grid_for(n, 8, 148 * 32), 256, 0, stream>>>(
      ids, static_cast<const bf16*>(dy), dtable, n, D, vocab);
  return static_cast<int>(cudaGetLastError());
}
