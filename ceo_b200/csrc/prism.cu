// PRISM refinement: the fused gate of one iteration (forward and backward) and the recurrent
// state.
//
// One iteration l of the refinement works in the head_dim-wide proxy space:
//     rp = r W_k^l      p = u W_p^l      bt = u W_beta^l        (three GEMMs, M x hd each)
//     bd = sigmoid(bt) * GELU(p * rp)                            (prism_gate_fwd_kernel)
//     c  = bd W_k^l^T ;  r <- r - c ;  out <- out + f^(l-1) c    (GEMM + prism_update_kernel)
// and the state the reference specifies (src/model/prism.zig:11-40, PrismState 480-523),
//     S_t = alpha S_{t-1} (I - b_t k_t^T) + sum_l bd_t^l k_t^l^T ,   b_t = sigmoid(bt_t^1) * k_t^1,
// is a (hd x hd) matrix per sequence whose ROWS evolve independently of each other:
//     S_t[i,:] = alpha (S[i,:] - (S[i,:] . b_t) k_t^1) + sum_l bd_t^l[i] k_t^l
// so prism_state_kernel gives one warp to each row and walks the tokens serially.
//
// The reference declares prism_forward_cuda (kernels/cuda/include/kernels.h:86) and a Zig
// extern for a backward (src/kernels/prism_kernels.zig:24-36) without any source; its CPU loop
// fixes beta at 0.5, reads p from one weight row and never touches the state
// (src/model/prism.zig:279-320).
#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace ceo {

__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }
// tanh GELU and its derivative
__device__ __forceinline__ float gelu_t(float x) {
  const float c = 0.7978845608f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(c));
}
__device__ __forceinline__ float gelu_t_grad(float x) {
  const float c = 0.7978845608f * (x + 0.044715f * x * x * x);
  const float t = tanhf(c);
  const float dc = 0.7978845608f * (1.f + 3.f * 0.044715f * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * dc;
}

__global__ void __launch_bounds__(256)
prism_gate_fwd_kernel(const bf16* __restrict__ rp, const bf16* __restrict__ p,
                      const bf16* __restrict__ bt, bf16* __restrict__ bd, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8], b[8], c[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(rp)[i], a);
    unpack8(reinterpret_cast<const uint4*>(p)[i], b);
    unpack8(reinterpret_cast<const uint4*>(bt)[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = sigm(c[j]) * gelu_t(a[j] * b[j]);
    reinterpret_cast<uint4*>(bd)[i] = pack8(o);
  }
}

__global__ void __launch_bounds__(256)
prism_gate_bwd_kernel(const bf16* __restrict__ dbd, const bf16* __restrict__ rp,
                      const bf16* __restrict__ p, const bf16* __restrict__ bt,
                      bf16* __restrict__ drp, bf16* __restrict__ dp, bf16* __restrict__ dbt,
                      long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[8], a[8], b[8], c[8], da[8], db[8], dc[8];
    unpack8(reinterpret_cast<const uint4*>(dbd)[i], g);
    unpack8(reinterpret_cast<const uint4*>(rp)[i], a);
    unpack8(reinterpret_cast<const uint4*>(p)[i], b);
    unpack8(reinterpret_cast<const uint4*>(bt)[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float z = a[j] * b[j], s = sigm(c[j]);
      const float dz = g[j] * s * gelu_t_grad(z);
      da[j] = dz * b[j];
      db[j] = dz * a[j];
      dc[j] = g[j] * gelu_t(z) * s * (1.f - s);
    }
    reinterpret_cast<uint4*>(drp)[i] = pack8(da);
    reinterpret_cast<uint4*>(dp)[i] = pack8(db);
    reinterpret_cast<uint4*>(dbt)[i] = pack8(dc);
  }
}

// r <- r - c ;  out <- out + scale * c   (one pass over the three streams instead of two)
__global__ void __launch_bounds__(256)
prism_update_kernel(const bf16* __restrict__ c, const bf16* __restrict__ r_in,
                    const bf16* __restrict__ out_in, bf16* __restrict__ r_out,
                    bf16* __restrict__ out_out, long long n8, float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8], r[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(c)[i], x);
    unpack8(reinterpret_cast<const uint4*>(r_in)[i], r);
    unpack8(reinterpret_cast<const uint4*>(out_in)[i], o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      r[j] -= x[j];
      o[j] += scale * x[j];
    }
    reinterpret_cast<uint4*>(r_out)[i] = pack8(r);
    reinterpret_cast<uint4*>(out_out)[i] = pack8(o);
  }
}

// One warp per state row (b, i); HD / 32 columns per lane in registers; the token's vectors are
// staged in shared memory once per CTA (8 rows share them).  bd, k: (L, B, T, HD); bt1: (B, T, HD)
// holds the first iteration's beta LOGITS; state: (B, HD, HD) fp32, row = value index.
template <int HD>
__global__ void __launch_bounds__(256)
prism_state_kernel(const bf16* __restrict__ bd, const bf16* __restrict__ k,
                   const bf16* __restrict__ bt1, const float* __restrict__ s_in,
                   float* __restrict__ s_out, int B, int T, int L, float alpha) {
  constexpr int PER = HD / 32, ROWS = 8;
  __shared__ float ks[4][HD];     // k^l of the token, l < 4
  __shared__ float bs[HD];        // b = sigmoid(bt^1) * k^1
  __shared__ float bds[4][ROWS];  // bd^l[row] of this CTA's rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = HD / ROWS;
  const int b = blockIdx.x / groups, row0 = (blockIdx.x % groups) * ROWS, row = row0 + warp;
  float s[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j)
    s[j] = s_in ? s_in[(static_cast<long long>(b) * HD + row) * HD + lane + 32 * j] : 0.f;
  const long long lstride = static_cast<long long>(B) * T * HD;
  for (int t = 0; t < T; ++t) {
    const long long tok = (static_cast<long long>(b) * T + t) * HD;
    __syncthreads();  // the previous token's vectors have been consumed
    for (int i = threadIdx.x; i < L * HD; i += blockDim.x) {
      const int l = i / HD, c = i - l * HD;
      const float kv = __bfloat162float(k[l * lstride + tok + c]);
      ks[l][c] = kv;
      if (l == 0) bs[c] = sigm(__bfloat162float(bt1[tok + c])) * kv;
    }
    if (threadIdx.x < L * ROWS) {
      const int l = threadIdx.x / ROWS, r = threadIdx.x - l * ROWS;
      bds[l][r] = __bfloat162float(bd[l * lstride + tok + row0 + r]);
    }
    __syncthreads();
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) dot += s[j] * bs[lane + 32 * j];
    dot = warp_reduce_sum(dot);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int c = lane + 32 * j;
      float v = alpha * (s[j] - dot * ks[0][c]);
      for (int l = 0; l < L; ++l) v += bds[l][warp] * ks[l][c];
      s[j] = v;
    }
  }
#pragma unroll
  for (int j = 0; j < PER; ++j)
    s_out[(static_cast<long long>(b) * HD + row) * HD + lane + 32 * j] = s[j];
}

}  // namespace ceo
using namespace ceo;

static bool aligned16(const void* a, const void* b, const void* c, const void* d) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
           reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}

extern "C" int ceo_prism_gate_fwd(const void* rp, const void* p, const void* bt, void* bd,
                                  long long n, cudaStream_t stream) {
  if (n <= 0 || (n & 7) || !aligned16(rp, p, bt, bd)) return -5;
  prism_gate_fwd_kernel<<<grid_for(n >> 3, 256 * 2, 148 * 8), 256, 0, stream>>>(
      static_cast<const bf16*>(rp), static_cast<const bf16*>(p), static_cast<const bf16*>(bt),
      static_cast<bf16*>(bd), n >> 3);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_prism_gate_bwd(const void* dbd, const void* rp, const void* p, const void* bt,
                                  void* drp, void* dp, void* dbt, long long n,
                                  cudaStream_t stream) {
  if (n <= 0 || (n & 7) || !aligned16(dbd, rp, p, bt) || !aligned16(drp, dp, dbt, dbt)) return -5;
  prism_gate_bwd_kernel<<<grid_for(n >> 3, 256 * 2, 148 * 8), 256, 0, stream>>>(
      static_cast<const bf16*>(dbd), static_cast<const bf16*>(rp), static_cast<const bf16*>(p),
      static_cast<const bf16*>(bt), static_cast<bf16*>(drp), static_cast<bf16*>(dp),
      static_cast<bf16*>(dbt), n >> 3);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_prism_update(const void* c, const void* r_in, const void* out_in, void* r_out,
                                void* out_out, long long n, float scale, cudaStream_t stream) {
  if (n <= 0 || (n & 7) || !aligned16(c, r_in, out_in, r_out) ||
      (reinterpret_cast<uintptr_t>(out_out) & 15))
    return -5;
  prism_update_kernel<<<grid_for(n >> 3, 256 * 2, 148 * 8), 256, 0, stream>>>(
      static_cast<const bf16*>(c), static_cast<const bf16*>(r_in),
      static_cast<const bf16*>(out_in), static_cast<bf16*>(r_out), static_cast<bf16*>(out_out),
      n >> 3, scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_prism_state(const void* bd, const void* k, const void* bt1, const float* s_in,
                               float* s_out, int B, int T, int hd, int L, float alpha,
                               cudaStream_t stream) {
  if (B <= 0 || T <= 0 || L < 1 || L > 4 || !s_out) return -5;
  const bf16* bdp = static_cast<const bf16*>(bd);
  const bf16* kp = static_cast<const bf16*>(k);
  const bf16* btp = static_cast<const bf16*>(bt1);
  if (hd == 32)
    prism_state_kernel<32><<<B * 4, 256, 0, stream>>>(bdp, kp, btp, s_in, s_out, B, T, L, alpha);
  else if (hd == 64)
    prism_state_kernel<64><<<B * 8, 256, 0, stream>>>(bdp, kp, btp, s_in, s_out, B, T, L, alpha);
  else if (hd == 128)
    prism_state_kernel<128><<<B * 16, 256, 0, stream>>>(bdp, kp, btp, s_in, s_out, B, T, L, alpha);
  else
    return -5;
  return static_cast<int>(cudaGetLastError());
}
