// Collectives fused with their adjacent compute, over peer-mapped memory (NVLink / NVSwitch).
//
// Every rank maps every other rank's communication buffers (CUDA IPC handles, exchanged on
// the host), so one kernel per rank can load from and store to its peers directly:
//
//   zero_step_kernel   gradient reduce-scatter (peer loads, fp32 sum) + global-norm clip +
//                      AdamW on the rank's fp32 master slice + bf16 parameter all-gather
//                      (peer stores) + gradient zeroing, in ONE cooperative launch.
//   symm_barrier_kernel / symm_allreduce_kernel   flag barrier and small all-reduce.
//
// Cross-rank synchronisation uses per-rank flag words in peer-mapped memory written with
// system-scope release stores and polled with a bounded loop: a wait that runs out writes a
// status word and the kernel carries on to its end, so the context stays usable.
// No multicast TMA and no multimem here: plain peer loads and stores only.
//
// The reference has NCCL wrappers only and no call site for any gradient or parameter
// collective (src/runtime/nccl.zig:214-345, src/runtime/main.zig:132-137).
#include <cooperative_groups.h>
#include <stdio.h>
#include <string.h>

#include "common/util.cuh"
#include "include/ceo_kernels.h"

namespace cg = cooperative_groups;

namespace ceo {

constexpr int MAXR = 8;
#ifndef CEO_PEER_WAIT_LIMIT
#define CEO_PEER_WAIT_LIMIT (1u << 24)
#endif

struct PeerPtrs {
  void* p[MAXR];
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by ONE thread.  Signals `epoch` into slot `slot` of every peer's flag array and waits
// until every peer has signalled this rank.  flags[r] is rank r's array of MAXR*slots words.
__device__ bool peer_barrier(const PeerPtrs& flags, int rank, int world, int slot, unsigned epoch,
                             int* status) {
  __threadfence_system();
  for (int r = 0; r < world; ++r)
    st_release_sys(reinterpret_cast<unsigned*>(flags.p[r]) + slot * MAXR + rank, epoch);
  const unsigned* mine = reinterpret_cast<const unsigned*>(flags.p[rank]) + slot * MAXR;
  bool ok = true;
  for (int r = 0; r < world; ++r) {
    unsigned it = 0;
    // epochs only grow; a signed difference tolerates wrap-around
    while (static_cast<int>(ld_acquire_sys(mine + r) - epoch) < 0) {
      if (++it > CEO_PEER_WAIT_LIMIT) {
        atomicCAS(status, 0, 100 + slot * 10 + r);
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  __threadfence_system();
  return ok;
}

struct ZeroStepArgs {
  PeerPtrs grads;    // float*  full gradient buffers (one per rank)
  PeerPtrs params;   // bf16*   full parameter buffers
  PeerPtrs flags;    // unsigned* flag arrays (4 slots x MAXR)
  PeerPtrs slots;    // float*  MAXR floats per rank: partial squared norms
  float* master;     // this rank's fp32 master slice
  float* m;
  float* v;
  float* local_acc;  // 1 float of local scratch (zeroed by the kernel)
  float* norm_out;
  int* status;
  long long lo, n, total, decay_end;
  int rank, world;
  unsigned epoch;
  float lr, b1, b2, eps, wd, bc1_inv, bc2_inv, gscale, max_norm;
};

__global__ void __launch_bounds__(512)
zero_step_kernel(const ZeroStepArgs a) {
  cg::grid_group grid = cg::this_grid();
  __shared__ float red[33];
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nth = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool leader = (blockIdx.x == 0 && threadIdx.x == 0);

  // ---- barrier 0: every rank has finished its backward pass --------------------------
  if (leader) {
    *a.local_acc = 0.f;
    peer_barrier(a.flags, a.rank, a.world, 0, a.epoch, a.status);
  }
  grid.sync();

  // ---- phase 1: reduce this rank's slice over all ranks, keep the sum locally ----------
  float* gl = reinterpret_cast<float*>(a.grads.p[a.rank]) + a.lo;
  float ss = 0.f;
  const long long n4 = a.n >> 2;
  for (long long i = tid; i < n4; i += nth) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.world; ++r) {
      // L2-only load: peer data must never be served from a stale L1 line
      const float4 g = __ldcg(reinterpret_cast<const float4*>(
                                  reinterpret_cast<const float*>(a.grads.p[r]) + a.lo) + i);
      s.x += g.x; s.y += g.y; s.z += g.z; s.w += g.w;
    }
    reinterpret_cast<float4*>(gl)[i] = s;
    ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  ss = block_reduce_sum(ss, red);
  if (threadIdx.x == 0) atomicAdd(a.local_acc, ss);
  grid.sync();

  // ---- exchange the partial squared norms; barrier 1 also means "all slices reduced" ---
  if (leader) {
    const float mine = *a.local_acc;
    for (int r = 0; r < a.world; ++r)
      reinterpret_cast<volatile float*>(a.slots.p[r])[a.rank] = mine;
    peer_barrier(a.flags, a.rank, a.world, 1, a.epoch, a.status);
  }
  grid.sync();
  float tot = 0.f;
  for (int r = 0; r < a.world; ++r)
    tot += reinterpret_cast<volatile const float*>(a.slots.p[a.rank])[r];
  const float nrm = sqrtf(tot) * a.gscale;
  float clip = 1.f;
  if (a.max_norm > 0.f && nrm > a.max_norm) clip = a.max_norm / (nrm + 1e-6f);
  if (!isfinite(nrm)) clip = 0.f;
  if (leader && a.norm_out) *a.norm_out = nrm;
  const float gs = a.gscale * clip;

  // ---- phase 2: AdamW on the slice; bf16 result stored into every rank's parameters ----
  for (long long i = tid; i < n4; i += nth) {
    const float4 g4 = reinterpret_cast<const float4*>(gl)[i];
    reinterpret_cast<float4*>(gl)[i] = make_float4(0.f, 0.f, 0.f, 0.f);  // consumed: zero it
    float4 m4 = reinterpret_cast<float4*>(a.m)[i];
    float4 v4 = reinterpret_cast<float4*>(a.v)[i];
    float4 p4 = reinterpret_cast<float4*>(a.master)[i];
    const float wd = (a.lo + 4 * i < a.decay_end) ? a.wd : 0.f;
    const float gg[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
    float* mp = reinterpret_cast<float*>(&m4);
    float* vp = reinterpret_cast<float*>(&v4);
    float* pp = reinterpret_cast<float*>(&p4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mp[j] = a.b1 * mp[j] + (1.f - a.b1) * gg[j];
      vp[j] = a.b2 * vp[j] + (1.f - a.b2) * gg[j] * gg[j];
      pp[j] = pp[j] * (1.f - a.lr * wd) -
              a.lr * (mp[j] * a.bc1_inv) / (sqrtf(vp[j] * a.bc2_inv) + a.eps);
    }
    reinterpret_cast<float4*>(a.m)[i] = m4;
    reinterpret_cast<float4*>(a.v)[i] = v4;
    reinterpret_cast<float4*>(a.master)[i] = p4;
    uint2 packed;
    bf162* h = reinterpret_cast<bf162*>(&packed);
    h[0] = __floats2bfloat162_rn(pp[0], pp[1]);
    h[1] = __floats2bfloat162_rn(pp[2], pp[3]);
    for (int r = 0; r < a.world; ++r)
      reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(a.params.p[r]) + a.lo)[i] = packed;
  }
  // every rank is past barrier 1, so nobody reads this rank's gradients any more: zero them
  float4* gz = reinterpret_cast<float4*>(a.grads.p[a.rank]);
  const long long t4 = a.total >> 2;
  // (the owned slice is zeroed above by the thread that consumed it)
  const long long s4 = a.lo >> 2, e4 = (a.lo + a.n) >> 2;
  for (long long i = tid; i < t4; i += nth)
    if (i < s4 || i >= e4) gz[i] = make_float4(0.f, 0.f, 0.f, 0.f);

  // ---- barrier 2: all parameter slices have landed everywhere -------------------------
  grid.sync();
  if (leader) peer_barrier(a.flags, a.rank, a.world, 2, a.epoch, a.status);
  grid.sync();
}

__global__ void symm_barrier_kernel(PeerPtrs flags, int rank, int world, int slot, unsigned epoch,
                                    int* status) {
  if (threadIdx.x == 0) peer_barrier(flags, rank, world, slot, epoch, status);
}

// out[i] = sum_r bufs[r][i] for i < n (small vectors: loss, norms).  Each rank first waits
// until every rank has written its buffer, and leaves only after every rank has read.
__global__ void symm_allreduce_kernel(PeerPtrs bufs, PeerPtrs flags, float* out, int n, int rank,
                                      int world, unsigned epoch, int* status) {
  __shared__ int okflag;
  if (threadIdx.x == 0) okflag = peer_barrier(flags, rank, world, 3, epoch, status) ? 1 : 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += reinterpret_cast<volatile const float*>(bufs.p[r])[i];
    out[i] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) peer_barrier(flags, rank, world, 3, epoch + 1, status);
}

}  // namespace ceo
using namespace ceo;

// ---- raw device memory + IPC plumbing (host side) --------------------------------------
extern "C" int ceo_dev_malloc(void** out, long long bytes) {
  return static_cast<int>(cudaMalloc(out, static_cast<size_t>(bytes)));
}
extern "C" int ceo_dev_free(void* p) { return static_cast<int>(cudaFree(p)); }
extern "C" int ceo_dev_memset(void* p, int value, long long bytes, cudaStream_t stream) {
  return static_cast<int>(cudaMemsetAsync(p, value, static_cast<size_t>(bytes), stream));
}
extern "C" int ceo_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int ceo_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int ceo_ipc_close(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

static void fill_peers(PeerPtrs& d, void* const* src, int world) {
  for (int i = 0; i < MAXR; ++i) d.p[i] = i < world ? src[i] : nullptr;
}

extern "C" int ceo_symm_barrier(void* const* flags, int rank, int world, int slot,
                                unsigned int epoch, int* status, cudaStream_t stream) {
  if (world < 1 || world > MAXR || slot < 0 || slot > 3) return -5;
  PeerPtrs f;
  fill_peers(f, flags, world);
  symm_barrier_kernel<<<1, 32, 0, stream>>>(f, rank, world, slot, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_symm_allreduce(void* const* bufs, void* const* flags, float* out, int n,
                                  int rank, int world, unsigned int epoch, int* status,
                                  cudaStream_t stream) {
  if (world < 1 || world > MAXR || n <= 0) return -5;
  PeerPtrs b, f;
  fill_peers(b, bufs, world);
  fill_peers(f, flags, world);
  symm_allreduce_kernel<<<1, 256, 0, stream>>>(b, f, out, n, rank, world, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_zero_step(void* const* grads, void* const* params, void* const* flags,
                             void* const* slots, float* master, float* m, float* v,
                             float* local_acc, float* norm_out, int* status, long long lo,
                             long long n, long long total, long long decay_end, int rank,
                             int world, unsigned int epoch, float lr, float beta1, float beta2,
                             float eps, float weight_decay, int step, float gscale,
                             float max_norm, cudaStream_t stream) {
  if (world < 1 || world > MAXR || n <= 0 || (n & 3) || (lo & 3) || (total & 3) || step < 1)
    return -5;
  ZeroStepArgs a;
  fill_peers(a.grads, grads, world);
  fill_peers(a.params, params, world);
  fill_peers(a.flags, flags, world);
  fill_peers(a.slots, slots, world);
  a.master = master; a.m = m; a.v = v; a.local_acc = local_acc; a.norm_out = norm_out;
  a.status = status;
  a.lo = lo; a.n = n; a.total = total; a.decay_end = decay_end;
  a.rank = rank; a.world = world; a.epoch = epoch;
  a.lr = lr; a.b1 = beta1; a.b2 = beta2; a.eps = eps; a.wd = weight_decay;
  a.bc1_inv = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  a.bc2_inv = 1.f / (1.f - powf(beta2, static_cast<float>(step)));
  a.gscale = gscale; a.max_norm = max_norm;
  static int grid = 0;
  if (grid == 0) {
    int dev = 0, sms = 0, occ = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, zero_step_kernel, 512, 0);
    if (occ < 1) return -5;
    grid = sms * (occ > 2 ? 2 : occ);
  }
  void* kargs[] = {&a};
  return static_cast<int>(cudaLaunchCooperativeKernel(
      reinterpret_cast<void*>(zero_step_kernel), dim3(grid), dim3(512), kargs, 0, stream));
}

// ---------------------------------------------------------------------------------------
// Context-parallel state exchange: every rank stores its block of `n` floats (the affine map
// (P_r, R_r) of its sequence span, or (Q_r) in backward) into slot `rank` of every peer's
// gather buffer and then joins a flag barrier, all in one launch: when the kernel ends, slot
// s of the local buffer holds rank s's block.  The last CTA to finish its stores runs the
// barrier (a device-wide counter elects it), so no second launch and no host round trip.
namespace ceo {
__global__ void __launch_bounds__(256)
cp_exchange_kernel(const float* __restrict__ src, PeerPtrs dst, PeerPtrs flags, long long n,
                   int rank, int world, unsigned epoch, unsigned* done_counter, int* status) {
  const long long n4 = n >> 2;
  const float4* s4 = reinterpret_cast<const float4*>(src);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = s4[i];
    for (int r = 0; r < world; ++r)
      reinterpret_cast<float4*>(reinterpret_cast<float*>(dst.p[r]) + rank * n)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {  // every CTA of this rank has issued and fenced its stores
      *done_counter = 0;
      peer_barrier(flags, rank, world, 2, epoch, status);
    }
  }
}
}  // namespace ceo

extern "C" int ceo_cp_exchange(const float* src, void* const* gather, void* const* flags,
                               long long n, int rank, int world, unsigned int epoch,
                               unsigned int* done_counter, int* status, cudaStream_t stream) {
  if (world < 1 || world > MAXR || n <= 0 || (n & 3)) return -5;
  PeerPtrs d, f;
  fill_peers(d, gather, world);
  fill_peers(f, flags, world);
  int grid = static_cast<int>((n / 4 + 255) / 256);
  if (grid > 64) grid = 64;
  cp_exchange_kernel<<<grid, 256, 0, stream>>>(src, d, f, n, rank, world, epoch, done_counter,
                                               status);
  return static_cast<int>(cudaGetLastError());
}
