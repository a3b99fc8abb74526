// Collectives fused with their adjacent compute, over peer-mapped memory (NVLink / NVSwitch).
//
// Every rank maps every other rank's communication buffers (CUDA IPC handles, exchanged on
// the host), so one kernel per rank can load from and store to its peers directly:
//
//   zero_step_kernel   gradient reduce-scatter (peer loads, fp32 sum) + global-norm clip +
//                      AdamW or Lion on the rank's fp32 master shard + bf16 parameter
//                      all-gather (peer stores) + gradient zeroing, in ONE cooperative launch.
//   zero_bucket_reduce_kernel   the reduce-scatter of one bucket of parameters, launched on a
//                      side stream as soon as the backward pass has finished that bucket.
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

#include "common/check.cuh"
#include "common/ptx.cuh"
#include "common/util.cuh"
#include "include/ceo_kernels.h"

CEO_BOUNDS_TU(comm)

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
  const unsigned limit = wait_limit(CEO_PEER_WAIT_LIMIT);
  bool ok = true;
  for (int r = 0; r < world; ++r) {
    unsigned it = 0;
    // epochs only grow; a signed difference tolerates wrap-around
    while (static_cast<int>(ld_acquire_sys(mine + r) - epoch) < 0) {
      if (++it > limit) {
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

// One range of the flat parameter space owned rank by rank: rank r owns the elements
// [goff + r * len, goff + (r + 1) * len) of the flat buffers and keeps their fp32 master
// weights and moments at [loff, loff + len) of its shard-local buffers.  `gather`: the updated
// bf16 values are stored into every rank's parameter buffer by the update itself (otherwise
// only into this rank's own; a later all-gather fused into the consuming GEMM moves them).
struct ZRange {
  long long goff, len, loff;
  int gather, pad;
};

constexpr int ZT = 512;  // threads per CTA of the zero-step and bucket-reduce kernels

struct ZeroStepArgs {
  PeerPtrs grads;    // float*  full gradient buffers (one per rank)
  PeerPtrs params;   // bf16*   full parameter buffers
  PeerPtrs flags;    // unsigned* flag arrays (slots x MAXR)
  PeerPtrs slots;    // float*  MAXR floats per rank: partial squared norms
  float* master;     // this rank's fp32 master shard
  float* m;
  float* v;          // AdamW only
  float* local_acc;  // [0] partial squared norm of this rank's shard, [1] scratch
  float* norm_out;
  float* clip_out;   // the clip scale the update used (0 = the step was skipped)
  int* status;
  const ZRange* ranges;
  int nranges;
  long long total, decay_end;
  int rank, world;
  unsigned epoch;
  int kind;        // 0 AdamW, 1 Lion
  int do_reduce;   // 1: reduce the gradients here; 0: zero_bucket_reduce launches did it
  float lr, b1, b2, eps, wd, bc1_inv, bc2_inv, gscale, max_norm;
};

// Sum of every rank's gradients over this rank's slice of ranges [r0, r1), left in this rank's
// own gradient buffer; returns the thread's share of the squared norm of the sums.
// WU = the world size rounded up to 2, 4 or 8.  A thread handles LOADS / WU float4 positions
// per iteration and issues all of their loads (LOADS in flight) before it consumes any: with one load
// in flight per thread the links and HBM idle.  The sum runs in rank order (reproducible).
template <int WU, int LOADS>
__device__ __forceinline__ float reduce_ranges_t(const PeerPtrs& grads, const ZRange* ranges,
                                                 int r0, int r1, int rank, int world,
                                                 long long tid, long long nth) {
  constexpr int NB = LOADS / WU;
  float ss = 0.f;
  for (int ri = r0; ri < r1; ++ri) {
    const ZRange rg = ranges[ri];
    const long long base = rg.goff + rank * rg.len;
    float* gl = reinterpret_cast<float*>(grads.p[rank]) + base;
    const long long n4 = rg.len >> 2;
    // a CTA takes NB * blockDim consecutive positions per iteration: the positions of one
    // thread sit at constant offsets from one another (one address register per stream)
    for (long long i0 = (tid - threadIdx.x) * NB + threadIdx.x; i0 < n4; i0 += nth * NB) {
      float4 g[NB][WU];
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const long long i = i0 + b * ZT;
#pragma unroll
        for (int r = 0; r < WU; ++r)
          if (r < world && i < n4)  // L2-only load: never a stale L1 line of peer data
            g[b][r] = __ldcg(reinterpret_cast<const float4*>(
                                 reinterpret_cast<const float*>(grads.p[r]) + base) + i);
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const long long i = i0 + b * ZT;
        if (i >= n4) break;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < WU; ++r)
          if (r < world) { s.x += g[b][r].x; s.y += g[b][r].y; s.z += g[b][r].z; s.w += g[b][r].w; }
        reinterpret_cast<float4*>(gl)[i] = s;
        ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
      }
    }
  }
  return ss;
}
template <int LOADS>
__device__ __forceinline__ float reduce_ranges(const PeerPtrs& grads, const ZRange* ranges, int r0,
                                               int r1, int rank, int world, long long tid,
                                               long long nth) {
  if (world <= 2) return reduce_ranges_t<2, LOADS>(grads, ranges, r0, r1, rank, world, tid, nth);
  if (world <= 4) return reduce_ranges_t<4, LOADS>(grads, ranges, r0, r1, rank, world, tid, nth);
  return reduce_ranges_t<8, LOADS>(grads, ranges, r0, r1, rank, world, tid, nth);
}

// The optimizer update of this rank's slice of one range (KIND 0 AdamW, 1 Lion).  A thread
// handles two float4 positions per iteration and issues the loads of all four streams of
// both (8 in flight) before it computes; the gradient slice is zeroed as it is consumed.
template <int KIND>
__device__ __forceinline__ void update_range(const ZeroStepArgs& a, const ZRange rg, float gs,
                                             long long tid, long long nth) {
  constexpr int U = 2;
  const long long base = rg.goff + a.rank * rg.len;
  float4* __restrict__ gl = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.grads.p[a.rank]) + base);
  float4* __restrict__ mm = reinterpret_cast<float4*>(a.m + rg.loff);
  float4* __restrict__ vv = reinterpret_cast<float4*>(KIND == 0 ? a.v + rg.loff : nullptr);
  float4* __restrict__ ms = reinterpret_cast<float4*>(a.master + rg.loff);
  const long long n4 = rg.len >> 2;
  const float lr = a.lr, b1 = a.b1, b2 = a.b2;
  // a CTA takes U * ZT consecutive positions per iteration (see reduce_ranges_t)
  for (long long i0 = (tid - threadIdx.x) * U + threadIdx.x; i0 < n4; i0 += nth * U) {
    float4 g4[U], m4[U], v4[U], p4[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * ZT;
      if (i < n4) {
        (void)CEO_IDX(base + 4 * i, a.total - 3, 501);  // the slice stays inside the flat buffers
        g4[u] = gl[i];
        m4[u] = mm[i];
        p4[u] = ms[i];
        if (KIND == 0) v4[u] = vv[i];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * ZT;
      if (i >= n4) break;
      const float decay = 1.f - lr * ((base + 4 * i < a.decay_end) ? a.wd : 0.f);
      const float* gp = reinterpret_cast<const float*>(&g4[u]);
      float* mp = reinterpret_cast<float*>(&m4[u]);
      float* vp = reinterpret_cast<float*>(&v4[u]);
      float* pp = reinterpret_cast<float*>(&p4[u]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g = gp[j] * gs;
        if (KIND == 0) {
          mp[j] = b1 * mp[j] + (1.f - b1) * g;
          vp[j] = b2 * vp[j] + (1.f - b2) * g * g;
          pp[j] = pp[j] * decay - lr * (mp[j] * a.bc1_inv) / (sqrtf(vp[j] * a.bc2_inv) + a.eps);
        } else {
          const float uu = b1 * mp[j] + (1.f - b1) * g;
          pp[j] = pp[j] * decay - lr * (uu > 0.f ? 1.f : (uu < 0.f ? -1.f : 0.f));
          mp[j] = b2 * mp[j] + (1.f - b2) * g;
        }
      }
      gl[i] = make_float4(0.f, 0.f, 0.f, 0.f);  // consumed
      mm[i] = m4[u];
      if (KIND == 0) vv[i] = v4[u];
      ms[i] = p4[u];
      uint2 packed;
      bf162* h = reinterpret_cast<bf162*>(&packed);
      h[0] = __floats2bfloat162_rn(pp[0], pp[1]);
      h[1] = __floats2bfloat162_rn(pp[2], pp[3]);
      if (rg.gather) {
        for (int r = 0; r < a.world; ++r)
          reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(a.params.p[r]) + base)[i] = packed;
      } else {
        reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(a.params.p[a.rank]) + base)[i] = packed;
      }
    }
  }
}

// A skipped step (non-finite norm): the owned gradient slices are dropped, nothing else moves.
__device__ __forceinline__ void zero_owned(const ZeroStepArgs& a, const ZRange rg, long long tid,
                                           long long nth) {
  float4* gl = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.grads.p[a.rank]) + rg.goff +
                                         a.rank * rg.len);
  for (long long i = tid; i < (rg.len >> 2); i += nth) gl[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

__global__ void __launch_bounds__(ZT, 1)
zero_step_kernel(const ZeroStepArgs a) {
  cg::grid_group grid = cg::this_grid();
  __shared__ float red[33];
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nth = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool leader = (blockIdx.x == 0 && threadIdx.x == 0);
  // local_acc[1] carries the leader's verdict on each peer barrier to the whole grid: when a
  // bounded wait ran out (a peer never arrived) nothing below touches master weights,
  // moments, parameters or gradients; the status word says which peer was missing.
  volatile float* okw = a.local_acc + 1;

  // ---- barrier 0: every rank has finished its backward pass --------------------------
  if (leader) {
    if (a.do_reduce) a.local_acc[0] = 0.f;
    // an earlier wait of this step that ran out (a bucket reduction's barrier) stops the step
    const bool clean = *reinterpret_cast<volatile int*>(a.status) == 0;
    const bool ok = clean && peer_barrier(a.flags, a.rank, a.world, 0, a.epoch, a.status);
    *okw = ok ? 1.f : 0.f;
  }
  grid.sync();
  if (*okw == 0.f) return;

  // ---- phase 1: reduce this rank's slices over all ranks, keep the sums locally ---------
  if (a.do_reduce) {
    float ss = reduce_ranges<8>(a.grads, a.ranges, 0, a.nranges, a.rank, a.world, tid, nth);
    ss = block_reduce_sum(ss, red);
    if (threadIdx.x == 0) atomicAdd(a.local_acc, ss);
  }
  grid.sync();

  // ---- exchange the partial squared norms; barrier 1 also means "all slices reduced" ---
  if (leader) {
    const float mine = a.local_acc[0];
    a.local_acc[0] = 0.f;  // ready for the next step's bucket reductions
    for (int r = 0; r < a.world; ++r)
      reinterpret_cast<volatile float*>(a.slots.p[r])[a.rank] = mine;
    const bool ok = peer_barrier(a.flags, a.rank, a.world, 1, a.epoch, a.status);
    *okw = ok ? 1.f : 0.f;
  }
  grid.sync();
  if (*okw == 0.f) return;
  float tot = 0.f;
  for (int r = 0; r < a.world; ++r)
    tot += reinterpret_cast<volatile const float*>(a.slots.p[a.rank])[r];
  const float nrm = sqrtf(tot) * a.gscale;
  float clip = 1.f;
  if (a.max_norm > 0.f && nrm > a.max_norm) clip = a.max_norm / (nrm + 1e-6f);
  // a non-finite norm skips the step: states and parameters stay, gradients are dropped
  const bool skip = !isfinite(nrm);
  if (skip) clip = 0.f;
  if (leader) {
    if (a.norm_out) *a.norm_out = nrm;
    if (a.clip_out) *a.clip_out = clip;
  }
  const float gs = a.gscale * clip;

  // ---- phase 2: update the slices; bf16 results stored into the parameter buffers --------
  for (int ri = 0; ri < a.nranges; ++ri) {
    if (skip) zero_owned(a, a.ranges[ri], tid, nth);
    else if (a.kind == 0) update_range<0>(a, a.ranges[ri], gs, tid, nth);
    else update_range<1>(a, a.ranges[ri], gs, tid, nth);
  }
  // every rank is past barrier 1, so nobody reads this rank's gradients any more: zero the
  // parts other ranks own (the owned slices were zeroed above by the threads that read them)
  float4* gz = reinterpret_cast<float4*>(a.grads.p[a.rank]);
  for (int ri = 0; ri < a.nranges; ++ri) {
    const ZRange rg = a.ranges[ri];
    const long long s4 = rg.goff >> 2, n4 = (rg.len * a.world) >> 2;
    const long long o4 = (a.rank * rg.len) >> 2, l4 = rg.len >> 2;
    for (long long i = tid; i < n4; i += nth)
      if (i < o4 || i >= o4 + l4)
        gz[CEO_IDX(s4 + i, a.total >> 2, 502)] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  // ---- barrier 2: all parameter slices have landed everywhere -------------------------
  grid.sync();
  if (leader) peer_barrier(a.flags, a.rank, a.world, 2, a.epoch, a.status);
  grid.sync();
}

// Gradient reduce-scatter of one bucket of ranges, launched on a side stream while the rest
// of the backward pass still runs: the sums land in this rank's own gradient buffer and their
// squared norm is added to local_acc[0].  The launch is preceded by a flag barrier (its own
// kernel on the same stream) that tells every rank the bucket's gradients are final
// everywhere; when that barrier's wait ran out the status word is set and nothing is reduced.
__global__ void __launch_bounds__(ZT)
zero_bucket_reduce_kernel(PeerPtrs grads, const ZRange* ranges, int r0, int r1, int rank,
                          int world, float* local_acc, const int* status) {
  __shared__ float red[33];
  if (*reinterpret_cast<const volatile int*>(status) != 0) return;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nth = static_cast<long long>(gridDim.x) * blockDim.x;
  float ss = reduce_ranges<8>(grads, ranges, r0, r1, rank, world, tid, nth);
  ss = block_reduce_sum(ss, red);
  if (threadIdx.x == 0) atomicAdd(local_acc, ss);
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
  if (world < 1 || world > MAXR || slot < 0 || slot > 7) return -5;
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
                             float* local_acc, float* norm_out, float* clip_out, int* status,
                             const void* ranges, int nranges, long long total,
                             long long decay_end, int rank, int world, unsigned int epoch,
                             int kind, int do_reduce, float lr, float beta1, float beta2,
                             float eps, float weight_decay, int step, float gscale,
                             float max_norm, int max_ctas, cudaStream_t stream) {
  if (world < 1 || world > MAXR || nranges <= 0 || (total & 3) || step < 1 || kind < 0 ||
      kind > 1 || (kind == 0 && !v))
    return -5;
  ZeroStepArgs a;
  fill_peers(a.grads, grads, world);
  fill_peers(a.params, params, world);
  fill_peers(a.flags, flags, world);
  fill_peers(a.slots, slots, world);
  a.master = master; a.m = m; a.v = v; a.local_acc = local_acc; a.norm_out = norm_out;
  a.clip_out = clip_out;
  a.status = status;
  a.ranges = static_cast<const ZRange*>(ranges); a.nranges = nranges;
  a.total = total; a.decay_end = decay_end;
  a.rank = rank; a.world = world; a.epoch = epoch;
  a.kind = kind; a.do_reduce = do_reduce;
  a.lr = lr; a.b1 = beta1; a.b2 = beta2; a.eps = eps; a.wd = weight_decay;
  a.bc1_inv = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  a.bc2_inv = 1.f / (1.f - powf(beta2, static_cast<float>(step)));
  a.gscale = gscale; a.max_norm = max_norm;
  static int full_grid = 0;
  if (full_grid == 0) {
    int dev = 0, sms = 0, occ = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, zero_step_kernel, 512, 0);
    if (occ < 1) return -5;
    full_grid = sms * (occ > 2 ? 2 : occ);  // one CTA of 16 warps per SM at 128 registers
  }
  int grid = full_grid;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  void* kargs[] = {&a};
  return static_cast<int>(cudaLaunchCooperativeKernel(
      reinterpret_cast<void*>(zero_step_kernel), dim3(grid), dim3(512), kargs, 0, stream));
}

// Flag barrier (slot 4) + reduce-scatter of ranges [r0, r1) on `stream` (see
// zero_bucket_reduce_kernel).  `ctas` bounds the grid so the reduction shares the GPU with
// the backward pass it overlaps.
extern "C" int ceo_zero_bucket_reduce(void* const* grads, void* const* flags, const void* ranges,
                                      int r0, int r1, int rank, int world, unsigned int epoch,
                                      float* local_acc, int* status, int ctas,
                                      cudaStream_t stream) {
  if (world < 1 || world > MAXR || r0 < 0 || r1 <= r0) return -5;
  PeerPtrs g, f;
  fill_peers(g, grads, world);
  fill_peers(f, flags, world);
  symm_barrier_kernel<<<1, 32, 0, stream>>>(f, rank, world, 4, epoch, status);
  if (ctas <= 0) ctas = 32;
  zero_bucket_reduce_kernel<<<ctas, 512, 0, stream>>>(g, static_cast<const ZRange*>(ranges), r0,
                                                      r1, rank, world, local_acc, status);
  return static_cast<int>(cudaGetLastError());
}

// Run-time override of every bounded wait's iteration limit in the library (0 restores the
// compile-time defaults).  Tests use a small value to make a wait that nothing will ever
// satisfy run out quickly; production code never calls this.
extern "C" int ceo_gemm_set_wait_limit(unsigned int iterations);
extern "C" int ceo_efla_set_wait_limit(unsigned int iterations);
extern "C" int ceo_set_wait_limit(unsigned int iterations) {
  int rc = set_wait_limit_override(iterations);
  if (rc == 0) rc = ceo_gemm_set_wait_limit(iterations);
  if (rc == 0) rc = ceo_efla_set_wait_limit(iterations);
  return rc;
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


// ---------------------------------------------------------------------------------------
// out[b] = P[b] s[b] + R[b]  (or P[b]^T s[b] + R[b]) for `nb` independent d x d fp32 matrices:
// one step of folding a rank's affine state map onto the incoming state in context
// parallelism.  fp32 on purpose (the maps compose over up to 8 ranks); the matrices are tiny
// (d <= 128), so a 16 x 16 shared-memory tiling per CTA is enough.
namespace ceo {
__global__ void __launch_bounds__(256)
fold_affine_kernel(const float* __restrict__ P, const float* __restrict__ s,
                   const float* __restrict__ R, float* __restrict__ out, int d, int transpose) {
  __shared__ float ps[16][17], ss[16][17];
  const int tiles = d / 16;
  const int b = blockIdx.x / (tiles * tiles), t = blockIdx.x % (tiles * tiles);
  const int ti = t / tiles, tj = t % tiles, ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const long long base = static_cast<long long>(b) * d * d;
  const int row = ti * 16 + ty, col = tj * 16 + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < d; k0 += 16) {
    // ps[ty][tx] = Pm[row][k0 + tx] with Pm = P or P^T
    ps[ty][tx] = transpose ? P[base + static_cast<long long>(k0 + tx) * d + ti * 16 + ty]
                           : P[base + static_cast<long long>(row) * d + k0 + tx];
    ss[ty][tx] = s[base + static_cast<long long>(k0 + ty) * d + col];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) acc += ps[ty][k] * ss[k][tx];
    __syncthreads();
  }
  out[base + static_cast<long long>(row) * d + col] = acc + R[base + static_cast<long long>(row) * d + col];
}
}  // namespace ceo

extern "C" int ceo_fold_affine(const float* P, const float* s, const float* R, float* out, int nb,
                               int d, int transpose, cudaStream_t stream) {
  if (nb <= 0 || d <= 0 || (d & 15)) return -5;
  const int tiles = d / 16;
  fold_affine_kernel<<<nb * tiles * tiles, 256, 0, stream>>>(P, s, R, out, d, transpose);
  return static_cast<int>(cudaGetLastError());
}
