// bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma with
// fp32 accumulators in TMEM -> tcgen05.ld epilogue with fused scale / bias /
// residual / accumulate and bf16 or fp32 store.
//
// Persistent kernel, one CTA per SM, warp-specialised:
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation + MMA issue (one lane)
//   warps 2..5  epilogue (each owns one 32-lane TMEM quadrant)
// Two 128x256 fp32 accumulators (all 512 TMEM columns) are double-buffered so
// the epilogue of tile i overlaps the main loop of tile i+1.
//
// Replaces the library GEMM + separate bias / column-sum kernels of the
// reference (kernels/cuda/gemm.cu:182-234, 50-72) with one fused kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "common/check.cuh"
#include "common/ptx.cuh"
#include "include/ceo_kernels.h"

CEO_BOUNDS_TU(gemm)

namespace ceo {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int PANEL_BYTES = 64 * BK * 2;  // one 64-wide MN-major panel, 8 KB
constexpr int GEMM_THREADS = 192;
constexpr int EPI_ROW_BYTES = 144;  // 64 bf16 + 16 B pad: conflict-free 16-byte accesses
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int ACT_ROW_BYTES = 80;  // 32 bf16 + 16 B pad
constexpr int ACT_WARP_BYTES = 32 * ACT_ROW_BYTES;
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ +
                          4 * EPI_WARP_BYTES /*store staging*/ + 4 * ACT_WARP_BYTES /*SwiGLU*/;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t AG_CHUNK = 32768;                             // bytes per bulk copy
constexpr int AG_RING = (STAGES * STAGE_BYTES) / AG_CHUNK;       // 6 buffers of 32 KB
constexpr int AG_RING_BAR = 16;  // mbarriers of the copy-first mode (the pipeline's stay untouched)

struct GemmParams {
  void* C;
  const void* residual;  // same dtype/layout family as C (bf16), optional
  const float* bias;     // fp32 [N], optional
  int M, N, K;
  long long ldc, ldr;
  long long batch_stride_c, batch_stride_r;
  int batch;
  int out_f32;     // 1: C is fp32, 0: C is bf16
  int accumulate;  // C = alpha*acc + C
  float alpha;
  // 8-bit float operands (K-major only): element formats (0 e4m3, 1 e5m2) and the device-side
  // quantisation scales; the epilogue multiplies by alpha / (scale_a * scale_b)
  int fp8_a, fp8_b;
  const float* scale_a;
  const float* scale_b;
  int num_m, num_n;
  int* status;
  // ---- collectives fused into the kernel (all zero for a plain GEMM) --------------------
  int m_rot, n_rot;        // tile traversal starts at this m / n block (local data first)
  int grp_m;               // row blocks per traversal group (see tile_coords)
  int split_k;             // >1: k-slices of a tile accumulate into fp32 C with atomics
  int a_4d, b_4d;          // M/N-major operand mapped as (64, k, panel, batch): one TMA per stage
  // all-gather of one operand: the first `ag_ctas` CTAs pull the peers' row-shards into
  // the local gathered buffer (which the tensor map reads) and publish one flag per block
  // of BM (A) or BN (B) rows; the TMA producer waits for a block's flag before loading it.
  int ag_operand;          // 0 none, 1 A, 2 B
  int ag_ctas;
  int ag_all;  // 1: every CTA copies its share of the peers' shards first, then computes
  int ag_rows_per_shard;   // rows of the gathered operand owned by each rank
  int ag_blk_rows;         // rows per flag (a divisor of ag_rows_per_shard)
  long long ag_row_bytes;  // bytes per row (dense rows)
  const void* ag_src[8];   // rank r's shard, as mapped on this rank (entry `rank` unused)
  void* ag_dst;            // local gathered buffer
  unsigned* ag_flags;      // local, one per row block, counts up by 1 per call
  unsigned ag_target;
  // a second tensor gathered by the same copy CTAs after the operand (no flags: it is complete
  // when the kernel ends); rank r's shard of it is ag_extra_bytes at ag_extra_src[r]
  const void* ag_extra_src[8];
  void* ag_extra_dst;      // local buffer, shard r at r * ag_extra_bytes
  long long ag_extra_bytes;
  // reduce-scatter of C over M: the epilogue stores each partial tile into the staging
  // area of the rank that owns those rows and bumps a counter there; after its last tile a
  // CTA reduces its share of this rank's own rows from the staged partials of all ranks.
  int rs_on;
  int rs_rows_per_rank;
  void* rs_stage[8];       // rank j's staging: [world][rows_per_rank][N] bf16
  unsigned* rs_count[8];   // rank j's counters: [world][rows_per_rank / BM]
  unsigned rs_target;      // counter value that means "all tiles of this call arrived"
  void* rs_out;            // bf16 [rows_per_rank][N], ld = rs_ldo
  const void* rs_residual; // optional bf16, same shape/ld as rs_out
  long long rs_ldo;
  int rank, world;
  // SwiGLU fused into the epilogue (bf16 C, K-major or MN-major operands alike):
  //   1  C holds gate/up in INTERLEAVED columns (2j = gate_j, 2j+1 = up_j); besides C the
  //      epilogue writes act[:, j] = silu(gate_j) * up_j into aux (M x N/2, ld_aux)
  //   2  the accumulator is d(act) (M x N); aux is the saved interleaved gate/up (M x 2N,
  //      ld_aux); C receives the interleaved d(gate/up) (M x 2N, ldc) and d(act) never
  //      goes to memory
  int epi_mode;
  void* aux;
  long long ld_aux;
};

enum : int { ST_PRODUCER = 1, ST_MMA_FULL = 2, ST_MMA_TMEM = 3, ST_EPILOGUE = 4, ST_AG_WAIT = 5,
             ST_RS_WAIT = 6, ST_COPY = 7 };

// Tile r of a batch -> (m block, n block).  m runs fastest inside a group of `grp_m` row
// blocks and a group is finished (all n blocks) before the next one starts; groups and n
// blocks are visited starting at m_rot / n_rot.  With grp_m = num_m this is plain m-fastest
// order; with grp_m = row blocks per rank the kernel works through one rank's rows at a time
// (local rows first for an all-gathered A, the other ranks' rows first for a reduce-scatter).
__device__ __forceinline__ void tile_coords(const GemmParams& p, int r, int& m_blk, int& n_blk) {
  if (p.rs_on) {
    // reduce-scatter: stripe by stripe (the lb-th row block of EVERY owner, the other ranks'
    // first), so that all partials of a stripe arrive everywhere within one stripe's time and
    // the reducer CTAs work through the stripes while later ones are still being computed
    const int bpr = p.rs_rows_per_rank / BM;
    const int per_stripe = p.world * p.num_n;
    const int lb = r / per_stripe, rem = r - lb * per_stripe;
    const int oi = rem / p.num_n;
    n_blk = rem - oi * p.num_n;
    m_blk = ((p.rank + 1 + oi) % p.world) * bpr + lb;
    return;
  }
  const int per_group = p.grp_m * p.num_n;
  const int g = r / per_group, rem = r - g * per_group;
  const int left = p.num_m - g * p.grp_m;           // the last group may be narrower
  const int gsz = left < p.grp_m ? left : p.grp_m;
  m_blk = (g * p.grp_m + rem % gsz + p.m_rot) % p.num_m;
  n_blk = (rem / gsz + p.n_rot) % p.num_n;
}

// Reducer CTAs of the GEMM -> reduce-scatter kernel.  Work item = one (row block, 256-column
// block) of the rows this rank owns, in stripe order (the order the partial tiles are produced
// in everywhere); an item is ready when every source rank's counter for its row block has
// reached the target.  A warp takes 8 rows of an item at a time and keeps RU rows x W sources
// of 16-byte loads in flight per lane (W x RU = 16): with few CTAs reducing, memory-level
// parallelism per CTA is what bounds the reduction.
template <int W, int RU>
__device__ __forceinline__ void rs_reduce(const GemmParams& p, int warp, int lane) {
  const int bpr = p.rs_rows_per_rank / BM;
  const int items = bpr * p.num_n;
  const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(p.rs_stage[p.rank]);
  const __nv_bfloat16* resid = reinterpret_cast<const __nv_bfloat16*>(p.rs_residual);
  __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.rs_out);
  const unsigned* cnt = p.rs_count[p.rank];
  constexpr int GROUP = 8, GPI = BM / GROUP, WARPS = GEMM_THREADS / 32;
  const int my_items = static_cast<int>(blockIdx.x) < items
                           ? (items - static_cast<int>(blockIdx.x) + p.ag_ctas - 1) / p.ag_ctas
                           : 0;
  int ready_item = -1;
  const int c = lane * 8;  // a warp covers one 256-column row segment per row
  for (int u = warp; u < my_items * GPI; u += WARPS) {
    const int item = static_cast<int>(blockIdx.x) + (u / GPI) * p.ag_ctas, grp = u % GPI;
    const int lb = item / p.num_n, nb = item - lb * p.num_n;
    if (item != ready_item) {
      for (int src = 0; src < p.world; ++src)
        if (!flag_wait_ge<true>(cnt + src * bpr + lb, p.rs_target)) {
          if (lane == 0) atomicCAS(p.status, 0, ST_RS_WAIT);
          return;
        }
      ready_item = item;
    }
    if (c >= min(BN, p.N - nb * BN)) continue;
#pragma unroll 1
    for (int rr = 0; rr < GROUP; rr += RU) {
      const int row0 = lb * BM + grp * GROUP + rr;  // rows within this rank's slice
      uint4 part[RU][W];
      uint4 resv[RU];
#pragma unroll
      for (int q = 0; q < RU; ++q) {
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < p.world)
            part[q][src] = __ldcg(reinterpret_cast<const uint4*>(
                stage + CEO_IDX((static_cast<long long>(src) * p.rs_rows_per_rank + row0 + q) * p.ldc +
                                    nb * BN + c,
                                static_cast<long long>(p.world) * p.rs_rows_per_rank * p.ldc - 7, 406)));
        if (resid)
          resv[q] = *reinterpret_cast<const uint4*>(resid + (row0 + q) * p.rs_ldo + nb * BN + c);
      }
#pragma unroll
      for (int q = 0; q < RU; ++q) {
        float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < p.world) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&part[q][src]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 x = __bfloat1622float2(h[j]);
              acc8[2 * j] += x.x;
              acc8[2 * j + 1] += x.y;
            }
          }
        if (resid) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&resv[q]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 x = __bfloat1622float2(h[j]);
            acc8[2 * j] += x.x;
            acc8[2 * j + 1] += x.y;
          }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc8[2 * j], acc8[2 * j + 1]);
        *reinterpret_cast<uint4*>(
            outp + CEO_IDX((row0 + q) * p.rs_ldo + nb * BN + c,
                           static_cast<long long>(p.rs_rows_per_rank - 1) * p.rs_ldo + p.N - 7, 407)) = o;
      }
    }
  }
}

// FP8 = 1: both operands are K-major 8-bit floats; a stage row is still 128 bytes, i.e. 128
// elements of K, and one MMA covers 32 of them.
// Copy-first all-gather (one thread per CTA): the peers' shards of the gathered operand and of
// the extra tensor are cut into 32 KB chunks, interleaved over the peers and dealt round-robin
// to ALL CTAs of the grid; each CTA moves its few chunks peer -> shared memory -> local buffer
// through the (still empty) pipeline stages with bulk async copies, then adds 1 to the launch's
// counter.  With ~150 CTAs x 6 chunks in flight the gather runs at link rate and is over
// within the first tiles, which are the local shard's; a producer waits for the counter once,
// before its first tile with remote rows.
__device__ __forceinline__ bool ag_copy_all(const GemmParams& p, uint8_t* smem, uint64_t* rbar) {
  const int cn = static_cast<int>(gridDim.x), ci = static_cast<int>(blockIdx.x);
  const long long shard_bytes = p.ag_rows_per_shard * p.ag_row_bytes;
  const int cpp = static_cast<int>((shard_bytes + AG_CHUNK - 1) / AG_CHUNK);
  const int xpp = static_cast<int>((p.ag_extra_bytes + AG_CHUNK - 1) / AG_CHUNK);
  const int peers = p.world - 1;
  const int nchunks = peers * (cpp + xpp);
  const int mine = ci < nchunks ? (nchunks - ci + cn - 1) / cn : 0;
  auto locate = [&](int i, const uint8_t*& src, uint8_t*& dst, uint32_t& nb) {
    const int g = ci + i * cn;
    const int peer = (p.rank + 1 + g % peers) % p.world;
    int c = g / peers;
    long long off, left;
    if (c < cpp) {
      off = static_cast<long long>(c) * AG_CHUNK;
      left = shard_bytes - off;
      src = reinterpret_cast<const uint8_t*>(p.ag_src[peer]) + off;
      dst = reinterpret_cast<uint8_t*>(p.ag_dst) + peer * shard_bytes + off;
    } else {
      off = static_cast<long long>(c - cpp) * AG_CHUNK;
      left = p.ag_extra_bytes - off;
      src = reinterpret_cast<const uint8_t*>(p.ag_extra_src[peer]) + off;
      dst = reinterpret_cast<uint8_t*>(p.ag_extra_dst) + peer * p.ag_extra_bytes + off;
    }
    nb = static_cast<uint32_t>(left < AG_CHUNK ? left : AG_CHUNK);
  };
  uint32_t ring_ph = 0;
  int issued = 0;
  bool ok = true;
  for (int done = 0; done < mine && ok; ++done) {
    while (issued < mine && issued < done + AG_RING) {
      if (issued >= AG_RING) bulk_wait_read<0>();  // the ring slot's last store has read it
      const uint8_t* src; uint8_t* dst; uint32_t nb;
      locate(issued, src, dst, nb);
      const int slot = issued % AG_RING;
      mbar_arrive_expect_tx(&rbar[slot], nb);
      bulk_load(smem + slot * AG_CHUNK, src, nb, &rbar[slot]);
      ++issued;
    }
    const uint8_t* src; uint8_t* dst; uint32_t nb;
    locate(done, src, dst, nb);
    const int slot = done % AG_RING;
    if (!mbar_wait(&rbar[slot], (ring_ph >> slot) & 1)) {
      atomicCAS(p.status, 0, ST_COPY);
      ok = false;
      break;
    }
    ring_ph ^= 1u << slot;
    fence_proxy_async_smem();
    bulk_store(dst, smem + slot * AG_CHUNK, nb);
    bulk_commit();
  }
  if (!ok) for (int i = 0; i < 200; ++i) __nanosleep(1000);
  bulk_wait<0>();  // every byte is in local memory, and the stages are free for the pipeline
  fence_proxy_async_all();
  __threadfence();
  if (ok) atomicAdd(p.ag_flags, 1u);
  return ok;
}

template <int A_MN, int B_MN, int FP8 = 0>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128B swizzle atom (8 rows x 128 B).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    if (p.ag_all)
      for (int i = 0; i < AG_RING; ++i) mbar_init(&bars[AG_RING_BAR + i], 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_batch = p.num_m * p.num_n;
  const int total_tiles = tiles_per_batch * p.batch;
  constexpr int BKE = FP8 ? 2 * BK : BK;  // elements of K per stage
  const int num_kb = (p.K + BKE - 1) / BKE;
  // the first ag_ctas CTAs are helpers: they copy (all-gather) or reduce (reduce-scatter);
  // the others walk the output tiles
  const bool copy_cta = static_cast<int>(blockIdx.x) < p.ag_ctas;
  const int tile_step = static_cast<int>(gridDim.x) - p.ag_ctas;
  // split-K: a work unit is (k-slice, tile); slices of one tile accumulate into C with atomics
  const int total_units = total_tiles * p.split_k;
  const int kb_per_split = (num_kb + p.split_k - 1) / p.split_k;
  const int first_tile = copy_cta ? total_units : static_cast<int>(blockIdx.x) - p.ag_ctas;

  if (p.rs_on && copy_cta) {
    // ------------------------------------------------ reduce-scatter: reducer CTA
    // All six warps reduce this rank's own rows from the staged partial tiles, item by item in
    // stripe order, while the other CTAs compute.
    if (p.world <= 2) rs_reduce<2, 8>(p, warp, lane);
    else if (p.world <= 4) rs_reduce<4, 4>(p, warp, lane);
    else rs_reduce<8, 2>(p, warp, lane);
  } else if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      bool all_ready = false;
      if (p.ag_all) ok = ag_copy_all(p, smem, bars + AG_RING_BAR);
      for (int t = first_tile; t < total_units && ok; t += tile_step) {
        const int ks = t / total_tiles, tt = t - ks * total_tiles;
        const int kb0 = ks * kb_per_split, kb1 = min(num_kb, kb0 + kb_per_split);
        const int b = tt / tiles_per_batch;
        const int r = tt - b * tiles_per_batch;
        int mb_, nb_;
        tile_coords(p, r, mb_, nb_);
        const int m0 = mb_ * BM, n0 = nb_ * BN;
        if (p.ag_operand) {
          // rows pulled from a peer become loadable once the copy CTAs have published them
          const int row0 = p.ag_operand == 1 ? m0 : n0;
          const int rows = p.ag_operand == 1 ? p.M : p.N;
          const int row1 = min(rows, row0 + (p.ag_operand == 1 ? BM : BN));
          const int bps = p.ag_rows_per_shard / p.ag_blk_rows;
          bool waited = false;
          if (p.ag_all) {
            // copy-first mode: one counter says every CTA has landed its share
            const int own0 = p.rank * p.ag_rows_per_shard;
            if (!all_ready && (row0 < own0 || row1 > own0 + p.ag_rows_per_shard)) {
              if (!flag_wait_ge<false>(p.ag_flags, gridDim.x)) {
                atomicCAS(p.status, 0, ST_AG_WAIT);
                ok = false;
              }
              all_ready = waited = true;
            }
          } else
          for (int blk = row0 / p.ag_blk_rows; blk * p.ag_blk_rows < row1 && ok; ++blk) {
            if (blk / bps == p.rank) continue;
            waited = true;
            if (!flag_wait_ge<false>(p.ag_flags + blk, p.ag_target)) {
              atomicCAS(p.status, 0, ST_AG_WAIT);
              ok = false;
            }
          }
          if (!ok) break;
          if (waited) fence_proxy_async_all();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            atomicCAS(p.status, 0, ST_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
          const int k0 = kb * BKE;
          if (A_MN == 0) {
            tma_load_3d(sa, &tmA, &full_bar[s], k0, m0, b);
          } else if (p.a_4d) {
            tma_load_4d(sa, &tmA, &full_bar[s], 0, k0, m0 / 64, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sa + j * PANEL_BYTES, &tmA, &full_bar[s], m0 + j * 64, k0, b);
          }
          if (B_MN == 0) {
            tma_load_3d(sb, &tmB, &full_bar[s], k0, n0, b);
          } else if (p.b_4d) {
            tma_load_4d(sb, &tmB, &full_bar[s], 0, k0, n0 / 64, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * PANEL_BYTES, &tmB, &full_bar[s], n0 + j * 64, k0, b);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {
        // let any copy still in flight land before the CTA's shared memory goes away
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
      }
      if (copy_cta && p.ag_operand) {
        // ---------------------------------------------------- all-gather copy CTA
        // Pulls row blocks of the peers' shards through a ring of shared-memory buffers with
        // bulk async copies (peer -> smem -> local gathered buffer), nearest peer first, and
        // publishes a block's flag once its bytes have landed in local memory.
        const int blk_rows = p.ag_blk_rows;
        const int blks_per_shard = p.ag_rows_per_shard / blk_rows;
        const long long blk_bytes = p.ag_row_bytes * blk_rows;
        constexpr uint32_t CHUNK = 32768;
        constexpr int RING = (STAGES * STAGE_BYTES) / CHUNK;  // 6 buffers of 32 KB
        const int cpb = static_cast<int>((blk_bytes + CHUNK - 1) / CHUNK);  // chunks per block
        const int my_blks = static_cast<int>(blockIdx.x) < blks_per_shard
                                ? (blks_per_shard - static_cast<int>(blockIdx.x) + p.ag_ctas - 1) /
                                      p.ag_ctas
                                : 0;
        const int per_peer = my_blks * cpb;
        const int total_main = (p.world - 1) * per_peer;
        // the extra tensor: 32 KB chunks of every peer's shard, dealt round-robin to the copy CTAs
        const int xchunks = static_cast<int>((p.ag_extra_bytes + CHUNK - 1) / CHUNK);
        const int per_peer_x = static_cast<int>(blockIdx.x) < xchunks
                                   ? (xchunks - static_cast<int>(blockIdx.x) + p.ag_ctas - 1) / p.ag_ctas
                                   : 0;
        const int total = total_main + (p.world - 1) * per_peer_x;
        uint32_t ring_ph = 0;  // bit i = phase of ring barrier i (bars[0..RING) are count-1)
        // chunk idx -> peer (nearest first), block, byte offset
        auto locate = [&](int idx, const uint8_t*& src, uint8_t*& dst, uint32_t& nb, int& flag,
                          bool& last) {
          if (idx >= total_main) {
            const int e = idx - total_main;
            const int peer = (p.rank + 1 + e / per_peer_x) % p.world;
            const long long off =
                (static_cast<long long>(blockIdx.x) + static_cast<long long>(e % per_peer_x) * p.ag_ctas) *
                CHUNK;
            const long long left = p.ag_extra_bytes - off;
            nb = static_cast<uint32_t>(left < CHUNK ? left : CHUNK);
            src = reinterpret_cast<const uint8_t*>(p.ag_extra_src[peer]) + off;
            dst = reinterpret_cast<uint8_t*>(p.ag_extra_dst) + peer * p.ag_extra_bytes + off;
            flag = 0;
            last = false;
            return;
          }
          const int peer = (p.rank + 1 + idx / per_peer) % p.world;
          const int rem = idx % per_peer;
          const int bi = static_cast<int>(blockIdx.x) + (rem / cpb) * p.ag_ctas;
          const long long off = static_cast<long long>(bi) * blk_bytes +
                                static_cast<long long>(rem % cpb) * CHUNK;
          const long long left = static_cast<long long>(bi + 1) * blk_bytes - off;
          nb = static_cast<uint32_t>(left < CHUNK ? left : CHUNK);
          src = reinterpret_cast<const uint8_t*>(p.ag_src[peer]) + off;
          dst = reinterpret_cast<uint8_t*>(p.ag_dst) +
                static_cast<long long>(peer) * p.ag_rows_per_shard * p.ag_row_bytes + off;
          flag = peer * blks_per_shard + bi;
          last = (rem % cpb) == cpb - 1;
        };
        int issued = 0;
        bool cok = true;
        for (int done = 0; done < total && cok; ++done) {
          while (issued < total && issued < done + RING) {
            if (issued >= RING) bulk_wait_read<0>();  // the ring slot's last store has read it
            const uint8_t* src; uint8_t* dst; uint32_t nb; int flag; bool last;
            locate(issued, src, dst, nb, flag, last);
            const int slot = issued % RING;
            mbar_arrive_expect_tx(&bars[slot], nb);
            bulk_load(smem + slot * CHUNK, src, nb, &bars[slot]);
            ++issued;
          }
          const uint8_t* src; uint8_t* dst; uint32_t nb; int flag; bool last;
          locate(done, src, dst, nb, flag, last);
          const int slot = done % RING;
          if (!mbar_wait(&bars[slot], (ring_ph >> slot) & 1)) {
            atomicCAS(p.status, 0, ST_COPY);
            cok = false;
            break;
          }
          ring_ph ^= 1u << slot;
          fence_proxy_async_smem();
          bulk_store(dst, smem + slot * CHUNK, nb);
          bulk_commit();
          if (last) {
            bulk_wait<0>();  // every byte of this block is in local memory
            fence_proxy_async_all();
            __threadfence();
            st_release_gpu(p.ag_flags + flag, p.ag_target);
          }
        }
        if (!cok) for (int i = 0; i < 200; ++i) __nanosleep(1000);
        bulk_wait<0>();
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = FP8 ? umma_idesc_f8(BM, BN, p.fp8_a, p.fp8_b)
                                 : umma_idesc_bf16(BM, BN, A_MN, B_MN);
      const uint32_t smem0 = smem_u32(smem);
      const uint64_t adesc0 = A_MN ? umma_smem_desc(smem0, PANEL_BYTES, 1024)
                                   : umma_smem_desc(smem0, 16, 1024);
      const uint64_t bdesc0 = B_MN ? umma_smem_desc(smem0 + A_STAGE_BYTES, PANEL_BYTES, 1024)
                                   : umma_smem_desc(smem0 + A_STAGE_BYTES, 16, 1024);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = first_tile; t < total_units && ok; t += tile_step, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        const int kb0 = (t / total_tiles) * kb_per_split, kb1 = min(num_kb, kb0 + kb_per_split);
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1)) {
          atomicCAS(p.status, 0, ST_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[s], ph)) {
            atomicCAS(p.status, 0, ST_MMA_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          // descriptors of the stage's first k-step; the next ones differ only in the start
          // address field (16-byte units in the low 14 bits, which cannot carry: shared
          // memory addresses stay below 256 KB)
          const uint64_t ad0 = adesc0 + static_cast<uint64_t>(s) * (STAGE_BYTES >> 4);
          const uint64_t bd0 = bdesc0 + static_cast<uint64_t>(s) * (STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = ad0 + static_cast<uint64_t>(k) * ((A_MN ? 2048 : 32) >> 4);
            const uint64_t bd = bd0 + static_cast<uint64_t>(k) * ((B_MN ? 2048 : 32) >> 4);
            const uint32_t accf = (kb > kb0 || k != 0) ? 1u : 0u;
            if (FP8) umma_f8(d_tmem, ad, bd, idesc, accf);
            else umma_f16(d_tmem, ad, bd, idesc, accf);
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    const float alpha = (FP8 && p.scale_a) ? p.alpha / (__ldg(p.scale_a) * __ldg(p.scale_b))
                                           : p.alpha;
    int it = 0;
    bool ok = true;
    for (int t = first_tile; t < total_units && ok; t += tile_step, ++it) {
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      const int tt = t % total_tiles;
      const int b = tt / tiles_per_batch;
      const int r = tt - b * tiles_per_batch;
      int mb_, nb_;
      tile_coords(p, r, mb_, nb_);
      const int m0 = mb_ * BM, n0 = nb_ * BN;
      if (!mbar_wait(&tfull_bar[acc], acc_ph)) {
        if (lane == 0) atomicCAS(p.status, 0, ST_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      uint8_t* cbase = reinterpret_cast<uint8_t*>(p.C);
      long long coff = static_cast<long long>(b) * p.batch_stride_c + row * p.ldc;
      int rs_owner = 0;
      if (p.rs_on) {
        // partial tile -> staging area of the rank that owns these rows (peer store)
        rs_owner = m0 / p.rs_rows_per_rank;
        cbase = reinterpret_cast<uint8_t*>(p.rs_stage[rs_owner]);
        coff = (static_cast<long long>(p.rank) * p.rs_rows_per_rank +
                (row - rs_owner * p.rs_rows_per_rank)) * p.ldc;
      }
      const __nv_bfloat16* rrow =
          p.residual ? reinterpret_cast<const __nv_bfloat16*>(p.residual) +
                           static_cast<long long>(b) * p.batch_stride_r + row * p.ldr
                     : nullptr;
      if (p.rs_on) {
        // Peer stores want whole 128-byte lines: transpose 64 columns at a time through a
        // per-warp shared-memory tile so that 8 lanes write one row's 128 contiguous bytes.
        uint8_t* sb = smem + STAGES * STAGE_BYTES + 256 + quad * EPI_WARP_BYTES;
        __nv_bfloat16* gbase = reinterpret_cast<__nv_bfloat16*>(cbase) +
                               (coff - static_cast<long long>(lane) * p.ldc);  // row of lane 0
#pragma unroll 1
        for (int c2 = 0; c2 < BN / 64; ++c2) {
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c2 * 64 + hc * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                oh[j] = __floats2bfloat162_rn(__uint_as_float(v[q4 * 8 + 2 * j]) * alpha,
                                              __uint_as_float(v[q4 * 8 + 2 * j + 1]) * alpha);
              *reinterpret_cast<uint4*>(
                  sb + CEO_IDX(lane * EPI_ROW_BYTES + hc * 64 + q4 * 16, EPI_WARP_BYTES - 15, 401)) = o;
            }
          }
          __syncwarp();
          const int ncol = n0 + c2 * 64 + (lane & 7) * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            const uint4 o = *reinterpret_cast<const uint4*>(
                sb + CEO_IDX(rl * EPI_ROW_BYTES + (lane & 7) * 16, EPI_WARP_BYTES - 15, 402));
            if (m0 + quad * 32 + rl < p.M && ncol < p.N)
              *reinterpret_cast<uint4*>(
                  gbase + CEO_IDX(static_cast<long long>(rl) * p.ldc + ncol,
                                  static_cast<long long>(p.world) * p.rs_rows_per_rank * p.ldc -
                                      (coff - static_cast<long long>(lane) * p.ldc) - 7, 403)) = o;
          }
          __syncwarp();
        }
      } else if (p.epi_mode == 1) {
        // gate/up projection with SiLU(gate) * up in the epilogue: C (interleaved gate/up,
        // kept for the backward pass) and act leave together, both as whole 32-byte sectors
        uint8_t* sb = smem + STAGES * STAGE_BYTES + 256 + quad * EPI_WARP_BYTES;
        uint8_t* sa = smem + STAGES * STAGE_BYTES + 256 + 4 * EPI_WARP_BYTES + quad * ACT_WARP_BYTES;
        const int row0 = m0 + quad * 32;
        __nv_bfloat16* gbase = reinterpret_cast<__nv_bfloat16*>(cbase) +
                               static_cast<long long>(row0) * p.ldc;
        __nv_bfloat16* abase = reinterpret_cast<__nv_bfloat16*>(p.aux) +
                               static_cast<long long>(row0) * p.ld_aux;
#pragma unroll 1
        for (int c2 = 0; c2 < BN / 64; ++c2) {
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c2 * 64 + hc * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[q4 * 8 + j]) * alpha;
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
              *reinterpret_cast<uint4*>(sb + lane * EPI_ROW_BYTES + hc * 64 + q4 * 16) = o;
              float a4[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float g = f[2 * j];
                a4[j] = g / (1.f + __expf(-g)) * f[2 * j + 1];
              }
              uint2 ao;
              __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(&ao);
              ah[0] = __floats2bfloat162_rn(a4[0], a4[1]);
              ah[1] = __floats2bfloat162_rn(a4[2], a4[3]);
              *reinterpret_cast<uint2*>(sa + lane * ACT_ROW_BYTES + hc * 32 + q4 * 8) = ao;
            }
          }
          __syncwarp();
          const int ncol = n0 + c2 * 64 + (lane & 7) * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            const uint4 o = *reinterpret_cast<const uint4*>(sb + rl * EPI_ROW_BYTES + (lane & 7) * 16);
            if (row0 + rl < p.M && ncol < p.N)
              *reinterpret_cast<uint4*>(gbase + static_cast<long long>(rl) * p.ldc + ncol) = o;
          }
          const int acol = (n0 + c2 * 64) / 2 + (lane & 3) * 8;  // 32 act columns per chunk
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int rl = i * 8 + (lane >> 2);
            const uint4 o = *reinterpret_cast<const uint4*>(sa + rl * ACT_ROW_BYTES + (lane & 3) * 16);
            if (row0 + rl < p.M && 2 * acol < p.N)
              *reinterpret_cast<uint4*>(abase + static_cast<long long>(rl) * p.ld_aux + acol) = o;
          }
          __syncwarp();
        }
      } else if (p.epi_mode == 2) {
        // down projection's data gradient with the SwiGLU backward in the epilogue: the
        // accumulator holds d(act) for 256 columns; the matching 512 interleaved gate/up
        // columns are read, and d(gate), d(up) written, 128 bytes per row at a time
        uint8_t* sb = smem + STAGES * STAGE_BYTES + 256 + quad * EPI_WARP_BYTES;
        const int row0 = m0 + quad * 32;
        const __nv_bfloat16* gubase = reinterpret_cast<const __nv_bfloat16*>(p.aux) +
                                      static_cast<long long>(row0) * p.ld_aux;
        __nv_bfloat16* gbase = reinterpret_cast<__nv_bfloat16*>(cbase) +
                               static_cast<long long>(row0) * p.ldc;
        // the gate/up rows of step c + 1 are requested while step c is being computed, so the
        // latency of those global loads stays off the epilogue's critical path
        uint4 pre[8];
        auto fetch = [&](int c) {
          const int gcol = 2 * (n0 + c * 32) + (lane & 7) * 8;  // 64 gate/up columns per step
          const bool col_ok = n0 + c * 32 < p.N;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            pre[i] = make_uint4(0, 0, 0, 0);
            if (row0 + rl < p.M && col_ok)
              pre[i] = *reinterpret_cast<const uint4*>(gubase + static_cast<long long>(rl) * p.ld_aux + gcol);
          }
        };
        fetch(0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int gcol = 2 * (n0 + c * 32) + (lane & 7) * 8;
          const bool col_ok = n0 + c * 32 < p.N;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            *reinterpret_cast<uint4*>(sb + rl * EPI_ROW_BYTES + (lane & 7) * 16) = pre[i];
          }
          __syncwarp();
          if (c + 1 < BN / 32) fetch(c + 1);
          uint32_t v[32];
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) {  // 4 d(act) values <-> 8 interleaved gate/up values
            uint4* slot = reinterpret_cast<uint4*>(sb + lane * EPI_ROW_BYTES + q * 16);
            const uint4 u4 = *slot;
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u4);
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 gu = __bfloat1622float2(h[j]);  // (gate, up)
              const float d = __uint_as_float(v[q * 4 + j]) * alpha;
              const float sg = 1.f / (1.f + __expf(-gu.x));
              const float silu = gu.x * sg;
              oh[j] = __floats2bfloat162_rn(d * gu.y * (sg + silu * (1.f - sg)), d * silu);
            }
            *slot = o;
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            const uint4 o = *reinterpret_cast<const uint4*>(sb + rl * EPI_ROW_BYTES + (lane & 7) * 16);
            if (row0 + rl < p.M && col_ok)
              *reinterpret_cast<uint4*>(gbase + static_cast<long long>(rl) * p.ldc + gcol) = o;
          }
          __syncwarp();
        }
      } else if (!p.out_f32 && !p.accumulate && !p.bias && ((p.N | p.ldc) & 7) == 0 &&
                 (!p.residual || (p.ldr & 7) == 0)) {
        // bf16 output (+ bf16 residual): same 64-column transpose through the per-warp tile,
        // so both the residual read and the store move whole 128-byte lines (a lane-per-row
        // store touches 32 different lines per instruction)
        uint8_t* sb = smem + STAGES * STAGE_BYTES + 256 + quad * EPI_WARP_BYTES;
        const int row0 = m0 + quad * 32;  // row of lane 0
        __nv_bfloat16* gbase = reinterpret_cast<__nv_bfloat16*>(cbase) +
                               static_cast<long long>(b) * p.batch_stride_c +
                               static_cast<long long>(row0) * p.ldc;
        const __nv_bfloat16* rbase =
            p.residual ? reinterpret_cast<const __nv_bfloat16*>(p.residual) +
                             static_cast<long long>(b) * p.batch_stride_r +
                             static_cast<long long>(row0) * p.ldr
                       : nullptr;
        // the residual rows of chunk c2 + 1 are requested while chunk c2 is converted and
        // stored: their global-load latency stays off the epilogue's critical path
        uint4 pre[8];
        auto fetch_res = [&](int c2) {
          const int ncol = n0 + c2 * 64 + (lane & 7) * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            pre[i] = make_uint4(0, 0, 0, 0);
            if (row0 + rl < p.M && ncol < p.N)
              pre[i] = *reinterpret_cast<const uint4*>(rbase + static_cast<long long>(rl) * p.ldr + ncol);
          }
        };
        if (rbase) fetch_res(0);
#pragma unroll 1
        for (int c2 = 0; c2 < BN / 64; ++c2) {
          const int ncol = n0 + c2 * 64 + (lane & 7) * 8;
          if (rbase) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = i * 4 + (lane >> 3);
              *reinterpret_cast<uint4*>(sb + rl * EPI_ROW_BYTES + (lane & 7) * 16) = pre[i];
            }
            __syncwarp();
            if (c2 + 1 < BN / 64) fetch_res(c2 + 1);
          }
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c2 * 64 + hc * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4* slot = reinterpret_cast<uint4*>(
                  sb + CEO_IDX(lane * EPI_ROW_BYTES + hc * 64 + q4 * 16, EPI_WARP_BYTES - 15, 404));
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[q4 * 8 + j]) * alpha;
              if (rbase) {
                const uint4 u = *slot;
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 x = __bfloat1622float2(h[j]);
                  f[2 * j] += x.x;
                  f[2 * j + 1] += x.y;
                }
              }
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
              *slot = o;
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            const uint4 o = *reinterpret_cast<const uint4*>(sb + rl * EPI_ROW_BYTES + (lane & 7) * 16);
            if (row0 + rl < p.M && ncol < p.N)
              *reinterpret_cast<uint4*>(
                  gbase + CEO_IDX(static_cast<long long>(rl) * p.ldc + ncol,
                                  static_cast<long long>(p.M - row0 - 1) * p.ldc + p.N - 7, 405)) = o;
          }
          __syncwarp();
        }
      } else if (p.out_f32 && !p.bias && !p.residual && p.split_k == 1 &&
                 ((p.N | p.ldc) & 3) == 0) {
        // fp32 output (weight gradients, usually accumulating): 32 columns at a time through
        // the same per-warp tile, so the read-modify-write of C moves whole 128-byte lines
        uint8_t* sb = smem + STAGES * STAGE_BYTES + 256 + quad * EPI_WARP_BYTES;
        const int row0 = m0 + quad * 32;
        float* gbase = reinterpret_cast<float*>(cbase) + static_cast<long long>(b) * p.batch_stride_c +
                       static_cast<long long>(row0) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(sb + lane * EPI_ROW_BYTES + q * 16) =
                make_float4(__uint_as_float(v[4 * q]) * alpha, __uint_as_float(v[4 * q + 1]) * alpha,
                            __uint_as_float(v[4 * q + 2]) * alpha,
                            __uint_as_float(v[4 * q + 3]) * alpha);
          __syncwarp();
          const int ncol = n0 + c * 32 + (lane & 7) * 4;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3);
            float4 o = *reinterpret_cast<const float4*>(sb + rl * EPI_ROW_BYTES + (lane & 7) * 16);
            if (row0 + rl < p.M && ncol < p.N) {
              float4* dst = reinterpret_cast<float4*>(gbase + static_cast<long long>(rl) * p.ldc + ncol);
              if (p.accumulate) {
                const float4 old = *dst;
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *dst = o;
            }
          }
          __syncwarp();
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the masked stores
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        const int n = n0 + c * 32;
        if (!row_ok || n >= p.N) continue;
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * alpha;
        const bool full = (n + 32 <= p.N);
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (full || n + j < p.N) f[j] += p.bias[n + j];
        }
        if (rrow) {
          if (full && ((p.ldr & 7) == 0)) {
            const uint4* rp = reinterpret_cast<const uint4*>(rrow + n);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u = rp[q];
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 x = __bfloat1622float2(h[j]);
                f[q * 8 + 2 * j] += x.x;
                f[q * 8 + 2 * j + 1] += x.y;
              }
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (n + j < p.N) f[j] += __bfloat162float(rrow[n + j]);
          }
        }
        if (p.out_f32) {
          float* crow = reinterpret_cast<float*>(cbase) + coff + n;
          if (p.split_k > 1) {
            // k-slices of this tile land in any order: accumulate with vector reductions
            if (full && ((p.ldc & 3) == 0)) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(crow + 4 * q),
                             "f"(f[4 * q]), "f"(f[4 * q + 1]), "f"(f[4 * q + 2]), "f"(f[4 * q + 3])
                             : "memory");
            } else {
              for (int j = 0; j < 32; ++j)
                if (n + j < p.N) atomicAdd(crow + j, f[j]);
            }
          } else if (full && ((p.ldc & 3) == 0)) {
            float4* cp = reinterpret_cast<float4*>(crow);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
              if (p.accumulate) {
                float4 old = cp[q];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              cp[q] = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (n + j < p.N) crow[j] = f[j] + (p.accumulate ? crow[j] : 0.f);
          }
        } else {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(cbase) + coff + n;
          if (full && ((p.ldc & 7) == 0)) {
            uint4* cp = reinterpret_cast<uint4*>(crow);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (p.accumulate) {
                uint4 u = cp[q];
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 x = __bfloat1622float2(h[j]);
                  f[q * 8 + 2 * j] += x.x;
                  f[q * 8 + 2 * j + 1] += x.y;
                }
              }
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                oh[j] = __floats2bfloat162_rn(f[q * 8 + 2 * j], f[q * 8 + 2 * j + 1]);
              cp[q] = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (n + j < p.N) {
                float o = f[j] + (p.accumulate ? __bfloat162float(crow[j]) : 0.f);
                crow[j] = __float2bfloat16(o);
              }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (p.rs_on) {
        // the warp barrier orders every lane's stores before lane 0's system-scope release
        __syncwarp();
        if (lane == 0)
          red_release_sys_add(p.rs_count[rs_owner] + p.rank * (p.rs_rows_per_rank / BM) +
                                  (m0 - rs_owner * p.rs_rows_per_rank) / BM,
                              1u);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map over (batch, outer, inner) with a box of 128 bytes x box_outer rows and 128B
// swizzle; elements are bf16 (esize 2) or 8-bit floats moved as bytes (esize 1).
static int make_tmap(CUtensorMap* tm, const void* ptr, uint64_t inner, uint64_t outer,
                     uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                     uint32_t box_outer, uint32_t esize = 2) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  // The driver entry point needs a current context; a thread that has made no runtime
  // call yet (an autograd worker thread, for one) has none until the runtime binds it.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {ld_elems * esize,
                           (batch > 1 ? batch_stride_elems : ld_elems * outer) * esize};
  cuuint32_t box[3] = {128 / esize, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                  3, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr,
            "ceo: cuTensorMapEncodeTiled failed (%d): ptr=%p dims={%llu,%llu,%llu} strides={%llu,%llu} "
            "box={%u,%u,1}\n",
            static_cast<int>(r), ptr, (unsigned long long)dims[0], (unsigned long long)dims[1],
            (unsigned long long)dims[2], (unsigned long long)strides[0],
            (unsigned long long)strides[1], box[0], box_outer);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// M/N-major operand whose contiguous extent is a multiple of 64: map it as
// (64, k, panel, batch) so that one box {64, BK, panels, 1} brings a whole stage tile in the
// [panel][k][64] layout the MMA descriptors expect (one TMA instruction instead of one per
// 64-wide panel).  A partial last tile reads panels past the extent as zeros (out-of-bounds
// fill), exactly like the per-panel loads.
static int make_tmap_mn4(CUtensorMap* tm, const void* ptr, uint64_t inner, uint64_t outer,
                         uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                         uint32_t panels) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[4] = {64, outer, inner / 64, batch};
  cuuint64_t strides[3] = {ld_elems * 2, 128,
                           (batch > 1 ? batch_stride_elems : ld_elems * outer) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(ceo::BK), panels, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static int g_num_sms = 0;
static int g_deterministic = 0;  // 1: no split-K (its atomics make the fp32 sum order vary)

template <int A_MN, int B_MN, int FP8 = 0>
static cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                          int grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<A_MN, B_MN, FP8>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  gemm_bf16_tcgen05_kernel<A_MN, B_MN, FP8><<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace ceo

// 8-bit float operands of a GEMM launch (see GemmParams).
struct Fp8Desc {
  int on = 0;
  int kind_a = 0, kind_b = 0;  // 0 e4m3, 1 e5m2
  const float* scale_a = nullptr;
  const float* scale_b = nullptr;
};

// SwiGLU fused into the epilogue (see GemmParams::epi_mode).
struct EpiDesc {
  int mode = 0;
  void* aux = nullptr;
  long long ld_aux = 0;
};

// Host-side description of the collective fused into a GEMM launch (see GemmParams).
struct FusedDesc {
  int kind = 0;  // 0 plain, 1 all-gather of A, 2 all-gather of B, 3 reduce-scatter of C
  int rank = 0, world = 1;
  int copy_ctas = 0;
  void* const* peers = nullptr;    // AG: gathered buffers per rank; RS: staging per rank
  void* const* counters = nullptr; // RS: counters per rank
  unsigned* flags = nullptr;       // AG: local flags
  unsigned target = 0;
  int blk_rows = 0;                // AG: rows per flag (0: the tile height of the operand)
  void* const* extra = nullptr;    // AG: a second tensor's buffers per rank (optional)
  long long extra_shard_bytes = 0;
  void* rs_out = nullptr;
  const void* rs_residual = nullptr;
  long long rs_ldo = 0;
  int rs_ctas = 0;                 // RS: CTAs that only reduce (0: 32)
};

static int gemm_run(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int a_mn_major, int b_mn_major, int batch,
                    long long batch_stride_a, long long batch_stride_b, long long batch_stride_c,
                    int out_f32, int accumulate, float alpha, const float* bias,
                    const void* residual, long long ldr, long long batch_stride_r, int* status,
                    int max_ctas, const FusedDesc& fz, cudaStream_t stream, int split_k_mode = 1,
                    const Fp8Desc& f8 = Fp8Desc(), const EpiDesc& epi = EpiDesc()) {
  using namespace ceo;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (f8.on && (a_mn_major || b_mn_major || fz.kind != 0)) return -5;
  const uint32_t esize = f8.on ? 1 : 2;
  const long long amask = 16 / esize - 1;
  // TMA needs 16-byte aligned bases and row strides
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (lda & amask) || (ldb & amask) ||
      (batch > 1 && ((batch_stride_a & amask) || (batch_stride_b & amask))))
    return -2;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int rc;
  const bool a4 = a_mn_major && fz.kind == 0 && (M & 63) == 0;
  const bool b4 = b_mn_major && fz.kind == 0 && (N & 63) == 0;
  if (a_mn_major == 0)
    rc = make_tmap(&ta, A, K, M, batch, lda, batch_stride_a, BM, esize);
  else if (a4)
    rc = make_tmap_mn4(&ta, A, M, K, batch, lda, batch_stride_a, BM / 64);
  else
    rc = make_tmap(&ta, A, M, K, batch, lda, batch_stride_a, BK);
  if (rc) return -3;
  if (b_mn_major == 0)
    rc = make_tmap(&tb, B, K, N, batch, ldb, batch_stride_b, BN, esize);
  else if (b4)
    rc = make_tmap_mn4(&tb, B, N, K, batch, ldb, batch_stride_b, BN / 64);
  else
    rc = make_tmap(&tb, B, N, K, batch, ldb, batch_stride_b, BK);
  if (rc) return -4;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.a_4d = a4;
  p.b_4d = b4;
  p.C = C;
  p.residual = residual;
  p.bias = bias;
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.batch_stride_c = batch_stride_c;
  p.batch_stride_r = batch_stride_r;
  p.batch = batch;
  p.out_f32 = out_f32;
  p.accumulate = accumulate;
  p.alpha = alpha;
  p.fp8_a = f8.kind_a;
  p.fp8_b = f8.kind_b;
  p.scale_a = f8.scale_a;
  p.scale_b = f8.scale_b;
  p.num_m = (M + BM - 1) / BM;
  p.num_n = (N + BN - 1) / BN;
  p.status = status;
  p.rank = fz.rank;
  p.world = fz.world;
  if (epi.mode) {
    // bf16 output, one matrix, no other epilogue term; whole 64-column groups of gate/up
    if (epi.mode < 0 || epi.mode > 2 || !epi.aux || out_f32 || accumulate || bias || residual ||
        batch != 1 || fz.kind != 0 || (epi.ld_aux & 7) || (ldc & 7) ||
        (reinterpret_cast<uintptr_t>(epi.aux) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) ||
        (epi.mode == 1 ? (N & 63) : (N & 31)))
      return -5;
    p.epi_mode = epi.mode;
    p.aux = epi.aux;
    p.ld_aux = epi.ld_aux;
  }
  // bands of 16 row blocks: a wave of 148 tiles is then ~16 x 9 tiles whose A and B panels
  // both stay in L2 (m-fastest over all rows re-reads A once per ~2 n-blocks)
  p.grp_m = p.num_m > 16 ? 16 : p.num_m;
  int cap = g_num_sms;
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (fz.kind == 1 || fz.kind == 2) {
    // gathered operand: K-major rows only, shards of whole row blocks, dense rows
    const int rows = fz.kind == 1 ? M : N;
    const int tile = fz.kind == 1 ? BM : BN;
    const int blk = fz.blk_rows > 0 ? fz.blk_rows : tile;
    const long long ld = fz.kind == 1 ? lda : ldb;
    if ((fz.kind == 1 ? a_mn_major : b_mn_major) || batch != 1 || ld != K ||
        rows % fz.world || (rows / fz.world) % blk || fz.world < 2 || fz.world > 8 ||
        (fz.extra_shard_bytes & 15) || (fz.extra_shard_bytes > 0 && !fz.extra))
      return -5;
    p.ag_operand = fz.kind;
    if (fz.copy_ctas < 0) {
      // copy-first mode (see ag_copy_all): flags[0] is the launch's counter, zeroed in stream
      p.ag_all = 1;
      p.ag_ctas = 0;
      const cudaError_t ez = cudaMemsetAsync(fz.flags, 0, sizeof(unsigned), stream);
      if (ez != cudaSuccess) return static_cast<int>(ez);
    } else {
      p.ag_ctas = fz.copy_ctas > 0 ? fz.copy_ctas : 8;
      if (p.ag_ctas > cap / 4) p.ag_ctas = cap / 4;
    }
    p.ag_rows_per_shard = rows / fz.world;
    p.ag_blk_rows = blk;
    p.ag_row_bytes = static_cast<long long>(K) * 2;
    if (fz.extra_shard_bytes > 0) {
      p.ag_extra_bytes = fz.extra_shard_bytes;
      for (int r = 0; r < fz.world; ++r)
        p.ag_extra_src[r] = static_cast<const uint8_t*>(fz.extra[r]) + r * fz.extra_shard_bytes;
      p.ag_extra_dst = fz.extra[fz.rank];
    }
    for (int r = 0; r < fz.world; ++r)
      p.ag_src[r] = static_cast<const uint8_t*>(fz.peers[r]) +
                    static_cast<long long>(r) * p.ag_rows_per_shard * p.ag_row_bytes;
    p.ag_dst = const_cast<void*>(fz.kind == 1 ? A : B);
    p.ag_flags = fz.flags;
    p.ag_target = fz.target;
    // the traversal starts at the tile that holds this rank's first row
    const int rot = static_cast<int>(static_cast<long long>(fz.rank) * p.ag_rows_per_shard / tile);
    if (fz.kind == 1) {
      p.m_rot = rot;
      if (p.ag_rows_per_shard % tile == 0) p.grp_m = p.ag_rows_per_shard / tile;
    } else {
      p.n_rot = rot;
    }
  } else if (fz.kind == 3) {
    if (batch != 1 || out_f32 || accumulate || bias || residual || M % fz.world ||
        (M / fz.world) % BM || (N & 7) || fz.world < 2 || fz.world > 8)
      return -5;
    p.rs_on = 1;
    p.rs_rows_per_rank = M / fz.world;
    for (int r = 0; r < fz.world; ++r) {
      p.rs_stage[r] = fz.peers[r];
      p.rs_count[r] = static_cast<unsigned*>(fz.counters[r]);
    }
    p.rs_target = fz.target;
    p.rs_out = fz.rs_out;
    p.rs_residual = fz.rs_residual;
    p.rs_ldo = fz.rs_ldo;
    p.ldc = N;  // staging rows are dense
    // tile order: see tile_coords (stripes); a few CTAs do nothing but reduce
    p.ag_ctas = fz.rs_ctas > 0 ? fz.rs_ctas : 32;
    if (p.ag_ctas > cap / 3) p.ag_ctas = cap / 3;
    if (p.ag_ctas < 1) p.ag_ctas = 1;
    p.grp_m = p.num_m;
  }
  long long total = static_cast<long long>(p.num_m) * p.num_n * batch;
  p.split_k = 1;
  if (fz.kind == 0 && out_f32 && accumulate && !bias && !residual && split_k_mode != 0 &&
      !ceo::g_deterministic) {
    // few tiles with a long K (weight gradients): pick the split that fills whole waves best
    const int bke = f8.on ? 2 * BK : BK;
    const int num_kb = (K + bke - 1) / bke;
    // every extra slice re-sends the whole fp32 C through L2 atomics, so a split has to buy a
    // clear gain in wave efficiency (measured: 5 slices of the 2048x5632 gradient lose)
    double best = 0.0;
    for (int s = 1; s <= 3 && s * 16 <= num_kb; ++s) {
      const long long units = total * s;
      const long long waves = (units + cap - 1) / cap;
      const double eff = static_cast<double>(units) / (waves * cap) - 0.05 * (s - 1);
      if (eff > best + (s > 1 ? 0.05 : 0.0)) { best = eff; p.split_k = s; }
    }
  }
  total *= p.split_k;
  int grid = static_cast<int>(total + p.ag_ctas < cap ? total + p.ag_ctas : cap);
  cudaError_t e;
  if (f8.on) e = launch<0, 0, 1>(ta, tb, p, grid, stream);
  else if (a_mn_major == 0 && b_mn_major == 0) e = launch<0, 0>(ta, tb, p, grid, stream);
  else if (a_mn_major == 0) e = launch<0, 1>(ta, tb, p, grid, stream);
  else if (b_mn_major == 0) e = launch<1, 0>(ta, tb, p, grid, stream);
  else e = launch<1, 1>(ta, tb, p, grid, stream);
  return static_cast<int>(e);
}

extern "C" int ceo_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                             long long lda, long long ldb, long long ldc, int a_mn_major,
                             int b_mn_major, int batch, long long batch_stride_a,
                             long long batch_stride_b, long long batch_stride_c, int out_f32,
                             int accumulate, float alpha, const float* bias, const void* residual,
                             long long ldr, long long batch_stride_r, int* status, int max_ctas,
                             cudaStream_t stream) {
  FusedDesc fz;
  return gemm_run(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, batch, batch_stride_a,
                  batch_stride_b, batch_stride_c, out_f32, accumulate, alpha, bias, residual, ldr,
                  batch_stride_r, status, max_ctas, fz, stream);
}

// The bf16 GEMM with SwiGLU in its epilogue.  mode 1: C[M,N] = A B^T holds gate/up in
// interleaved columns and aux (M x N/2, bf16, ld_aux) receives silu(gate) * up.  mode 2: the
// product A B^T is d(act) (M x N); aux is the saved interleaved gate/up (M x 2N, ld_aux) and
// C (M x 2N, ldc) receives the interleaved d(gate/up).
extern "C" int ceo_gemm_bf16_swiglu(const void* A, const void* B, void* C, int M, int N, int K,
                                    long long lda, long long ldb, long long ldc, int a_mn_major,
                                    int b_mn_major, float alpha, int mode, void* aux,
                                    long long ld_aux, int* status, cudaStream_t stream) {
  FusedDesc fz;
  EpiDesc epi;
  epi.mode = mode;
  epi.aux = aux;
  epi.ld_aux = ld_aux;
  if (mode != 1 && mode != 2) return -5;
  return gemm_run(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, 1, 0, 0, 0, 0, 0, alpha,
                  nullptr, nullptr, 0, 0, status, 0, fz, stream, 1, Fp8Desc(), epi);
}

// C[M,N] = alpha / (scale_a * scale_b) * A[M,K] @ B[N,K]^T (+ bias) (+ residual) with 8-bit
// float operands (kind 0 = e4m3, 1 = e5m2), both K-major, strides in elements (= bytes) and
// multiples of 16.  scale_a / scale_b are the device-side scales the operands were quantised
// with (q = x * scale); both null means no rescaling.  C is bf16 or fp32.
extern "C" int ceo_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int kind_a, int kind_b,
                            int out_f32, int accumulate, float alpha, const float* scale_a,
                            const float* scale_b, const float* bias, const void* residual,
                            long long ldr, int* status, cudaStream_t stream) {
  if (kind_a < 0 || kind_a > 1 || kind_b < 0 || kind_b > 1 || (!scale_a != !scale_b)) return -5;
  FusedDesc fz;
  Fp8Desc f8;
  f8.on = 1;
  f8.kind_a = kind_a;
  f8.kind_b = kind_b;
  f8.scale_a = scale_a;
  f8.scale_b = scale_b;
  return gemm_run(A, B, C, M, N, K, lda, ldb, ldc, 0, 0, 1, 0, 0, 0, out_f32, accumulate, alpha,
                  bias, residual, ldr, 0, status, 0, fz, stream, 1, f8);
}

// All-gather fused into the GEMM that consumes the gathered operand.  `gathered` is the table
// of every rank's gathered buffer (rows x K bf16, dense); rank r's own shard already sits in
// rows [r*rows/world, (r+1)*rows/world) of ITS buffer, and copy CTAs of this launch pull the
// other shards from the peers while the remaining CTAs compute, local rows first.
// operand: 1 = A (M rows gathered), 2 = B (N rows gathered).  The non-gathered operand and C
// are ordinary local tensors.  `flags`: local unsigned[rows/blk_rows]; target grows by 1 per
// call.  blk_rows (0 = 128 for A, 256 for B) is the row granularity of the flags: shards must
// be whole multiples of it, which lets a weight matrix whose row count is not a multiple of
// world x 256 be gathered (FSDP weight shards).  `extra` (optional): the per-rank buffers of
// a second tensor sharded the same way (extra_shard_bytes per rank, shard r at byte offset
// r * extra_shard_bytes); the copy CTAs gather it after the operand, complete at kernel end.
extern "C" int ceo_ag_gemm_bf16(void* const* gathered, int operand, const void* other, void* C,
                                int M, int N, int K, long long ld_other, long long ldc,
                                int other_mn_major, int out_f32, int accumulate, float alpha,
                                const void* residual, long long ldr, void* flags,
                                unsigned int target, int rank, int world, int copy_ctas,
                                int blk_rows, void* const* extra, long long extra_shard_bytes,
                                int* status, cudaStream_t stream) {
  if (operand != 1 && operand != 2) return -5;
  FusedDesc fz;
  fz.kind = operand;
  fz.rank = rank;
  fz.world = world;
  fz.copy_ctas = copy_ctas;
  fz.peers = gathered;
  fz.flags = static_cast<unsigned*>(flags);
  fz.target = target;
  fz.blk_rows = blk_rows;
  fz.extra = extra;
  fz.extra_shard_bytes = extra_shard_bytes;
  const void* A = operand == 1 ? gathered[rank] : other;
  const void* B = operand == 2 ? gathered[rank] : other;
  return gemm_run(A, B, C, M, N, K, operand == 1 ? K : ld_other, operand == 2 ? K : ld_other, ldc,
                  operand == 1 ? 0 : other_mn_major, operand == 2 ? 0 : other_mn_major, 1, 0, 0, 0,
                  out_f32, accumulate, alpha, nullptr, residual, ldr, 0, status, 0, fz, stream);
}

// GEMM fused with the reduce-scatter of its output over M: every rank computes the partial
// product of its K-slice; out (M/world x N bf16, this rank's rows) = sum over ranks (+residual).
// `stage`: table of per-rank staging buffers [world][M/world][N] bf16; `counters`: table of
// per-rank unsigned[world][M/world/128], never reset: `target` is the value every counter of
// this rank reaches when all partial tiles of THIS call have arrived (it grows by
// 4 * ceil(N/256) per call as long as M stays the same).  rs_ctas CTAs (0 = 32) only reduce:
// tiles are computed stripe by stripe so the reduction of a stripe overlaps the next ones.
// Successive calls must alternate between two staging buffers (a rank can be one call ahead
// of a peer that is still reducing), which replaces a barrier between calls.
extern "C" int ceo_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, long long lda,
                                long long ldb, int a_mn_major, int b_mn_major, float alpha,
                                void* const* stage, void* const* counters, unsigned int target,
                                void* out, const void* residual, long long ldo, int rank,
                                int world, int rs_ctas, int* status, cudaStream_t stream) {
  FusedDesc fz;
  fz.kind = 3;
  fz.rs_ctas = rs_ctas;
  fz.rank = rank;
  fz.world = world;
  fz.peers = stage;
  fz.counters = counters;
  fz.target = target;
  fz.rs_out = out;
  fz.rs_residual = residual;
  fz.rs_ldo = ldo;
  return gemm_run(A, B, stage[rank], M, N, K, lda, ldb, N, a_mn_major, b_mn_major, 1, 0, 0, 0, 0,
                  0, alpha, nullptr, nullptr, 0, 0, status, 0, fz, stream);
}

extern "C" int ceo_gemm_set_wait_limit(unsigned int iterations) {
  return ceo::set_wait_limit_override(iterations);
}

// 1 = bit-reproducible GEMM results (weight-gradient GEMMs then never split K).
extern "C" int ceo_set_deterministic(int on) {
  ceo::g_deterministic = on ? 1 : 0;
  return 0;
}
