// Generic tensor utilities: prefix scan, row gather / scatter / scatter-add, pitched copy,
// 2-D transpose and 32-bit fill.  The reference only names these units in its build list
// (build.zig:149-161: scan, gather, scatter, memory) and ships no source for them.
#include "common/util.cuh"
#include "common/check.cuh"
#include "include/ceo_kernels.h"

CEO_BOUNDS_TU(scan)

namespace ceo {

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_TILE = SCAN_THREADS * 4;     // elements one CTA scans per iteration
constexpr int SCAN_SEG = 16 * SCAN_TILE;        // elements per segment of a split row

// Inclusive scan of one value per thread over the CTA; returns the CTA total through `total`.
__device__ __forceinline__ float block_scan_incl(float v, float* warp_sums, float& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) warp_sums[warp] = v;
  __syncthreads();
  float before = 0.f, all = 0.f;
#pragma unroll
  for (int w = 0; w < SCAN_THREADS / 32; ++w) {
    const float s = warp_sums[w];
    if (w < warp) before += s;
    all += s;
  }
  __syncthreads();
  total = all;
  return v + before;
}

// Scans elements [lo, hi) of a row (logical order; `reverse` maps logical i to n-1-i) starting
// from `carry`.
__device__ void scan_span(const float* __restrict__ x, float* __restrict__ y, long long n,
                          long long lo, long long hi, float carry, bool exclusive, bool reverse,
                          float* warp_sums) {
  for (long long base = lo; base < hi; base += SCAN_TILE) {
    float v[4];
    float local = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = base + threadIdx.x * 4 + j;
      v[j] = i < hi ? x[reverse ? n - 1 - i : i] : 0.f;
      local += v[j];
    }
    float total;
    const float incl = block_scan_incl(local, warp_sums, total);
    float run = carry + incl - local;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = base + threadIdx.x * 4 + j;
      const float out = exclusive ? run : run + v[j];
      run += v[j];
      if (i < hi) y[reverse ? n - 1 - i : i] = out;
    }
    carry += total;
  }
}

__global__ void __launch_bounds__(SCAN_THREADS)
cumsum_rows_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, int exclusive,
                   int reverse) {
  __shared__ float warp_sums[SCAN_THREADS / 32];
  const long long row = blockIdx.x;
  scan_span(x + row * n, y + row * n, n, 0, n, 0.f, exclusive, reverse, warp_sums);
}

// Split rows: pass 1 writes the sum of each segment, pass 2 scans a segment from the sum of
// the segments before it.
__global__ void __launch_bounds__(SCAN_THREADS)
segment_sum_kernel(const float* __restrict__ x, float* __restrict__ seg_sums, long long n,
                   int nseg, int reverse) {
  const long long row = blockIdx.y;
  const long long lo = static_cast<long long>(blockIdx.x) * SCAN_SEG;
  const long long hi = lo + SCAN_SEG < n ? lo + SCAN_SEG : n;
  const float* xr = x + row * n;
  __shared__ float red[33];
  float s = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += SCAN_THREADS) s += xr[reverse ? n - 1 - i : i];
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) seg_sums[row * nseg + blockIdx.x] = s;
}
__global__ void __launch_bounds__(SCAN_THREADS)
cumsum_segments_kernel(const float* __restrict__ x, float* __restrict__ y,
                       const float* __restrict__ seg_sums, long long n, int nseg, int exclusive,
                       int reverse) {
  __shared__ float warp_sums[SCAN_THREADS / 32];
  __shared__ float red[33];
  const long long row = blockIdx.y;
  float c = 0.f;
  for (int s = threadIdx.x; s < static_cast<int>(blockIdx.x); s += SCAN_THREADS)
    c += seg_sums[row * nseg + s];
  const float carry_s = block_reduce_sum(c, red);
  const long long lo = static_cast<long long>(blockIdx.x) * SCAN_SEG;
  const long long hi = lo + SCAN_SEG < n ? lo + SCAN_SEG : n;
  scan_span(x + row * n, y + row * n, n, lo, hi, carry_s, exclusive, reverse, warp_sums);
}

// dst[r] = src[idx[r]] for rows of `units` 16-byte units; out-of-range indices give zero rows.
__global__ void gather_rows_kernel(const long long* __restrict__ idx, const uint4* __restrict__ src,
                                   uint4* __restrict__ dst, long long n, int units,
                                   long long src_rows) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = w; r < n; r += nw) {
    const long long id = idx[r];
    const bool ok = id >= 0 && id < src_rows;
    for (int c = lane; c < units; c += 32)
      dst[CEO_IDX(r * units + c, n * units, 101)] =
          ok ? src[CEO_IDX(id * units + c, src_rows * units, 102)] : make_uint4(0, 0, 0, 0);
  }
}
// dst[idx[r]] = src[r]  (duplicate indices: one of the writers wins)
__global__ void scatter_rows_kernel(const long long* __restrict__ idx,
                                    const uint4* __restrict__ src, uint4* __restrict__ dst,
                                    long long n, int units, long long dst_rows) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = w; r < n; r += nw) {
    const long long id = idx[r];
    if (id < 0 || id >= dst_rows) continue;
    for (int c = lane; c < units; c += 32)
      dst[CEO_IDX(id * units + c, dst_rows * units, 103)] = src[CEO_IDX(r * units + c, n * units, 104)];
  }
}
// dst[idx[r]] += src[r], fp32 rows of D (multiple of 4) floats
__global__ void scatter_add_f32_kernel(const long long* __restrict__ idx,
                                       const float* __restrict__ src, float* __restrict__ dst,
                                       long long n, int D, long long dst_rows) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = w; r < n; r += nw) {
    const long long id = idx[r];
    if (id < 0 || id >= dst_rows) continue;
    for (int c = lane * 4; c < D; c += 128) {
      const float4 f = *reinterpret_cast<const float4*>(src + CEO_IDX(r * D + c, n * D - 3, 105));
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(
                       dst + CEO_IDX(id * D + c, dst_rows * D - 3, 106)),
                   "f"(f.x), "f"(f.y), "f"(f.z), "f"(f.w)
                   : "memory");
    }
  }
}

// rows x (units x 16 B) copy between pitched buffers
__global__ void copy2d_kernel(const uint8_t* __restrict__ src, long long src_pitch,
                              uint8_t* __restrict__ dst, long long dst_pitch, long long rows,
                              int units) {
  const long long total = rows * units;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / units;
    const int c = static_cast<int>(i - r * units);
    *reinterpret_cast<uint4*>(dst + r * dst_pitch + c * 16ll) =
        *reinterpret_cast<const uint4*>(src + r * src_pitch + c * 16ll);
  }
}

// dst (cols x rows) = src (rows x cols)^T for 2-byte elements, 64x64 tiles through shared memory
__global__ void __launch_bounds__(256)
transpose16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int rows,
                   int cols, long long lds, long long ldd) {
  __shared__ uint16_t tile[64][66];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int j = ty; j < 64; j += 4)
    if (r0 + j < rows && c0 + tx < cols)
      tile[j][tx] = src[CEO_IDX((r0 + j) * lds + c0 + tx, (rows - 1) * lds + cols, 107)];
  __syncthreads();
  for (int j = ty; j < 64; j += 4)
    if (c0 + j < cols && r0 + tx < rows)
      dst[CEO_IDX((c0 + j) * ldd + r0 + tx, (cols - 1) * ldd + rows, 108)] = tile[tx][j];
}

__global__ void memset32_kernel(uint32_t* __restrict__ x, long long n, uint32_t value) {
  const long long nv = n >> 2;
  uint4* xv = reinterpret_cast<uint4*>(x);
  const uint4 v4 = make_uint4(value, value, value, value);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (long long i = t; i < nv; i += stride) xv[i] = v4;
  for (long long i = (nv << 2) + t; i < n; i += stride) x[i] = value;
}

}  // namespace ceo
using namespace ceo;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int ceo_cumsum_scratch_floats(long long rows, long long n) {
  if (rows >= 64 || n <= 4 * SCAN_SEG) return 0;
  return static_cast<int>(rows * ((n + SCAN_SEG - 1) / SCAN_SEG));
}
extern "C" int ceo_cumsum_f32(const float* x, float* y, long long rows, long long n, int exclusive,
                              int reverse, float* scratch, cudaStream_t stream) {
  if (rows <= 0 || n <= 0 || rows > 0x7fffffffll) return -5;
  const long long need = ceo_cumsum_scratch_floats(rows, n);
  if (need == 0) {
    cumsum_rows_kernel<<<static_cast<unsigned>(rows), SCAN_THREADS, 0, stream>>>(x, y, n, exclusive,
                                                                                reverse);
    return static_cast<int>(cudaGetLastError());
  }
  if (!scratch || rows > 65535) return -5;
  const int nseg = static_cast<int>((n + SCAN_SEG - 1) / SCAN_SEG);
  const dim3 g(nseg, static_cast<unsigned>(rows));
  segment_sum_kernel<<<g, SCAN_THREADS, 0, stream>>>(x, scratch, n, nseg, reverse);
  cumsum_segments_kernel<<<g, SCAN_THREADS, 0, stream>>>(x, y, scratch, n, nseg, exclusive,
                                                        reverse);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ceo_gather_rows(const long long* idx, const void* src, void* dst, long long n,
                               long long row_bytes, long long src_rows, cudaStream_t stream) {
  if (n <= 0 || row_bytes <= 0 || (row_bytes & 15) || row_bytes > (1ll << 30)) return -5;
  if (!aligned16(src) || !aligned16(dst)) return -2;
  gather_rows_kernel<<<grid_for(n, 8, 148 * 32), 256, 0, stream>>>(
      idx, static_cast<const uint4*>(src), static_cast<uint4*>(dst), n,
      static_cast<int>(row_bytes >> 4), src_rows);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_scatter_rows(const long long* idx, const void* src, void* dst, long long n,
                                long long row_bytes, long long dst_rows, cudaStream_t stream) {
  if (n <= 0 || row_bytes <= 0 || (row_bytes & 15) || row_bytes > (1ll << 30)) return -5;
  if (!aligned16(src) || !aligned16(dst)) return -2;
  scatter_rows_kernel<<<grid_for(n, 8, 148 * 32), 256, 0, stream>>>(
      idx, static_cast<const uint4*>(src), static_cast<uint4*>(dst), n,
      static_cast<int>(row_bytes >> 4), dst_rows);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_scatter_add_f32(const long long* idx, const float* src, float* dst, long long n,
                                   int D, long long dst_rows, cudaStream_t stream) {
  if (n <= 0 || D <= 0 || (D & 3)) return -5;
  if (!aligned16(src) || !aligned16(dst)) return -2;
  scatter_add_f32_kernel<<<grid_for(n, 8, 148 * 32), 256, 0, stream>>>(idx, src, dst, n, D,
                                                                       dst_rows);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_copy2d(const void* src, long long src_pitch, void* dst, long long dst_pitch,
                          long long rows, long long row_bytes, cudaStream_t stream) {
  if (rows <= 0 || row_bytes <= 0 || (row_bytes & 15) || (src_pitch & 15) || (dst_pitch & 15) ||
      row_bytes > (1ll << 30))
    return -5;
  if (!aligned16(src) || !aligned16(dst)) return -2;
  const long long total = rows * (row_bytes >> 4);
  copy2d_kernel<<<grid_for(total, 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const uint8_t*>(src), src_pitch, static_cast<uint8_t*>(dst), dst_pitch, rows,
      static_cast<int>(row_bytes >> 4));
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ceo_transpose16(const void* src, void* dst, int rows, int cols, long long lds,
                               long long ldd, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || lds < cols || ldd < rows) return -5;
  const dim3 g((cols + 63) / 64, (rows + 63) / 64);
  if (g.y > 65535) return -5;
  transpose16_kernel<<<g, 256, 0, stream>>>(static_cast<const uint16_t*>(src),
                                            static_cast<uint16_t*>(dst), rows, cols, lds, ldd);
  return static_cast<int>(cudaGetLastError());
}
// Exercises the recorder of the checked build: reads buf[i] for i in [0, n + extra) through
// the checked accessor (indices past n are recorded and redirected to element 0, so nothing
// outside buf is touched) and adds the sum to buf[n]: buf holds n + 1 floats.  Normal build:
// returns -1.
#ifdef CEO_BOUNDS_CHECK
__global__ void bounds_selftest_kernel(float* buf, int n, int extra) {
  float s = 0.f;
  for (int i = threadIdx.x; i < n + extra; i += blockDim.x) s += buf[CEO_IDX(i, n, 199)];
  atomicAdd(&buf[n], s);  // one element past the indexed range holds the sum
}
#endif
extern "C" int ceo_bounds_selftest(float* buf, int n, int extra, cudaStream_t stream) {
#ifdef CEO_BOUNDS_CHECK
  if (n <= 0 || extra < 0) return -5;
  bounds_selftest_kernel<<<1, 64, 0, stream>>>(buf, n, extra);
  return static_cast<int>(cudaGetLastError());
#else
  (void)buf; (void)n; (void)extra; (void)stream;
  return -1;
#endif
}

extern "C" int ceo_memset32(void* x, long long n, unsigned int value, cudaStream_t stream) {
  if (n <= 0) return -5;
  if (!aligned16(x)) return -2;
  memset32_kernel<<<grid_for(n, 1024, 148 * 16), 256, 0, stream>>>(static_cast<uint32_t*>(x), n,
                                                                   value);
  return static_cast<int>(cudaGetLastError());
}
