/*
 * portable_kernels.cuh -- the benchmark workloads written against the CudaDMA
 * object API exactly as the reference offers it (no extension, dmaIDs 0..7,
 * two buffers handled the way src/examples/stencil/warp_specialized_manual_buffer.h
 * does). The same source is built twice: against cudadma.h inside the product
 * library (impl = portable) and against the reference headers as the
 * "reference CudaDMA compiled for sm_100a" baseline. The including file
 * provides the CudaDMA header and common_kernels.cuh.
 */
#ifndef CUDADMA_B200_PORTABLE_KERNELS_CUH
#define CUDADMA_B200_PORTABLE_KERNELS_CUH

#include <cuda_runtime.h>

#include "portable_stencil_math.cuh"

namespace portable {

constexpr int P_DMA = 128, P_COMPUTE = 256, P_CHUNK = 16384;

/* Sequential: 16 KiB chunks, two buffers, 4 DMA warps + 8 compute warps that
 * copy shared -> global with 16-byte accesses
 * (loop of src/perf/sequential/perf_sequential.cu:79-114 plus the write-back). */
template <int BPT>
__global__ void __launch_bounds__(P_DMA + P_COMPUTE)
seq_copy_kernel(char *__restrict__ dst, const char *__restrict__ src, const long long nchunks) {
  extern __shared__ float4 pbuf[];
  float4 *buf0 = pbuf, *buf1 = pbuf + P_CHUNK / 16;
  CudaDMASequential<true, 16, BPT, P_CHUNK, P_DMA> d0(1, P_COMPUTE, P_COMPUTE);
  CudaDMASequential<true, 16, BPT, P_CHUNK, P_DMA> d1(2, P_COMPUTE, P_COMPUTE);
  const long long stride = gridDim.x;
  if (d0.owns_this_thread()) {
    for (long long c = blockIdx.x; c < nchunks; c += 2 * stride) {
      d0.execute_dma(src + c * P_CHUNK, buf0);
      if (c + stride < nchunks) d1.execute_dma(src + (c + stride) * P_CHUNK, buf1);
    }
  } else {
    if (blockIdx.x < nchunks) d0.start_async_dma();
    if (blockIdx.x + stride < nchunks) d1.start_async_dma();
    for (long long c = blockIdx.x; c < nchunks; c += 2 * stride) {
      d0.wait_for_dma_finish();
      float4 *o = reinterpret_cast<float4 *>(dst + c * P_CHUNK);
#pragma unroll
      for (int i = threadIdx.x; i < P_CHUNK / 16; i += P_COMPUTE) o[i] = buf0[i];
      if (c + 2 * stride < nchunks) d0.start_async_dma();
      if (c + stride < nchunks) {
        d1.wait_for_dma_finish();
        o = reinterpret_cast<float4 *>(dst + (c + stride) * P_CHUNK);
#pragma unroll
        for (int i = threadIdx.x; i < P_CHUNK / 16; i += P_COMPUTE) o[i] = buf1[i];
        if (c + 3 * stride < nchunks) d1.start_async_dma();
      }
    }
  }
}

/* Strided: 128 x 64 fp32 tiles into a shared buffer whose rows are padded to
 * 272 bytes (the dst_stride argument), so that the transposing reads of eight
 * consecutive rows fall in eight bank groups; two buffers. */
constexpr int PT_ROWS = 128, PT_COLS = 64, PT_PITCH = 272, PT_BUF = PT_ROWS * PT_PITCH;

template <int BPT>
__device__ __forceinline__ void transpose_drain(const unsigned char *tile, float *__restrict__ out, const int rows,
                                                const int tx, const int ty) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rot = (lane >> 1) & 3;
#pragma unroll
  for (int k = warp; k < PT_COLS / 4; k += P_COMPUTE / 32) {
    float4 v[4], w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * lane + ((i + rot) & 3);
      v[i] = *reinterpret_cast<const float4 *>(tile + r * PT_PITCH + 16 * k);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = (j - rot) & 3;
      w[j] = (i == 0) ? v[0] : (i == 1) ? v[1] : (i == 2) ? v[2] : v[3];
    }
    float *o = out + ((long long)tx * PT_COLS + 4 * k) * rows + (long long)ty * PT_ROWS + 4 * lane;
    *reinterpret_cast<float4 *>(o) = make_float4(w[0].x, w[1].x, w[2].x, w[3].x);
    *reinterpret_cast<float4 *>(o + rows) = make_float4(w[0].y, w[1].y, w[2].y, w[3].y);
    *reinterpret_cast<float4 *>(o + 2ll * rows) = make_float4(w[0].z, w[1].z, w[2].z, w[3].z);
    *reinterpret_cast<float4 *>(o + 3ll * rows) = make_float4(w[0].w, w[1].w, w[2].w, w[3].w);
  }
}

template <int BPT>
__global__ void __launch_bounds__(P_DMA + P_COMPUTE)
transpose_kernel(float *__restrict__ out, const float *__restrict__ in, const int rows, const int cols) {
  extern __shared__ float4 pbuf[];
  unsigned char *buf0 = reinterpret_cast<unsigned char *>(pbuf), *buf1 = buf0 + PT_BUF;
  CudaDMAStrided<true, 16, BPT, PT_COLS * 4, P_DMA, PT_ROWS> d0(1, P_COMPUTE, P_COMPUTE, cols * 4, PT_PITCH);
  CudaDMAStrided<true, 16, BPT, PT_COLS * 4, P_DMA, PT_ROWS> d1(2, P_COMPUTE, P_COMPUTE, cols * 4, PT_PITCH);
  const int tiles_x = cols / PT_COLS;
  const long long ntiles = (long long)tiles_x * (rows / PT_ROWS);
  const long long stride = gridDim.x;
  if (d0.owns_this_thread()) {
    for (long long t = blockIdx.x; t < ntiles; t += 2 * stride) {
      long long ty = t / tiles_x, tx = t - ty * tiles_x;
      d0.execute_dma(in + (ty * PT_ROWS) * cols + tx * PT_COLS, buf0);
      if (t + stride < ntiles) {
        ty = (t + stride) / tiles_x; tx = (t + stride) - ty * tiles_x;
        d1.execute_dma(in + (ty * PT_ROWS) * cols + tx * PT_COLS, buf1);
      }
    }
  } else {
    if (blockIdx.x < ntiles) d0.start_async_dma();
    if (blockIdx.x + stride < ntiles) d1.start_async_dma();
    for (long long t = blockIdx.x; t < ntiles; t += 2 * stride) {
      long long ty = t / tiles_x, tx = t - ty * tiles_x;
      d0.wait_for_dma_finish();
      transpose_drain<BPT>(buf0, out, rows, (int)tx, (int)ty);
      if (t + 2 * stride < ntiles) d0.start_async_dma();
      if (t + stride < ntiles) {
        ty = (t + stride) / tiles_x; tx = (t + stride) - ty * tiles_x;
        d1.wait_for_dma_finish();
        transpose_drain<BPT>(buf1, out, rows, (int)tx, (int)ty);
        if (t + 3 * stride < ntiles) d1.start_async_dma();
      }
    }
  }
}


/* Stencil: the reference's stencil example (src/examples/stencil/warp_specialized_manual_buffer.h:
 * one compute thread per point of a 32 x 16 tile, two CudaDMAStrided objects loading the tile with its
 * halo, plane after plane, from an array padded with zero cells as src/examples/stencil/cudaDMA_stencil2D.cu:86-97
 * pads it) with the in-plane average replaced by the radius-4 25-point operator: the z neighbours live in
 * a per-thread register queue that each thread refills from global memory.
 * Padded layout: grid cell (x, y, z) is element ((z + 4) * py + (y + 4)) * px + (x + 4), px = nx + 8,
 * py = ny + 8, all border cells zero. Needs nx % 32 == 0 and ny % 16 == 0. */
/* tile shape, coefficients and the per-point arithmetic: portable_stencil_math.cuh */
template <int BPT>
__global__ void __launch_bounds__(PS_COMPUTE + PS_DMA)
stencil_kernel(float *__restrict__ out, const float *__restrict__ in, const int px, const int py, const int z_begin,
               const int z_end, const int z_chunk, const PCoeffs k) {
  __shared__ __align__(128) float buf0[PS_WX * PS_WY];
  __shared__ __align__(128) float buf1[PS_WX * PS_WY];
  CudaDMAStrided<true, 16, BPT, PS_WX * 4, PS_DMA, PS_WY> d0(1, PS_COMPUTE, PS_COMPUTE, px * 4, PS_WX * 4);
  CudaDMAStrided<true, 16, BPT, PS_WX * 4, PS_DMA, PS_WY> d1(2, PS_COMPUTE, PS_COMPUTE, px * 4, PS_WX * 4);
  const int x0 = blockIdx.x * PS_TX, y0 = blockIdx.y * PS_TY;
  const int z0 = z_begin + blockIdx.z * z_chunk;
  const int depth = (z_end - z0 < z_chunk) ? (z_end - z0) : z_chunk;
  const long long slice = (long long)px * py;
  if (d0.owns_this_thread()) {
    const float *win = in + (long long)(z0 + PS_R) * slice + (long long)y0 * px + x0;
    for (int i = 0; i < depth; i += 2) {
      d0.execute_dma(win, buf0);
      win += slice;
      if (i + 1 < depth) {
        d1.execute_dma(win, buf1);
        win += slice;
      }
    }
  } else {
    const int tx = threadIdx.x % PS_TX, ty = threadIdx.x / PS_TX;
    const long long cell = (long long)(z0 + PS_R) * slice + (long long)(y0 + ty + PS_R) * px + (x0 + tx + PS_R);
    const float *p = in + cell;
    float *o = out + cell;
    const float *w0 = buf0 + (ty + PS_R) * PS_WX + tx + PS_R;
    const float *w1 = buf1 + (ty + PS_R) * PS_WX + tx + PS_R;
    float b[4], f[4], cur = p[0];
#pragma unroll
    for (int r = 1; r <= PS_R; ++r) { b[r - 1] = p[-r * slice]; f[r - 1] = p[r * slice]; }
    d0.start_async_dma();
    if (depth > 1) d1.start_async_dma();
    for (int i = 0; i < depth; i += 2) {
      /* plane z + 5, the next front value, fetched early; not needed (and not there) after the last plane */
      const float n0 = (i + 1 < depth) ? p[(PS_R + 1) * slice] : 0.0f;
      d0.wait_for_dma_finish();
      o[0] = stencil_point(w0, cur, b, f, k);
      if (i + 2 < depth) d0.start_async_dma();
      b[3] = b[2]; b[2] = b[1]; b[1] = b[0]; b[0] = cur; cur = f[0]; f[0] = f[1]; f[1] = f[2]; f[2] = f[3]; f[3] = n0;
      p += slice; o += slice;
      if (i + 1 < depth) {
        const float n1 = (i + 2 < depth) ? p[(PS_R + 1) * slice] : 0.0f;
        d1.wait_for_dma_finish();
        o[0] = stencil_point(w1, cur, b, f, k);
        if (i + 3 < depth) d1.start_async_dma();
        b[3] = b[2]; b[2] = b[1]; b[1] = b[0]; b[0] = cur; cur = f[0]; f[0] = f[1]; f[1] = f[2]; f[2] = f[3]; f[3] = n1;
        p += slice; o += slice;
      }
    }
  }
}

/* ---- launchers: return a cudaError_t as int (0 = launched) ---- */

template <int BPT = 64>
inline int launch_seq_copy(char *dst, const char *src, long long nchunks, int sms, cudaStream_t s) {
  auto k = seq_copy_kernel<BPT>;
  /* one resident wave of at most four CTAs per SM (32 KiB of shared memory and 384 threads per CTA;
   * a large register budget per DMA thread leaves room for three) */
  int fit = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, k, P_DMA + P_COMPUTE, 2 * P_CHUNK);
  if (e != cudaSuccess) return (int)e;
  if (fit < 1) fit = 1;
  if (fit > 4) fit = 4;
  const long long want = (long long)fit * sms;
  const int grid = (int)(nchunks < want ? nchunks : want);
  k<<<grid, P_DMA + P_COMPUTE, 2 * P_CHUNK, s>>>(dst, src, nchunks);
  return (int)cudaGetLastError();
}

template <int BPT = 64>
inline int launch_transpose(float *dst, const float *src, int rows, int cols, int sms, cudaStream_t s) {
  auto k = transpose_kernel<BPT>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * PT_BUF);
  if (e != cudaSuccess) return (int)e;
  const long long ntiles = (long long)(rows / PT_ROWS) * (cols / PT_COLS);
  const long long want = 3ll * sms;
  const int grid = (int)(ntiles < want ? ntiles : want);
  k<<<grid, P_DMA + P_COMPUTE, 2 * PT_BUF, s>>>(dst, src, rows, cols);
  return (int)cudaGetLastError();
}

template <int RECORD_BYTES = 32, int BPT = 64>
inline int launch_gather_scatter(char *out, const char *table, const int *gidx, const int *sidx, long long nbuf,
                                 int sms, cudaStream_t s) {
  using namespace cudadma_b200::kernels;
  constexpr int STAGES = 4; /* dmaIDs 0..3 gather, 4..7 scatter: all sixteen named barriers of the reference */
  constexpr int SMEM = STAGES * 128 * RECORD_BYTES;
  auto k = gather_scatter_kernel<RECORD_BYTES, 128, STAGES, BPT>;
  if (SMEM > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  /* one resident wave: a CTA keeps its share of the buffers to itself, so CTAs that only start
   * when others have finished would run the tail of the job at a fraction of the occupancy */
  int fit = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, k, GS_THREADS, SMEM);
  if (e != cudaSuccess) return (int)e;
  if (fit < 1) fit = 1;
  const long long want = (long long)fit * sms;
  const int grid = (int)(nbuf < want ? nbuf : want);
  k<<<grid, GS_THREADS, SMEM, s>>>(out, table, gidx, sidx, nbuf);
  return (int)cudaGetLastError();
}

/* padded arrays (see stencil_kernel); output planes [z_begin, z_end) of the nx x ny x nz grid */
template <int BPT = 64>
inline int launch_stencil_padded(float *out, const float *in, int nx, int ny, int nz, int z_begin, int z_end,
                                 const float coeff[5], int z_chunk, int sms, cudaStream_t s) {
  if (nx % PS_TX || ny % PS_TY || z_begin < 0 || z_end > nz || z_begin >= z_end) return (int)cudaErrorInvalidValue;
  PCoeffs k;
  for (int i = 0; i < 5; ++i) k.c[i] = coeff[i];
  const int depth = z_end - z_begin;
  const long long tiles = (long long)(nx / PS_TX) * (ny / PS_TY);
  if (z_chunk <= 0) {
    const long long want = 12ll * sms;
    long long chunks = (want + tiles - 1) / tiles;
    if (chunks < 1) chunks = 1;
    z_chunk = (int)((depth + chunks - 1) / chunks);
    if (z_chunk < 16) z_chunk = 16;
    if (z_chunk > depth) z_chunk = depth;
  }
  dim3 grid(nx / PS_TX, ny / PS_TY, (depth + z_chunk - 1) / z_chunk);
  stencil_kernel<BPT><<<grid, PS_COMPUTE + PS_DMA, 0, s>>>(out, in, nx + 2 * PS_R, ny + 2 * PS_R, z_begin, z_end,
                                                          z_chunk, k);
  return (int)cudaGetLastError();
}

}  // namespace portable

#endif
