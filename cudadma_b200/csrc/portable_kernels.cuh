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

/* ---- launchers: return a cudaError_t as int (0 = launched) ---- */

inline int launch_seq_copy(char *dst, const char *src, long long nchunks, int sms, cudaStream_t s) {
  auto k = seq_copy_kernel<64>;
  const long long want = 4ll * sms; /* 32 KiB of shared memory and 384 threads per CTA */
  const int grid = (int)(nchunks < want ? nchunks : want);
  k<<<grid, P_DMA + P_COMPUTE, 2 * P_CHUNK, s>>>(dst, src, nchunks);
  return (int)cudaGetLastError();
}

inline int launch_transpose(float *dst, const float *src, int rows, int cols, int sms, cudaStream_t s) {
  auto k = transpose_kernel<64>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * PT_BUF);
  if (e != cudaSuccess) return (int)e;
  const long long ntiles = (long long)(rows / PT_ROWS) * (cols / PT_COLS);
  const long long want = 3ll * sms;
  const int grid = (int)(ntiles < want ? ntiles : want);
  k<<<grid, P_DMA + P_COMPUTE, 2 * PT_BUF, s>>>(dst, src, rows, cols);
  return (int)cudaGetLastError();
}

inline int launch_gather_scatter(char *out, const char *table, const int *gidx, const int *sidx, long long nbuf,
                                 int sms, cudaStream_t s) {
  using namespace cudadma_b200::kernels;
  constexpr int STAGES = 4; /* dmaIDs 0..3 gather, 4..7 scatter: all sixteen named barriers of the reference */
  auto k = gather_scatter_kernel<32, 128, STAGES>;
  const long long want = 6ll * sms;
  const int grid = (int)(nbuf < want ? nbuf : want);
  k<<<grid, GS_THREADS, STAGES * 128 * 32, s>>>(out, table, gidx, sidx, nbuf);
  return (int)cudaGetLastError();
}

}  // namespace portable

#endif
