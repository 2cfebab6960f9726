/*
 * ref_halo_stencil.cu -- the radius-4 25-point stencil step with its tile loaded the way the
 * reference's classes offer for a halo: the ring of a 32 x 16 tile by v1 cudaDMAHalo
 * (include/cudaDMA.h:3653-3692 of the CudaDMA project; ring only, no corners) and the tile's
 * interior by cudaDMAStrided, from arrays padded with four zero cells on every side
 * (src/examples/stencil/cudaDMA_stencil2D.cu:86-97). The halo class exists in the v1 header only, and
 * that header cannot share a translation unit with cudaDMAv2.h (both define the same barrier
 * helpers), hence this file of its own and the v1 strided class for the interior.
 * TEST INFRASTRUCTURE: second form of the "reference CudaDMA build" stencil baseline.
 *
 * Built twice by oracle/Makefile: `#include "cudaDMA.h"` finds the reference's header
 * (-> _ref/libhalo_stencil_ref.so) or this repository's shim of that name
 * (-> _ref/libhalo_stencil_ours.so); the kernel source is the same.
 *
 * One CTA: 512 compute threads (one per point), two warps that fill the rings of two buffers, two
 * warps that fill their interiors; the z neighbours live in a per-thread register queue refilled
 * from global memory, as in portable::stencil_kernel, whose arithmetic this kernel shares
 * (portable_stencil_math.cuh), so the two give the same bits.
 */
#include <cuda_runtime.h>

#include "cudaDMA.h"

#include "portable_stencil_math.cuh"

namespace {
using namespace portable;
constexpr int HS_RING_THREADS = 64, HS_IN_THREADS = 64;
constexpr int HS_THREADS = PS_COMPUTE + HS_RING_THREADS + HS_IN_THREADS;

__global__ void __launch_bounds__(HS_THREADS)
halo_stencil_kernel(float *__restrict__ out, const float *__restrict__ in, const int px, const int py, const int z_begin,
                    const int z_end, const int z_chunk, const PCoeffs k) {
  __shared__ __align__(128) float buf0[PS_WX * PS_WY];
  __shared__ __align__(128) float buf1[PS_WX * PS_WY];
  cudaDMAHalo<float, PS_R, false, 16> r0(1, HS_RING_THREADS, PS_COMPUTE, PS_COMPUTE, PS_TX, PS_TY, px);
  cudaDMAHalo<float, PS_R, false, 16> r1(2, HS_RING_THREADS, PS_COMPUTE, PS_COMPUTE, PS_TX, PS_TY, px);
  cudaDMAStrided<true, 16, PS_TX * 4, HS_IN_THREADS, PS_TY> c0(3, PS_COMPUTE, PS_COMPUTE + HS_RING_THREADS, px * 4, PS_WX * 4);
  cudaDMAStrided<true, 16, PS_TX * 4, HS_IN_THREADS, PS_TY> c1(4, PS_COMPUTE, PS_COMPUTE + HS_RING_THREADS, px * 4, PS_WX * 4);
  const int x0 = blockIdx.x * PS_TX, y0 = blockIdx.y * PS_TY;
  const int z0 = z_begin + blockIdx.z * z_chunk;
  const int depth = (z_end - z0 < z_chunk) ? (z_end - z0) : z_chunk;
  const long long slice = (long long)px * py;
  /* interior origin of the tile in plane z0 of the padded array, and in a buffer */
  const float *origin = in + (long long)(z0 + PS_R) * slice + (long long)(y0 + PS_R) * px + (x0 + PS_R);
  float *const o0 = buf0 + PS_R * PS_WX + PS_R, *const o1 = buf1 + PS_R * PS_WX + PS_R;
  if (r0.owns_this_thread()) {
    for (int i = 0; i < depth; i += 2) {
      r0.execute_dma(origin, o0);
      origin += slice;
      if (i + 1 < depth) {
        r1.execute_dma(origin, o1);
        origin += slice;
      }
    }
  } else if (c0.owns_this_thread()) {
    for (int i = 0; i < depth; i += 2) {
      c0.execute_dma(origin, o0);
      origin += slice;
      if (i + 1 < depth) {
        c1.execute_dma(origin, o1);
        origin += slice;
      }
    }
  } else {
    const int tx = threadIdx.x % PS_TX, ty = threadIdx.x / PS_TX;
    const float *p = origin + (long long)ty * px + tx;
    float *o = out + (p - in);
    const float *w0 = o0 + ty * PS_WX + tx, *w1 = o1 + ty * PS_WX + tx;
    float b[4], f[4], cur = p[0];
#pragma unroll
    for (int r = 1; r <= PS_R; ++r) { b[r - 1] = p[-r * slice]; f[r - 1] = p[r * slice]; }
    r0.start_async_dma(); c0.start_async_dma();
    if (depth > 1) { r1.start_async_dma(); c1.start_async_dma(); }
    for (int i = 0; i < depth; i += 2) {
      const float n0 = (i + 1 < depth) ? p[(PS_R + 1) * slice] : 0.0f;
      r0.wait_for_dma_finish(); c0.wait_for_dma_finish();
      o[0] = stencil_point(w0, cur, b, f, k);
      if (i + 2 < depth) { r0.start_async_dma(); c0.start_async_dma(); }
      advance_queue(b, cur, f, n0);
      p += slice; o += slice;
      if (i + 1 < depth) {
        const float n1 = (i + 2 < depth) ? p[(PS_R + 1) * slice] : 0.0f;
        r1.wait_for_dma_finish(); c1.wait_for_dma_finish();
        o[0] = stencil_point(w1, cur, b, f, k);
        if (i + 3 < depth) { r1.start_async_dma(); c1.start_async_dma(); }
        advance_queue(b, cur, f, n1);
        p += slice; o += slice;
      }
    }
  }
}
}  // namespace

extern "C" {

/* arrays padded by four zero cells on every side: (nx + 8) x (ny + 8) x (nz + 8) floats; output planes
 * [z_begin, z_end); z_chunk = planes per CTA (0: chosen here). Returns 0 or a cudaError_t. */
int halo_stencil25_step_padded(float *out, const float *in, int nx, int ny, int nz, int z_begin, int z_end,
                               const float coeff[5], int z_chunk, void *stream) {
  if (nx % PS_TX || ny % PS_TY || z_begin < 0 || z_end > nz || z_begin >= z_end) return (int)cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
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
  halo_stencil_kernel<<<grid, HS_THREADS, 0, (cudaStream_t)stream>>>(out, in, nx + 2 * PS_R, ny + 2 * PS_R, z_begin, z_end,
                                                                     z_chunk, k);
  return (int)cudaGetLastError();
}

#ifdef CUDADMA_B200_CUDADMA_H
/* reads and clears the status word of this library's kernels (0: no wait gave up) */
int halo_stencil_status(unsigned int *out) { return (int)cudadma_b200::read_status(out, 0); }
#endif

} /* extern "C" */
