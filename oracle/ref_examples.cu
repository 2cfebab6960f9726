/*
 * ref_examples.cu -- host driver for the reference's five stencil example kernels
 * (src/examples/stencil/warp_specialized_{single,double,manual}_buffer.h and
 * non_warp_specialized_{single,double}_buffer.h of the CudaDMA project), compiled from the
 * sources where they lie; nothing of them is copied here. TEST INFRASTRUCTURE.
 *
 * Built twice by oracle/Makefile:
 *   default          the kernels use the reference's own cudaDMAv2.h  -> _ref/libexamples_ref.so
 *   -DEXAMPLES_OURS  the same, unmodified kernel files use this repository's classes
 *                                                                    -> _ref/libexamples_ours.so
 * The example files include the reference header by a relative path, and that header is
 * "#pragma once". For the second build it is therefore read first, inside a namespace of its
 * own: its classes stay out of the global namespace, the examples' include of it becomes a
 * no-op, and the names the kernels use (CudaDMAStrided, ...) resolve to this repository's.
 *
 * The launch shape and the padded layout follow the reference's driver
 * (src/examples/stencil/cudaDMA_stencil2D.cu:86-218); sizes are run-time arguments here, the
 * template parameters are the reference's defaults (params_directed.h:17-24).
 */
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#ifdef EXAMPLES_OURS
#include "cudadma.h"
namespace reference_header_parked {
#include "include/cudaDMAv2.h" /* found through -I<reference checkout> */
}
#define ENTRY(name) examples_ours_##name
#else
#define ENTRY(name) examples_ref_##name
#endif

#include "warp_specialized_single_buffer.h"
#include "warp_specialized_double_buffer.h"
#include "warp_specialized_manual_buffer.h"
#include "non_warp_specialized_single_buffer.h"
#include "non_warp_specialized_double_buffer.h"

namespace {
constexpr int TILE_X = 32, TILE_Y = 4, RADIUS = 4, DMA_WARPS = 1, BPT = 12 * 16, ALIGN = 16;
constexpr int SAMPLES = 20;

void launch(int id, const float2 *src, float2 *dst, int offset, int row_stride, int slice_stride, int dim_z,
            dim3 grid, cudaStream_t s) {
  const unsigned compute = TILE_X * TILE_Y;
  switch (id) {
    case 0:
      stencil_2D_warp_specialized_single_buffer<ALIGN, BPT, TILE_X, TILE_Y, RADIUS, DMA_WARPS * 32>
          <<<grid, compute + DMA_WARPS * 32, 0, s>>>(src, dst, offset, row_stride, slice_stride, dim_z);
      break;
    case 1:
      stencil_2D_warp_specialized_double_buffer<ALIGN, BPT, TILE_X, TILE_Y, RADIUS, DMA_WARPS * 32>
          <<<grid, compute + 2 * DMA_WARPS * 32, 0, s>>>(src, dst, offset, row_stride, slice_stride, dim_z);
      break;
    case 2:
      stencil_2D_warp_specialized_manual_buffer<ALIGN, BPT, TILE_X, TILE_Y, RADIUS, DMA_WARPS * 32>
          <<<grid, compute + DMA_WARPS * 32, 0, s>>>(src, dst, offset, row_stride, slice_stride, dim_z);
      break;
    case 3:
      stencil_2D_non_warp_specialized_single_buffer<ALIGN, BPT, TILE_X, TILE_Y, RADIUS>
          <<<grid, compute, 0, s>>>(src, dst, offset, row_stride, slice_stride, dim_z);
      break;
    default:
      stencil_2D_non_warp_specialized_double_buffer<ALIGN, BPT, TILE_X, TILE_Y, RADIUS>
          <<<grid, compute, 0, s>>>(src, dst, offset, row_stride, slice_stride, dim_z);
      break;
  }
}
}  // namespace

extern "C" {

int ENTRY(num_kernels)(void) { return 5; }

/* h_src, h_dst: padded arrays of (dim_x + 8) * (dim_y + 8) * (dim_z + 8) float2, x fastest.
 * Runs kernel `id` once into a zeroed destination (copied back to h_dst), then SAMPLES more
 * times for the clock; *ms_per_launch gets the mean. Returns 0 or a cudaError_t. */
int ENTRY(run)(int id, const float *h_src, float *h_dst, int dim_x, int dim_y, int dim_z, float *ms_per_launch) {
  if (id < 0 || id > 4 || dim_x % TILE_X || dim_y % TILE_Y || dim_z % 2 || dim_z < 4) return (int)cudaErrorInvalidValue;
  const int row_stride = dim_x + 2 * RADIUS;
  const int slice_stride = (dim_y + 2 * RADIUS) * row_stride;
  const size_t cells = (size_t)slice_stride * (dim_z + 2 * RADIUS);
  const int offset = RADIUS * slice_stride + RADIUS * row_stride + RADIUS;
  float2 *src = nullptr, *dst = nullptr;
  cudaError_t e = cudaMalloc(&src, cells * sizeof(float2));
  if (e == cudaSuccess) e = cudaMalloc(&dst, cells * sizeof(float2));
  if (e == cudaSuccess) e = cudaMemcpy(src, h_src, cells * sizeof(float2), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(dst, 0, cells * sizeof(float2));
  cudaStream_t s = nullptr;
  if (e == cudaSuccess) e = cudaStreamCreate(&s);
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (e == cudaSuccess) e = cudaEventCreate(&t0);
  if (e == cudaSuccess) e = cudaEventCreate(&t1);
  if (e == cudaSuccess) {
    dim3 grid(dim_x / TILE_X, dim_y / TILE_Y);
    launch(id, src, dst, offset, row_stride, slice_stride, dim_z, grid, s);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess) e = cudaMemcpy(h_dst, dst, cells * sizeof(float2), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) {
      cudaEventRecord(t0, s);
      for (int i = 0; i < SAMPLES; ++i) launch(id, src, dst, offset, row_stride, slice_stride, dim_z, grid, s);
      cudaEventRecord(t1, s);
      e = cudaStreamSynchronize(s);
      float ms = 0.f;
      if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t0, t1);
      if (ms_per_launch) *ms_per_launch = ms / SAMPLES;
    }
  }
#ifdef EXAMPLES_OURS
  if (e == cudaSuccess) {
    unsigned int w = 0;
    e = cudadma_b200::read_status(&w, 0);
    if (e == cudaSuccess && w) e = cudaErrorLaunchTimeout; /* a bounded wait inside a kernel gave up */
  }
#endif
  if (t0) cudaEventDestroy(t0);
  if (t1) cudaEventDestroy(t1);
  if (s) cudaStreamDestroy(s);
  cudaFree(src);
  cudaFree(dst);
  return (int)e;
}

} /* extern "C" */
