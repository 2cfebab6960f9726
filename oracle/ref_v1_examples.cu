/*
 * ref_v1_examples.cu -- host driver for the reference's v1-API example kernels
 * (src/examples/saxpy/saxpy_cudaDMA_kernel.cu and src/examples/saxpy_strided/saxpy_cudaDMA_kernel.cu
 * of the CudaDMA project), compiled from the sources where they lie; nothing of them is copied
 * here. TEST INFRASTRUCTURE.
 *
 * Built four times by oracle/Makefile:
 *   default                 the kernels use the reference's own cudaDMA.h   -> _ref/libv1saxpy_ref.so
 *   -DEXAMPLES_OURS         the same, unmodified kernel file uses this repository's classes through
 *                           their v1 spellings (cudaDMASequential / cudaDMAStrided without
 *                           BYTES_PER_THREAD)                               -> _ref/libv1saxpy_ours.so
 *   -DV1_EXAMPLE_STRIDED    selects the strided example (the two files reuse kernel names)
 *                                                   -> _ref/libv1saxpy_strided_{ref,ours}.so
 * As in ref_examples.cu, for the builds against this repository the reference's "#pragma once"
 * header is read first inside a namespace, so that the example's relative include of it becomes a
 * no-op and its class names resolve to this repository's.
 *
 * Launch shape and problem size follow the reference's drivers (src/examples/saxpy/saxpy_cudaDMA.cu:84-135,
 * src/examples/saxpy_strided/saxpy_cudaDMA.cu:84-135): CTA_COUNT CTAs, COMPUTE_THREADS_PER_CTA compute
 * threads plus one group of DMA_THREADS_PER_LD threads per transfer object, CTA_COUNT * NUM_ITERS *
 * COMPUTE_THREADS_PER_CTA elements; the parameters are those of the example's own params_directed.h.
 */
#include <cstdio>
#include <cuda_runtime.h>

#ifdef EXAMPLES_OURS
#include "cudadma.h"
namespace reference_header_parked {
#include "include/cudaDMA.h" /* found through -I<reference checkout> */
}
#endif

#ifdef V1_EXAMPLE_STRIDED
#include "src/examples/saxpy_strided/saxpy_cudaDMA_kernel.cu"
#else
#include "src/examples/saxpy/saxpy_cudaDMA_kernel.cu"
#endif

extern "C" {

/* elements of x and of y */
long long v1saxpy_elements(void) { return (long long)(CTA_COUNT) * (NUM_ITERS) * (COMPUTE_THREADS_PER_CTA); }

/* kernel_id 0: saxpy_cudaDMA (two transfer objects), 1: saxpy_cudaDMA_doublebuffer (four).
 * h_y = a * h_x + h_y, computed once on the device; then the same launch SAMPLES more times on a
 * scratch copy for the clock. Returns 0 or a cudaError_t. */
int v1saxpy_run(int kernel_id, float *h_y, const float *h_x, float a, float *ms_per_launch) {
  const int SAMPLES = 10;
  if (kernel_id < 0 || kernel_id > 1) return (int)cudaErrorInvalidValue;
  const size_t bytes = (size_t)v1saxpy_elements() * sizeof(float);
  const unsigned threads = (COMPUTE_THREADS_PER_CTA) + (kernel_id ? 4 : 2) * (DMA_THREADS_PER_LD);
  float *x = nullptr, *y = nullptr, *scratch = nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  cudaError_t e = cudaMalloc(&x, bytes);
  if (e == cudaSuccess) e = cudaMalloc(&y, bytes);
  if (e == cudaSuccess) e = cudaMalloc(&scratch, bytes);
  if (e == cudaSuccess) e = cudaMemcpy(x, h_x, bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(y, h_y, bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(scratch, h_y, bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaEventCreate(&t0);
  if (e == cudaSuccess) e = cudaEventCreate(&t1);
  if (e == cudaSuccess) {
    /* the kernels take a timer array that they only touch under TIMERS_ON */
    if (kernel_id) saxpy_cudaDMA_doublebuffer<<<CTA_COUNT, threads>>>(y, x, a, nullptr);
    else saxpy_cudaDMA<<<CTA_COUNT, threads>>>(y, x, a, nullptr);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(h_y, y, bytes, cudaMemcpyDeviceToHost);
  }
  if (e == cudaSuccess) {
    cudaEventRecord(t0, 0);
    for (int i = 0; i < SAMPLES; ++i) {
      if (kernel_id) saxpy_cudaDMA_doublebuffer<<<CTA_COUNT, threads>>>(scratch, x, a, nullptr);
      else saxpy_cudaDMA<<<CTA_COUNT, threads>>>(scratch, x, a, nullptr);
    }
    cudaEventRecord(t1, 0);
    e = cudaDeviceSynchronize();
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t0, t1);
    if (ms_per_launch) *ms_per_launch = ms / SAMPLES;
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
  cudaFree(x);
  cudaFree(y);
  cudaFree(scratch);
  return (int)e;
}

} /* extern "C" */
