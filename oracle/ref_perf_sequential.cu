/*
 * ref_perf_sequential.cu -- host driver for the reference's throughput benchmark
 * (src/perf/sequential/perf_sequential.cu of the CudaDMA project: kernels non_specialized,
 * single_buffer, double_buffer and manual_buffer, :52-223), compiled from the source where it
 * lies; nothing of it is copied here. TEST INFRASTRUCTURE.
 *
 * Built twice by oracle/Makefile: with the reference's include directory first, the file's
 * `#include "cudaDMA.h"` finds the reference's v1 header (-> _ref/libperfseq_ref.so); with this
 * repository's include/cudadma first it finds the shim of the same name and the kernels use this
 * repository's classes through their v1 spellings (-> _ref/libperfseq_ours.so). The reference
 * file's own main() is renamed out of the way; launch shapes, sizes and the bandwidth formula are
 * those of its performance_test (:225-360) with the parameters of its params_directed.h.
 */
#include <cuda_runtime.h>

#define main cudadma_reference_perf_sequential_main
#include "src/perf/sequential/perf_sequential.cu" /* found through -I<reference checkout> */
#undef main

extern "C" {

/* kernel_id 0 non_specialized, 1 single_buffer, 2 double_buffer, 3 manual_buffer.
 * Returns 0 or a cudaError_t; *gbs = bytes loaded / mean launch time (perf_sequential.cu:355-360). */
int perfseq_run(int kernel_id, double *gbs, double *ms_per_launch) {
  const int SAMPLES = 10;
  if (kernel_id < 0 || kernel_id > 3) return (int)cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
  const int compute_warps = 1, dma_threads = (PARAM_DMA_WARPS) * WARP_SIZE;
  const int total_ctas = sms * (PARAM_CTA_PER_SM);
  const size_t total_mem = (size_t)total_ctas * (PARAM_ELMT_SIZE) * (PARAM_LOOP_ITERS);
  PARAM_ELMT_TYPE *d_src = nullptr, *d_dst = nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  e = cudaMalloc(&d_src, total_mem);
  if (e == cudaSuccess) e = cudaMalloc(&d_dst, 4096);
  if (e == cudaSuccess) e = cudaMemset(d_src, 0, total_mem);
  if (e == cudaSuccess) e = cudaEventCreate(&t0);
  if (e == cudaSuccess) e = cudaEventCreate(&t1);
  for (int i = 0; i <= SAMPLES && e == cudaSuccess; ++i) {
    if (i == 1) e = cudaEventRecord(t0, 0); /* launch 0 is the warm-up */
    switch (kernel_id) {
      case 0:
        non_specialized<PARAM_ELMT_TYPE, PARAM_ALIGNMENT, PARAM_ELMT_SIZE, (PARAM_DMA_WARPS) * WARP_SIZE, PARAM_LOOP_ITERS>
            <<<total_ctas, dma_threads>>>(d_src, d_dst, false);
        break;
      case 1:
        single_buffer<PARAM_ELMT_TYPE, PARAM_ALIGNMENT, PARAM_ELMT_SIZE, (PARAM_DMA_WARPS) * WARP_SIZE, PARAM_LOOP_ITERS>
            <<<total_ctas, dma_threads + compute_warps * WARP_SIZE>>>(d_src, d_dst, compute_warps * WARP_SIZE, false);
        break;
      case 2:
        double_buffer<PARAM_ELMT_TYPE, PARAM_ALIGNMENT, PARAM_ELMT_SIZE, (PARAM_DMA_WARPS) * WARP_SIZE, PARAM_LOOP_ITERS>
            <<<total_ctas, 2 * dma_threads + compute_warps * WARP_SIZE>>>(d_src, d_dst, compute_warps * WARP_SIZE, false);
        break;
      default:
        manual_buffer<PARAM_ELMT_TYPE, PARAM_ALIGNMENT, PARAM_ELMT_SIZE, (PARAM_DMA_WARPS) * WARP_SIZE, PARAM_LOOP_ITERS>
            <<<total_ctas, dma_threads + compute_warps * WARP_SIZE>>>(d_src, d_dst, compute_warps * WARP_SIZE, false);
        break;
    }
    if (e == cudaSuccess) e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaEventRecord(t1, 0);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t0, t1);
  if (e == cudaSuccess) {
    if (ms_per_launch) *ms_per_launch = ms / SAMPLES;
    if (gbs) *gbs = (double)total_mem / (double)(ms / SAMPLES) * 1e-6;
  }
#ifdef CUDADMA_B200_CUDADMA_H
  if (e == cudaSuccess) {
    unsigned int w = 0;
    e = cudadma_b200::read_status(&w, 0);
    if (e == cudaSuccess && w) e = cudaErrorLaunchTimeout; /* a bounded wait inside a kernel gave up */
  }
#endif
  if (t0) cudaEventDestroy(t0);
  if (t1) cudaEventDestroy(t1);
  cudaFree(d_src);
  cudaFree(d_dst);
  return (int)e;
}

} /* extern "C" */
