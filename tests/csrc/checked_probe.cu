/*
 * checked_probe.cu -- the -DCUDADMA_CHECKED build of the header on one small kernel: a
 * warp-specialised CudaDMASequential and a CudaDMAStrided load `count` floats (as `rows` runs) from
 * src + offset into shared memory, the compute threads write the buffer out. The host names
 * [src, src + window) as the only range transfers may touch; the allocation behind it is larger,
 * so a run outside the window is still inside the allocation: nothing here can fault whether
 * or not the check does its job. TEST INFRASTRUCTURE.
 */
#define CUDADMA_CHECKED
#include "cudadma.h"

namespace {
constexpr int DMA = 32, COMPUTE = 64, MAX_FLOATS = 2048;

__global__ void probe_kernel(const float *src, float *out, int count, int rows, int src_stride_floats) {
  __shared__ __align__(128) float buf[MAX_FLOATS];
  for (int i = threadIdx.x; i < MAX_FLOATS; i += blockDim.x) buf[i] = -1.0f; /* what an unfilled buffer holds */
  __syncthreads();
  if (rows <= 1) {
    CudaDMASequential<true, 4, 16> dma(0, DMA, COMPUTE, COMPUTE, count * 4);
    if (dma.owns_this_thread()) {
      dma.execute_dma(src, buf);
    } else {
      dma.start_async_dma();
      dma.wait_for_dma_finish();
      for (int i = threadIdx.x; i < count; i += COMPUTE) out[i] = buf[i];
    }
  } else {
    const int per_row = count / rows;
    CudaDMAStrided<true, 4, 16> dma(1, DMA, COMPUTE, COMPUTE, per_row * 4, rows, src_stride_floats * 4, per_row * 4);
    if (dma.owns_this_thread()) {
      dma.execute_dma(src, buf);
    } else {
      dma.start_async_dma();
      dma.wait_for_dma_finish();
      for (int i = threadIdx.x; i < count; i += COMPUTE) out[i] = buf[i];
    }
  }
}
}  // namespace

extern "C" {

/* h_src: alloc_floats floats. Transfers may touch floats [0, window_floats) of the device copy only.
 * The kernel loads `count` floats starting at float `offset` (as `rows` runs `stride` floats apart when
 * rows > 1) and writes them to h_out. status: the device status word; kind / address_off / bytes: the
 * recorded refusal (kind 0 = none; address_off in bytes from the start of the device copy).
 * Returns 0 or a cudaError_t. */
int checked_probe_run(const float *h_src, int alloc_floats, int window_floats, int offset, int count, int rows,
                      int stride, float *h_out, unsigned int *status, unsigned int *kind, long long *address_off,
                      unsigned long long *bytes) {
  if (count <= 0 || count > MAX_FLOATS || rows < 1 || count % rows) return (int)cudaErrorInvalidValue;
  const long long last = (long long)offset + (rows > 1 ? (long long)(rows - 1) * stride + count / rows : count);
  if (offset < 0 || last > alloc_floats || window_floats > alloc_floats) return (int)cudaErrorInvalidValue;
  float *src = nullptr, *out = nullptr;
  cudaError_t e = cudaMalloc(&src, (size_t)alloc_floats * 4);
  if (e == cudaSuccess) e = cudaMalloc(&out, (size_t)MAX_FLOATS * 4);
  if (e == cudaSuccess) e = cudaMemcpy(src, h_src, (size_t)alloc_floats * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(out, 0, (size_t)MAX_FLOATS * 4);
  if (e == cudaSuccess) {
    const void *bases[1] = {src};
    const size_t lens[1] = {(size_t)window_floats * 4};
    e = cudadma_b200::checked::set_windows(bases, lens, 1);
  }
  if (e == cudaSuccess) {
    probe_kernel<<<1, DMA + COMPUTE>>>(src + offset, out, count, rows, stride);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(h_out, out, (size_t)count * 4, cudaMemcpyDeviceToHost);
  cudadma_b200::checked::Violation v = {0, 0, 0, 0, 0, 0};
  if (e == cudaSuccess) e = cudadma_b200::read_status(status, 0);
  if (e == cudaSuccess) e = cudadma_b200::checked::read_violation(&v, 0);
  if (e == cudaSuccess) {
    *kind = v.kind;
    *bytes = v.bytes;
    *address_off = v.kind ? (long long)(v.address - (unsigned long long)reinterpret_cast<uintptr_t>(src)) : 0;
  }
  cudaFree(src);
  cudaFree(out);
  return (int)e;
}

} /* extern "C" */
