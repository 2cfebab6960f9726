/*
 * ref_bench.cu -- the benchmark workloads driven by the REFERENCE CudaDMA
 * classes (include/cudaDMAv2.h of the CudaDMA project, found through
 * -I$(REFERENCE_INCLUDE); nothing of it is copied here) compiled for sm_100a.
 * The kernels are the repository's portable kernels: the same source that the
 * product library builds against its own header. TEST INFRASTRUCTURE: this is
 * the "reference CudaDMA build" baseline and a device-side parity oracle.
 *
 * Entry points return 0 or a cudaError_t; stream is a cudaStream_t.
 */
#include <cuda_runtime.h>

#include "cudaDMAv2.h"

#include "common_kernels.cuh"
#include "portable_kernels.cuh"

namespace {
int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}
}  // namespace

/* BYTES_PER_THREAD of the objects, the reference's register staging budget: 64, 128 or 192 */
#define BPT_DISPATCH(bpt, CALL)                    \
  switch (bpt) {                                   \
    case 64: return CALL(64);                      \
    case 128: return CALL(128);                    \
    case 192: return CALL(192);                    \
    default: return (int)cudaErrorInvalidValue;    \
  }

extern "C" {

int cudadma_ref_seq_copy(void *dst, const void *src, size_t bytes, int bpt, void *stream) {
  if (bytes % portable::P_CHUNK) return (int)cudaErrorInvalidValue;
#define CALL(B) portable::launch_seq_copy<B>(static_cast<char *>(dst), static_cast<const char *>(src), \
                                             (long long)(bytes / portable::P_CHUNK), sm_count(), (cudaStream_t)stream)
  BPT_DISPATCH(bpt, CALL)
#undef CALL
}

int cudadma_ref_strided_transpose(float *dst, const float *src, int rows, int cols, int bpt, void *stream) {
  if (rows % portable::PT_ROWS || cols % portable::PT_COLS) return (int)cudaErrorInvalidValue;
#define CALL(B) portable::launch_transpose<B>(dst, src, rows, cols, sm_count(), (cudaStream_t)stream)
  BPT_DISPATCH(bpt, CALL)
#undef CALL
}

int cudadma_ref_gather_scatter(void *out, const void *table, const int *gather_idx, const int *scatter_idx, size_t n,
                               int bpt, void *stream) {
  if (n % 128) return (int)cudaErrorInvalidValue;
  /* 32-byte records: the reference wants BYTES_PER_THREAD / ALIGNMENT loads per thread, all three budgets are legal */
#define CALL(B) portable::launch_gather_scatter<32, B>(static_cast<char *>(out), static_cast<const char *>(table), gather_idx, \
                                                       scatter_idx, (long long)(n / 128), sm_count(), (cudaStream_t)stream)
  BPT_DISPATCH(bpt, CALL)
#undef CALL
}

/* arrays padded by four zero cells on every side: (nx + 8) x (ny + 8) x (nz + 8) floats */
int cudadma_ref_stencil25_step_padded(float *out, const float *in, int nx, int ny, int nz, int z_begin, int z_end,
                                      const float coeff[5], int z_chunk, int bpt, void *stream) {
#define CALL(B) portable::launch_stencil_padded<B>(out, in, nx, ny, nz, z_begin, z_end, coeff, z_chunk, sm_count(), \
                                                   (cudaStream_t)stream)
  BPT_DISPATCH(bpt, CALL)
#undef CALL
}

} /* extern "C" */
