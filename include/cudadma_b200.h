/*
 * cudadma_b200.h -- C ABI of libcudadma_b200.so.
 *
 * The reference (lightsighter/CudaDMA) is a header-only device library with no
 * host interface: each of its tests, benchmarks and examples is a main() that
 * allocates, launches one kernel and checks or times it. These entry points
 * are that host side as a library: every function states the reference
 * program whose launch it replaces. A caller binds them with any FFI (plain
 * pointers and sizes, no C++ types); device pointers are CUDA device
 * addresses of the current device, `stream` is a cudaStream_t (0 = default).
 *
 * Return value: 0 on success, negative for a rejected call, positive when
 * the kernel ran but a bounded wait inside it gave up.
 * Nothing here falls back to the CPU: without a CUDA device the compute calls
 * return CUDADMA_ERR_CUDA.
 */
#ifndef CUDADMA_B200_H
#define CUDADMA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  CUDADMA_OK = 0,
  CUDADMA_ERR_ARG = -1,         /* null pointer, size not a multiple of what the kernel needs */
  CUDADMA_ERR_CUDA = -2,        /* a CUDA call failed; see cudadma_last_cuda_error() */
  CUDADMA_ERR_UNSUPPORTED = -3, /* impl not built into this library */
  CUDADMA_ERR_NOMEM = -4,       /* device or pinned memory could not be had */
  CUDADMA_ERR_TOO_LARGE = -5,   /* cudadma_stencil25_step_noalloc: the padded grid exceeds its built-in scratch */
  CUDADMA_ERR_TIMEOUT = 1       /* a wait inside the kernel gave up; see cudadma_device_status() */
};

/* Which kernel family runs the workload. */
enum {
  CUDADMA_IMPL_NATIVE = 0,   /* sm_100a extensions: object rings, tensor maps, bulk stores */
  CUDADMA_IMPL_PORTABLE = 1  /* same objects through the reference's API only (double buffered) */
};

int cudadma_version(void);
const char *cudadma_status_string(int status);
/* cudaError_t of the last failed CUDA call of the calling thread, as an int */
int cudadma_last_cuda_error(void);
/* Reads and clears the device status word written by a wait that gave up
 * (bit 31 set | dmaID << 8 | 1 = empty wait, 2 = full wait). Synchronises `stream`. */
int cudadma_device_status(void *stream, unsigned int *out);
/* Number of kernels this library has launched in this process (all calls). */
unsigned long long cudadma_launch_count(void);

/* Sequential chunk copy: dst[0..bytes) = src[0..bytes), every chunk_bytes chunk
 * staged global -> shared -> global by CudaDMASequential (4 DMA + 8 compute
 * warps). Replaces the launch in src/perf/sequential/perf_sequential.cu:225-369
 * (whose kernels only load; the write-back is this benchmark's addition) and
 * the check of src/tests/test_sequential/cudaDMA_test_sequential_v2.cu:500-512.
 * bytes % 4 == 0; chunk_bytes % 16 == 0, 16 <= chunk_bytes <= 16384; pointers 16-byte aligned. */
int cudadma_seq_copy(void *dst, const void *src, size_t bytes, int chunk_bytes, int impl, void *stream);

/* Strided tile transpose: rows x cols fp32 row-major matrix, each 128-row x
 * 64-column tile pulled by CudaDMAStrided (row pitch = cols) and written back
 * transposed: dst[c * rows + r] = src[r * cols + c]. The transfer is the one
 * checked by src/tests/test_strided/cudaDMA_test_strided_v2.cu:659-676.
 * rows % 128 == 0, cols % 64 == 0; pointers 16-byte aligned. */
int cudadma_strided_transpose(float *dst, const float *src, int rows, int cols, int impl, void *stream);

/* Indirect gather + scatter: out[scatter_idx[i]] = table[gather_idx[i]] for
 * records of record_bytes, 128 records per shared buffer: CudaDMAIndirect
 * gather (src/tests/test_indirect/cudaDMA_test_indirect_v2.cu:661-692) then
 * CudaDMAIndirect scatter (include/cudaDMAv2.h:14021-14025).
 * n % 128 == 0; record_bytes 16, 32, 64 or 128 (32 is the benchmark's size); scatter_idx must not repeat. */
int cudadma_gather_scatter(void *out, const void *table, const int32_t *gather_idx, const int32_t *scatter_idx,
                           size_t n, int record_bytes, int impl, void *stream);

/* The same workload with the gather done by TMA row gathers (cp.async.bulk.tensor ... tile::gather4
 * through CudaDMAIndirect::execute_dma_gather4): four table records per instruction. The tensor map
 * needs the table's extent, hence table_records. Same result; on B200 it measured slower than the
 * 16-byte cp.async gather of cudadma_gather_scatter (1.63 against 1.76 TB/s on the benchmark
 * configuration), so the latter stays the default path. gather_idx entries must be < table_records. */
int cudadma_gather_scatter_tma(void *out, const void *table, size_t table_records, const int32_t *gather_idx,
                               const int32_t *scatter_idx, size_t n, int record_bytes, void *stream);

/* One step of the radius-4 25-point stencil on an nx x ny x nz fp32 grid (x
 * fastest), output planes [z_begin, z_end) only; reads outside the grid give
 * zero. 32 x 32 tiles (native; 32 x 16 portable) with their halo come in through CudaDMAHalo, z-marching.
 * The reference has no such kernel; its stencil example
 * (src/examples/stencil/cudaDMA_stencil2D.cu:60-264) is the launch replaced.
 * nx % 4 == 0; pointers 16-byte aligned; in and out must not overlap.
 * z_chunk = planes per CTA (0 = library's choice). */
int cudadma_stencil25_step(float *out, const float *in, int nx, int ny, int nz, int z_begin, int z_end,
                           const float coeff[5], int z_chunk, int impl, void *stream);
/* `steps` ping-pong steps a -> b -> a ...; the result is in a when steps is even, else in b. */
int cudadma_stencil25_run(float *a, float *b, int nx, int ny, int nz, const float coeff[5], int steps, int impl,
                          void *stream);

/* The same step on arrays padded by four zero cells on every side, the layout the reference's
 * stencil example gives its arrays (src/examples/stencil/cudaDMA_stencil2D.cu:86-97): grid cell
 * (x, y, z) is element ((z + 4) * (ny + 8) + (y + 4)) * (nx + 8) + (x + 4). Only the portable
 * kernels read this layout (CudaDMAStrided pulls each 40 x 24 window; there is no tensor map to
 * fill the border); impl must be CUDADMA_IMPL_PORTABLE. nx % 32 == 0, ny % 16 == 0.
 * With impl = portable, cudadma_stencil25_step/run above copy the field into padded arrays of
 * the library workspace, run this kernel there and copy the result back. */
int cudadma_stencil25_step_padded(float *out, const float *in, int nx, int ny, int nz, int z_begin, int z_end,
                                  const float coeff[5], int z_chunk, int impl, void *stream);

/* z-sharded stencil, one process per GPU, halo planes pushed straight into the z-neighbours'
 * memory. (The reference has no multi-GPU code; every program of it uses device 0,
 * src/examples/stencil/cudaDMA_stencil2D.cu:62.) A slab is this rank's nzl planes of an
 * nx x ny x nz grid plus four ghost planes on either side, in two ping-pong arrays that the
 * library allocates so that they can be shared between processes (CUDA IPC).
 *   create  -> export (cudadma_slab_handle_bytes() bytes to hand to both neighbours, by any
 *   means) -> connect (with the neighbours' bytes) -> fill buffer 0 (current field; ghost planes
 *   included) -> step, step, ... -> read buffer 0 -> destroy.
 * One step: wait until both neighbours have finished the previous step (a flag word they write
 * into this GPU's memory; the wait is bounded), compute all owned planes in one launch, the
 * first and last four of them stored twice, here and in the neighbour's ghost planes over
 * NVLink, then publish this rank's step count to both neighbours. No collective library is
 * involved. has_lower / has_upper say whether a neighbour exists on that side; nzl >= 8 then.
 * cudadma_slab_buffer: which = 0 the current field, 1 the other array; (nzl + 8) * ny * nx floats. */
int cudadma_slab_create(void **slab, int nx, int ny, int nzl, int has_lower, int has_upper);
size_t cudadma_slab_handle_bytes(void);
int cudadma_slab_export(void *slab, void *handles);
int cudadma_slab_connect(void *slab, const void *lower_handles, const void *upper_handles);
int cudadma_slab_buffer(void *slab, int which, float **ptr);
int cudadma_slab_step(void *slab, const float coeff[5], void *stream);
int cudadma_slab_destroy(void *slab);

/* One stencil step for callers that must not allocate device memory. (No counterpart in the
 * reference, which has no host library at all.)
 *
 * cudadma_stencil25_step with impl = portable keeps its two padded copies of the field in a
 * workspace that the library obtains with cudaMalloc the first time, and again whenever a
 * larger grid arrives. That is wrong for a solver whose framework has already taken the whole
 * device into its own memory pool (the driver allocation then fails, or succeeds and starves
 * the pool), and for a time-step loop that runs next to other streams, because cudaMalloc and
 * cudaFree stall the whole device while they work. This entry point runs the same kernel with
 * the padded copies in an array that is part of the library image instead, so it makes no
 * cudaMalloc, no cudaFree and no other allocating call, at any time.
 *
 * What that costs and what to watch:
 *   - the array is 16 MiB and every GPU that loads the library carries it until the process
 *     exits, whether or not this function is ever called;
 *   - the padded grid (nx + 8) * (ny + 8) * (nz + 8) may have at most 2^21 cells (for
 *     example 120 x 112 x 120); a larger one returns CUDADMA_ERR_TOO_LARGE and touches nothing;
 *   - all calls on a GPU share the array. Each call first re-makes the zero border it needs,
 *     so the previous call's leftovers do no harm, but two calls whose work overlaps on the GPU
 *     (different streams, no ordering between them) race on it: keep them on one stream or
 *     order them with events;
 *   - the first call on each GPU looks up the array's device address (one runtime query, with
 *     that GPU current); make that first call before any stream capture begins.
 * Same arguments and result as cudadma_stencil25_step(out, in, nx, ny, nz, 0, nz, coeff, 0,
 * CUDADMA_IMPL_PORTABLE, stream): nx % 32 == 0, ny % 16 == 0, pointers 16-byte aligned, in != out. */
int cudadma_stencil25_step_noalloc(float *out, const float *in, int nx, int ny, int nz, const float coeff[5],
                                   void *stream);

/* Host-buffer forms: the same workloads for callers that hold their data in
 * host memory. Inputs are copied to the device, the kernel runs, the result
 * is copied back; the call returns when the result is in h_* memory. Device
 * staging memory is a grow-only workspace kept by the library on the device
 * that is current at the call (one per process: a call with another device
 * current moves it there; cudadma_release_workspace() frees it). The calls
 * serialise on a lock. Pinned host memory copies fastest. */
int cudadma_seq_copy_host(void *h_dst, const void *h_src, size_t bytes, int chunk_bytes, int impl);
int cudadma_strided_transpose_host(float *h_dst, const float *h_src, int rows, int cols, int impl);
int cudadma_gather_scatter_host(void *h_out, size_t out_records, const void *h_table, size_t table_records,
                                const int32_t *h_gather_idx, const int32_t *h_scatter_idx, size_t n,
                                int record_bytes, int impl);
int cudadma_stencil25_run_host(float *h_out, const float *h_in, int nx, int ny, int nz, const float coeff[5],
                               int steps, int impl);
/* cudadma_stencil25_run_host with the piece size of its overlapped form given. With impl = native
 * the field is uploaded in pieces of chunk_planes planes; while later pieces are still on the
 * bus, the steps run on the planes that have arrived (step t trails the upload by 4 t planes)
 * and finished planes go back to the host, so on a grid much deeper than 4 * steps planes the
 * call takes about as long as the upload alone. The result is bit-identical to the plain
 * upload / run / download sequence. chunk_planes = 0: the library's choice (128 MiB pieces; the
 * plain sequence where the grid is too shallow to overlap anything), which is what
 * cudadma_stencil25_run_host does. impl = portable always runs the plain sequence. */
int cudadma_stencil25_run_host_pipelined(float *h_out, const float *h_in, int nx, int ny, int nz,
                                         const float coeff[5], int steps, int impl, int chunk_planes);
int cudadma_release_workspace(void);

#ifdef __cplusplus
}
#endif
#endif
