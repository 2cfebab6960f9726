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

/* Host side of the tensor-map extensions of the classes (CudaDMAStrided::execute_dma_tensor,
 * CudaDMAHalo::execute_dma_tile, CudaDMAIndirect::execute_dma_gather4 / execute_dma_scatter4).
 * The reference's constructors take their strides on the device (include/cudaDMAv2.h:8631-8651);
 * a tensor map has to be encoded on the host and handed to the kernel as a __grid_constant__
 * parameter, and these two calls do the encoding. out_map: 128 bytes, 64-byte aligned (a
 * CUtensorMap). Elements are 4-byte words; reads outside the tensor give zero.
 * 2-D: `rows` rows of `cols` words, row_pitch_bytes apart; the box is box_cols x box_rows
 * (each at most 256, box_cols * 4 a multiple of 16); swizzle_128b != 0 asks for the 128-byte
 * shared-memory swizzle (box_cols <= 32 then). 3-D: nx x ny x nz words, x fastest, rows
 * row_pitch_bytes and planes plane_pitch_bytes apart; box box_x x box_y x box_z.
 * base 16-byte aligned, pitches multiples of 16. */
int cudadma_make_tensor_map_2d(void *out_map, const void *base, unsigned long long cols, unsigned long long rows,
                               unsigned long long row_pitch_bytes, unsigned int box_cols, unsigned int box_rows,
                               int swizzle_128b);
int cudadma_make_tensor_map_3d(void *out_map, const void *base, unsigned long long nx, unsigned long long ny,
                               unsigned long long nz, unsigned long long row_pitch_bytes,
                               unsigned long long plane_pitch_bytes, unsigned int box_x, unsigned int box_y,
                               unsigned int box_z);

/* Seeded synthetic inputs on the device, for benchmarks and tests. (The reference fills its inputs
 * on the host: h_idata[i] = float(i), src/tests/test_sequential/cudaDMA_test_sequential_v2.cu:417-418,
 * or rand(), src/tests/test_halo/cudaDMA_test_halo.cu:245-246.) Element i of a field is a function of
 * seed + first_index + i alone (splitmix64; uniform = lo + (hi - lo) * top 24 bits * 2^-24;
 * index = value mod modulo), so a field can be produced in pieces, on any GPU, and every piece
 * equals the same range of the whole. */
int cudadma_fill_uniform(float *dst, size_t n, unsigned long long seed, unsigned long long first_index, float lo,
                         float hi, void *stream);
int cudadma_fill_index(int32_t *dst, size_t n, unsigned long long seed, unsigned long long first_index,
                       unsigned int modulo, void *stream);
/* Measurement aid: a one-thread kernel that spins for spin_ns nanoseconds and writes the SM cycles
 * and the nanoseconds that passed to out[0], out[1] (device memory). Launched on a second stream
 * beside a workload it reports the SM clock the workload actually ran at. */
int cudadma_clock_probe(unsigned long long *out, long long spin_ns, void *stream);

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

/* The same workload with TMA row instructions, four records each: mode bit 0 = the gather through
 * cp.async.bulk.tensor ... tile::gather4 (CudaDMAIndirect::execute_dma_gather4), bit 1 = the scatter
 * through ... tile::scatter4 (execute_dma_scatter4); mode 1, 2 or 3. The tensor maps need the
 * extents of table and output, hence table_records and out_records. Same result as
 * cudadma_gather_scatter, which stays the default path: on B200 neither TMA form was faster than
 * its 16-byte cp.async gather and 16-byte stores (benchmark configuration, same CTAs per SM: 1.81
 * TB/s with row gathers, 1.73 with row scatters, 1.73 without). gather_idx entries must be < table_records, scatter_idx
 * entries < out_records; record_bytes must be 32. */
int cudadma_gather_scatter_tma(void *out, size_t out_records, const void *table, size_t table_records,
                               const int32_t *gather_idx, const int32_t *scatter_idx, size_t n, int record_bytes,
                               int mode, void *stream);

/* One step of the radius-4 25-point stencil on an nx x ny x nz fp32 grid (x
 * fastest), output planes [z_begin, z_end) only; reads outside the grid give
 * zero. 64 x 16 tiles (native; 32 x 16 portable) with their halo come in through CudaDMAHalo, z-marching.
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

/* z-sharded stencil, halo planes pushed straight into the z-neighbours' memory. (The reference has
 * no multi-GPU code; every program of it uses device 0, src/examples/stencil/cudaDMA_stencil2D.cu:62.)
 * A slab is one rank's nzl planes of an nx x ny x nz grid plus four ghost planes on either side,
 * in two ping-pong arrays that the library allocates on the current device so that they can be
 * shared between processes (CUDA IPC).
 *   create  -> export (cudadma_slab_handle_bytes() bytes to hand to both neighbours, by any
 *   means) -> connect (with the neighbours' bytes) -> fill buffer 0 (current field; ghost planes
 *   included) -> step, step, ... -> status -> read buffer 0 -> destroy.
 * Slabs of one process (one per GPU, or several on one GPU) are joined with
 * cudadma_slab_connect_local instead of export / connect; it enables peer access where the
 * slabs sit on different GPUs.
 * One step: the kernel's CTAs at a boundary shared with a neighbour first wait until that
 * neighbour has finished the previous step (a flag word it writes into this GPU's memory; the
 * wait is bounded, about two seconds unless cudadma_slab_set_wait_limit says otherwise), all owned
 * planes are computed, the first and last four of them stored twice, here and in the neighbour's
 * ghost planes over NVLink, and this rank's step count is published to both neighbours, either
 * by a one-thread launch behind the kernel or from inside it (cudadma_slab_set_signal_mode). No
 * collective library is involved. has_lower / has_upper say whether a neighbour exists on that
 * side; nzl >= 8 then.
 * When a wait runs out (a neighbour is gone or more than the limit behind), the step records
 * it, stores nothing more into the neighbours and does not publish its step count, so the
 * neighbours' own waits run out as well instead of taking over wrong planes; this rank's own
 * field is undefined from then on. cudadma_slab_status(slab, stream) synchronises the stream and
 * returns CUDADMA_ERR_TIMEOUT if that has happened, and from then on so does every
 * cudadma_slab_step, without launching.
 * cudadma_slab_buffer: which = 0 the current field, 1 the other array; (nzl + 8) * ny * nx floats. */
int cudadma_slab_create(void **slab, int nx, int ny, int nzl, int has_lower, int has_upper);
size_t cudadma_slab_handle_bytes(void);
int cudadma_slab_export(void *slab, void *handles);
int cudadma_slab_connect(void *slab, const void *lower_handles, const void *upper_handles);
int cudadma_slab_connect_local(void *slab, void *lower_slab, void *upper_slab);
int cudadma_slab_set_wait_limit(void *slab, long long sm_cycles);
/* Who publishes a rank's step count to its neighbours.
 * CUDADMA_SLAB_SIGNAL_TRAILING (default): a one-thread launch behind the step's kernel, so a step is
 * two launches and the count goes out when the whole step is done.
 * CUDADMA_SLAB_SIGNAL_FUSED: the step is ONE launch; the slab is cut so that the CTAs at its two
 * boundaries run first, each of them makes its stores into the neighbour visible system-wide and
 * takes a ticket, and the last one publishes while the interior is still being computed. The
 * neighbours get half a step of slack, but every boundary CTA pays for a system-scope fence behind
 * its remote stores: on B200 / NVLink 5 the trailing form measured faster (weak-scaling steps of
 * 256 planes per GPU). Set the same mode on every slab of a job before its first step. */
enum { CUDADMA_SLAB_SIGNAL_TRAILING = 0, CUDADMA_SLAB_SIGNAL_FUSED = 1 };
int cudadma_slab_set_signal_mode(void *slab, int mode);
/* Trailing mode: the order in which the kernel's runs of planes are dispatched. highest_first = 1
 * (default): from the top of the slab down. The CTAs of the top run need the upper neighbour only
 * before their last four planes, and those of the bottom run, which need the lower neighbour before
 * their first load, start in the second half of the launch: no CTA waits at the start of a kernel,
 * and neighbouring GPUs may drift against each other by a good part of a step. 0: from the bottom up. */
int cudadma_slab_set_run_order(void *slab, int highest_first);
/* Tuning: depth of the two boundary runs of a step, which are dispatched first so that the step
 * count can go out early (default 32; 0 = equal runs, the count then goes out at the end of the
 * step; at least 8 otherwise). Slabs shallower than two such runs plus one plane use equal runs. */
int cudadma_slab_set_edge_planes(void *slab, int planes);
int cudadma_slab_buffer(void *slab, int which, float **ptr);
int cudadma_slab_step(void *slab, const float coeff[5], void *stream);
int cudadma_slab_status(void *slab, void *stream);
int cudadma_slab_destroy(void *slab);

/* The whole sharded stencil driven from ONE process: n_gpus slabs (planes split as evenly as
 * possible, lower ranks take the remainder), one per entry of `devices` (null: devices 0 ..
 * n_gpus - 1), one stream per GPU, neighbours joined by peer access, the step as above. A C or
 * C++ solver links against these five calls and needs no process launcher. Entries of `devices`
 * may repeat: slabs that share a GPU share its stream, so their steps run one after the other,
 * each after the steps it waits for (a way to run the N-rank path on fewer GPUs).
 * load: the whole nx x ny x nz field from host memory into the slabs, ghost planes included.
 * run: `steps` steps on every slab; returns after all GPUs have finished, with
 * CUDADMA_ERR_TIMEOUT if any wait gave up. store: the whole field back to host memory.
 * slab: the slab handle and plane range [z_lo, z_hi) of one rank, for callers that fill or read
 * device memory themselves (cudadma_slab_buffer). nz / n_gpus >= 8 for n_gpus > 1. */
int cudadma_stencil25_multi_create(void **handle, int n_gpus, const int *devices, int nx, int ny, int nz);
int cudadma_stencil25_multi_load(void *handle, const float *h_field);
int cudadma_stencil25_multi_run(void *handle, const float coeff[5], int steps);
int cudadma_stencil25_multi_store(void *handle, float *h_field);
int cudadma_stencil25_multi_slab(void *handle, int rank, void **slab, int *z_lo, int *z_hi);
int cudadma_stencil25_multi_destroy(void *handle);

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
 * cudaMalloc, no cudaFree and no other allocating call (see the last point below for the one
 * allocation the CUDA runtime itself makes when it loads the library's device code).
 *
 * What that costs and what to watch:
 *   - the array is 16 MiB and every GPU that loads the library carries it until the process
 *     exits, whether or not this function is ever called;
 *   - the padded grid (nx + 8) * (ny + 8) * (nz + 8) may have at most 2^21 cells (for
 *     example 128 x 112 x 120: 136 * 120 * 128 = 2 088 960 cells); a larger one returns
 *     CUDADMA_ERR_TOO_LARGE and touches nothing;
 *   - all calls on a GPU share the array. Each call first re-makes the zero border it needs,
 *     so the previous call's leftovers do no harm, but two calls whose work overlaps on the GPU
 *     (different streams, no ordering between them) race on it: keep them on one stream or
 *     order them with events;
 *   - the first call on each GPU looks up the array's device address (one runtime query, with
 *     that GPU current); make that first call before any stream capture begins;
 *   - the 16 MiB are reserved when the CUDA runtime loads this library's device code on a GPU,
 *     which it does lazily, at the library's first kernel launch or address query there. A
 *     framework that takes all remaining device memory into its pool must therefore make one
 *     call into this library on every GPU BEFORE it sizes that pool (any launching call will
 *     do, this one included), or the load itself fails for lack of memory.
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
