/*
 * dma_kernels.cuh -- sequential chunk copy and strided tile transpose as
 * persistent kernels built on the CudaDMA objects of cudadma.h, using the
 * sm_100a extensions (multi-stage rings of objects, tensor-map tile loads,
 * bulk stores). The gather + scatter kernel needs no extension and lives in
 * common_kernels.cuh.
 *
 * Loop structure follows the reference's throughput benchmark
 * (src/perf/sequential/perf_sequential.cu:79-114): a CTA walks its share of
 * the units, DMA warps fill shared-memory buffers, compute warps drain them.
 */
#ifndef CUDADMA_B200_DMA_KERNELS_CUH
#define CUDADMA_B200_DMA_KERNELS_CUH

#include "cudadma.h"
#include "common_kernels.cuh"

namespace cudadma_b200 {
namespace kernels {

/* ------------------------------------------------------------------------ */
/* Sequential: CHUNK-byte chunks global -> shared -> global.                 */
/* 4 DMA warps + 8 compute warps; STAGES buffers per CTA.                    */
/* Chunk c of the array is handled by CTA c % gridDim.x.                     */
/* BULK_STORE == false (what the library launches): the DMA threads stage a  */
/* chunk through registers (BYTES_PER_THREAD = 128: eight 16-byte loads per  */
/* thread, issued before the thread waits for the buffer, stored into it     */
/* after), the compute threads write it back with 16-byte loads and stores.  */
/* BULK_STORE == true: cp.async.bulk in both directions (the DMA warps fill, */
/* one compute thread writes a chunk back with a bulk store).                */
/* Measured on 1 GiB, rotating (two GPUs): staged with 4 buffers x 3 CTAs per */
/* SM 6.54 - 6.62 TB/s (a device-to-device cudaMemcpy 6.42 - 6.52, the        */
/* reference classes 6.35 - 6.40); staged 3 x 3 6.44 - 6.49, 3 x 4 6.54,      */
/* 2 x 4 6.16, 6 x 2 6.03; 128 or 192 compute threads 6.50, 384 6.13; 256 DMA */
/* threads 6.41; bulk copies with 4 x 2 6.27 - 6.30. On 64 MiB arrays back to */
/* back: staged 4 x 3 5.44 (cudaMemcpy 5.44, bulk 5.24 - 5.35, the reference  */
/* classes 5.04 - 5.32).                                                      */
/* Not kept for the bulk form: handing a buffer back one chunk late, so that */
/* the storing thread waits for the read of the PREVIOUS chunk's store, 1 to */
/* 3 % slower with four to seven buffers; L2 evict-first hints on the loads, */
/* the stores or both, 0 to 2 % slower; 2 to 4 buffers x 2 to 4 CTAs per SM, */
/* and plain 16-byte stores for the write-back, all within 3 % below.        */
/* ------------------------------------------------------------------------ */
#ifndef SEQ_DMA_THREADS_N
#define SEQ_DMA_THREADS_N 128
#endif
#ifndef SEQ_COMPUTE_THREADS_N
#define SEQ_COMPUTE_THREADS_N 256
#endif
constexpr int SEQ_DMA_THREADS = SEQ_DMA_THREADS_N;
constexpr int SEQ_COMPUTE_THREADS = SEQ_COMPUTE_THREADS_N;

#ifndef SEQ_MIN_BLOCKS
#define SEQ_MIN_BLOCKS 3
#endif
#ifndef SEQ_LOAD_FORM
#define SEQ_LOAD_FORM 0 /* staged loads: 0 plain, 1 ld.global.cg (1 GiB: 6.30 TB/s against 6.54) */
#endif

template <int CHUNK, int STAGES, bool BULK_STORE>
__global__ void __launch_bounds__(SEQ_DMA_THREADS + SEQ_COMPUTE_THREADS, SEQ_MIN_BLOCKS)
seq_copy_kernel(char *__restrict__ dst, const char *__restrict__ src, const long long nchunks) {
  extern __shared__ __align__(128) unsigned char smem[];
  typedef CudaDMASequential<true, 16, BULK_STORE ? 64 : 128, CHUNK, SEQ_DMA_THREADS> Dma;
  Ring<Dma, STAGES> ring(SEQ_COMPUTE_THREADS, SEQ_COMPUTE_THREADS);
  const long long stride = gridDim.x;

  if (ring.stage[0].owns_this_thread()) {
    for (long long c0 = blockIdx.x;; c0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long c = c0 + s * stride;
        if (c >= nchunks) return;
#if SEQ_LOAD_FORM == 1
        ring.stage[s].template execute_dma<true, LOAD_CACHE_GLOBAL, STORE_WRITE_BACK>(src + c * CHUNK, smem + s * CHUNK);
#else
        ring.stage[s].execute_dma(src + c * CHUNK, smem + s * CHUNK);
#endif
      }
    }
  } else {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) ring.stage[s].start_async_dma();
    bool more = true;
    for (long long c0 = blockIdx.x; more; c0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long c = c0 + s * stride;
        if (c >= nchunks) { more = false; break; }
        ring.stage[s].wait_for_dma_finish();
        if (BULK_STORE) {
          if (threadIdx.x == 0) {
            ptx::bulk_s2g(dst + c * CHUNK, ptx::smem_u32(smem + s * CHUNK), CHUNK);
            ptx::bulk_commit();
            ptx::bulk_wait_read<0>();
          }
          /* the bulk-copy engine read the buffer and the bulk-copy engine refills it: no proxy fence */
          ring.stage[s].start_async_dma_after_reads();
        } else {
          const uint4 *b = reinterpret_cast<const uint4 *>(smem + s * CHUNK);
          uint4 *o = reinterpret_cast<uint4 *>(dst + c * CHUNK);
#pragma unroll
          for (int i = threadIdx.x; i < CHUNK / 16; i += SEQ_COMPUTE_THREADS) o[i] = b[i];
          ring.stage[s].start_async_dma();
        }
      }
    }
    if (BULK_STORE && threadIdx.x == 0) ptx::bulk_wait<0>();
  }
}

/* Same loop for a chunk size known only at run time (used for the last,
 * shorter chunk and for odd chunk sizes); single buffer. */
__global__ void __launch_bounds__(SEQ_DMA_THREADS + SEQ_COMPUTE_THREADS, 1)
seq_copy_runtime_kernel(char *__restrict__ dst, const char *__restrict__ src, const long long nchunks,
                        const int chunk_bytes) {
  extern __shared__ __align__(128) unsigned char smem[];
  CudaDMASequential<true, 4, 16> dma(0, SEQ_DMA_THREADS, SEQ_COMPUTE_THREADS, SEQ_COMPUTE_THREADS, chunk_bytes);
  if (dma.owns_this_thread()) {
    for (long long c = blockIdx.x; c < nchunks; c += gridDim.x) dma.execute_dma(src + c * chunk_bytes, smem);
  } else {
    dma.start_async_dma();
    for (long long c = blockIdx.x; c < nchunks; c += gridDim.x) {
      dma.wait_for_dma_finish();
      const unsigned int *b = reinterpret_cast<const unsigned int *>(smem);
      unsigned int *o = reinterpret_cast<unsigned int *>(dst + c * chunk_bytes);
      for (int i = threadIdx.x; i < chunk_bytes / 4; i += SEQ_COMPUTE_THREADS) o[i] = b[i];
      dma.start_async_dma();
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Strided: 128-row x 64-column fp32 tiles (row pitch = matrix width) pulled  */
/* into shared memory by CudaDMAStrided through a tensor map, written back    */
/* transposed: out[c * rows + r] = in[r * cols + c].                          */
/* The tile arrives as two 128 x 32 boxes in the 128-byte-swizzle layout:     */
/* element (r, c) of a box sits at r*128 + 16*((c/4) ^ (r%8)) + 4*(c%4), so   */
/* a quarter-warp reading one 16-byte column chunk of eight consecutive rows  */
/* touches eight different bank groups. Lane l then owns rows 4l..4l+3 of a   */
/* 4-column chunk, transposes the 4x4 block in registers and stores four      */
/* 16-byte pieces, one per output row: 512 contiguous bytes per warp store.   */
/* ------------------------------------------------------------------------ */
constexpr int TR_TILE_ROWS = 128, TR_TILE_COLS = 64, TR_BOX_COLS = 32;
#ifndef TR_SUPER
#define TR_SUPER 1 /* tiles are numbered down columns of TR_SUPER tiles, then across (see tile_of) */
#endif
/* Tile number -> (tile row, tile column). Tiles in flight at one time are consecutive numbers
 * (tile t belongs to CTA t % gridDim.x). With TR_SUPER == 1 they lie side by side in a tile row, so
 * their reads join into long runs of each matrix row, but every tile's writes are 512-byte pieces
 * of 64 different output rows. Numbering TR_SUPER tiles downwards first lets the writes of
 * vertically adjacent tiles join into TR_SUPER * 512-byte runs as well. */
__device__ __forceinline__ void tile_of(const long long t, const int tiles_x, const int tiles_y, int &ty, int &tx) {
  if (TR_SUPER <= 1) {
    ty = (int)(t / tiles_x);
    tx = (int)(t - (long long)ty * tiles_x);
  } else {
    const long long band = (long long)tiles_x * TR_SUPER;   /* tiles in a band of TR_SUPER tile rows */
    const int b = (int)(t / band);
    const long long in_band = t - (long long)b * band;
    const int h = (tiles_y - b * TR_SUPER < TR_SUPER) ? (tiles_y - b * TR_SUPER) : TR_SUPER; /* last band may be lower */
    tx = (int)(in_band / h);
    ty = b * TR_SUPER + (int)(in_band - (long long)tx * h);
  }
}
constexpr int TR_DMA_THREADS = 32, TR_COMPUTE_THREADS = 256;
constexpr int TR_TILE_BYTES = TR_TILE_ROWS * TR_TILE_COLS * 4;
constexpr int TR_BOX_BYTES = TR_TILE_ROWS * TR_BOX_COLS * 4;

template <int STAGES>
__global__ void __launch_bounds__(TR_DMA_THREADS + TR_COMPUTE_THREADS)
transpose_kernel(const __grid_constant__ CUtensorMap in_map, float *__restrict__ out, const int rows,
                 const int cols, const int src_pitch_bytes) {
  extern __shared__ unsigned char smem_raw[];
  /* the 128-byte swizzle pattern repeats every 1024 bytes: align the ring to it */
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  typedef CudaDMAStrided<true, 16, 64, TR_TILE_COLS * 4, TR_DMA_THREADS, TR_TILE_ROWS> Dma;
  Ring<Dma, STAGES> ring(TR_COMPUTE_THREADS, TR_COMPUTE_THREADS, src_pitch_bytes, TR_TILE_COLS * 4);
  const int tiles_x = cols / TR_TILE_COLS, tiles_y = rows / TR_TILE_ROWS;
  const long long ntiles = (long long)tiles_x * tiles_y;
  const long long stride = gridDim.x;

  if (ring.stage[0].owns_this_thread()) {
    for (long long t0 = blockIdx.x;; t0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long t = t0 + s * stride;
        if (t >= ntiles) return;
        int ty, tx;
        tile_of(t, tiles_x, tiles_y, ty, tx);
        ring.stage[s].execute_dma_tensor(&in_map, tx * TR_TILE_COLS, ty * TR_TILE_ROWS, smem + s * TR_TILE_BYTES,
                                         TR_TILE_COLS / TR_BOX_COLS, TR_BOX_COLS, TR_BOX_BYTES);
      }
    }
  } else {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    /* rotation that makes the four row loads of a lane conflict-free: in a quarter-warp the
     * rows 4l + ((i + l/2) % 4) take all eight values mod 8 */
    const int rot = (lane >> 1) & 3;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) ring.stage[s].start_async_dma();
    bool more = true;
    for (long long t0 = blockIdx.x; more; t0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long t = t0 + s * stride;
        if (t >= ntiles) { more = false; break; }
        int ty, tx;
        tile_of(t, tiles_x, tiles_y, ty, tx);
        ring.stage[s].wait_for_dma_finish();
        const unsigned char *tile = smem + s * TR_TILE_BYTES;
#pragma unroll
        for (int task = warp; task < 16; task += TR_COMPUTE_THREADS / 32) {
          const int box = task >> 3, k = task & 7;
          const unsigned char *b = tile + box * TR_BOX_BYTES;
          float4 v[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = 4 * lane + ((i + rot) & 3);
            v[i] = *reinterpret_cast<const float4 *>(b + r * 128 + 16 * (k ^ (r & 7)));
          }
          /* v[i] holds row 4*lane + (i + rot) % 4; put row 4*lane + j into w[j] */
          float4 w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = (j - rot) & 3;
            w[j] = (i == 0) ? v[0] : (i == 1) ? v[1] : (i == 2) ? v[2] : v[3];
          }
          const long long c0 = (long long)tx * TR_TILE_COLS + box * TR_BOX_COLS + 4 * k;
          float *o = out + c0 * rows + (long long)ty * TR_TILE_ROWS + 4 * lane;
          __stcs(reinterpret_cast<float4 *>(o), make_float4(w[0].x, w[1].x, w[2].x, w[3].x));
          __stcs(reinterpret_cast<float4 *>(o + rows), make_float4(w[0].y, w[1].y, w[2].y, w[3].y));
          __stcs(reinterpret_cast<float4 *>(o + 2ll * rows), make_float4(w[0].z, w[1].z, w[2].z, w[3].z));
          __stcs(reinterpret_cast<float4 *>(o + 3ll * rows), make_float4(w[0].w, w[1].w, w[2].w, w[3].w));
        }
        ring.stage[s].start_async_dma();
      }
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Indirect with TMA row gathers and / or row scatters: with G4 the gather      */
/* object fetches four table records per cp.async.bulk.tensor ... tile::gather4 */
/* instruction through a tensor map of the table, with S4 the scatter object     */
/* writes four records per ... tile::scatter4 instruction through a tensor map   */
/* of the output; the side without its flag works as in gather_scatter_kernel,   */
/* whose bridge is used unchanged.                                               */
/* ------------------------------------------------------------------------ */
template <int RECORD_BYTES, int RECORDS, int STAGES, bool G4, bool S4>
__global__ void __launch_bounds__(GS_THREADS)
gather4_scatter_kernel(const __grid_constant__ CUtensorMap table_map, const __grid_constant__ CUtensorMap out_map,
                       char *__restrict__ out, const char *__restrict__ table, const int *__restrict__ gather_idx,
                       const int *__restrict__ scatter_idx, const long long nbuffers) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int BUF = RECORD_BYTES * RECORDS;
  typedef CudaDMAIndirect<true, true, 16, 64, RECORD_BYTES, GS_GATHER_THREADS, RECORDS> Gather;
  typedef CudaDMAIndirect<false, true, 16, 64, RECORD_BYTES, GS_SCATTER_THREADS, RECORDS> Scatter;
  Ring<Gather, STAGES, 0> g(GS_BRIDGE_THREADS, GS_BRIDGE_THREADS);
  Ring<Scatter, STAGES, STAGES> sc(GS_BRIDGE_THREADS, GS_BRIDGE_THREADS + GS_GATHER_THREADS);
  const long long stride = gridDim.x;
  if (g.stage[0].owns_this_thread()) {
    for (long long b0 = blockIdx.x;; b0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long b = b0 + s * stride;
        if (b >= nbuffers) return;
        if (G4) g.stage[s].execute_dma_gather4(&table_map, gather_idx + b * RECORDS, smem + s * BUF);
        else g.stage[s].execute_dma(gather_idx + b * RECORDS, table, smem + s * BUF);
      }
    }
  } else if (sc.stage[0].owns_this_thread()) {
    for (long long b0 = blockIdx.x;; b0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long b = b0 + s * stride;
        if (b >= nbuffers) return;
        if (S4) sc.stage[s].execute_dma_scatter4(&out_map, scatter_idx + b * RECORDS, smem + s * BUF);
        else sc.stage[s].execute_dma(scatter_idx + b * RECORDS, smem + s * BUF, out);
      }
    }
  } else {
    bridge_gather_to_scatter<STAGES>(g, sc, nbuffers, stride);
  }
}

}  // namespace kernels
}  // namespace cudadma_b200

#endif
