/*
 * common_kernels.cuh -- kernels written against the CudaDMA object API only
 * (no sm_100a extension), so the same source builds against cudadma.h and
 * against the reference headers. The including file provides the CudaDMA
 * header.
 */
#ifndef CUDADMA_B200_COMMON_KERNELS_CUH
#define CUDADMA_B200_COMMON_KERNELS_CUH

#include <utility>

namespace cudadma_b200 {
namespace kernels {

/* STAGES objects of type T with dmaIDs FIRST_ID .. FIRST_ID + STAGES - 1; the
 * remaining constructor arguments are the same for every stage. */
template <typename T, int FIRST_ID, typename SEQ>
struct StageRing;
template <typename T, int FIRST_ID, int... I>
struct StageRing<T, FIRST_ID, std::integer_sequence<int, I...>> {
  T stage[sizeof...(I)];
  template <typename... A>
  __device__ __forceinline__ StageRing(A... rest) : stage{T(FIRST_ID + I, rest...)...} {}
};
template <typename T, int STAGES, int FIRST_ID = 0>
using Ring = StageRing<T, FIRST_ID, std::make_integer_sequence<int, STAGES>>;

/* The bridging warp of the gather + scatter kernels: buffer full (gather done) -> start its
 * scatter; LAG buffers later, once that scatter has read the buffer, hand it back to the gather
 * object. Every arrival made here is matched by a wait on the other side (named barriers must
 * not be left with arrivals nobody waits for), hence the guards and the drain at the end. */
template <int STAGES, typename GRING, typename SRING>
__device__ __forceinline__ void bridge_gather_to_scatter(GRING &g, SRING &sc, const long long nbuffers,
                                                         const long long stride) {
  static_assert(STAGES >= 2, "the bridge needs at least two buffers");
  constexpr int LAG = STAGES / 2;
#pragma unroll
  for (int s = 0; s < STAGES; ++s)
    if (blockIdx.x + s * stride < nbuffers) g.stage[s].start_async_dma();
  bool more = true;
  long long done = 0;   /* buffers of this CTA handed to a scatter object so far */
  unsigned pending = 0; /* stages whose scatter has been started and not yet waited for */
  for (long long b0 = blockIdx.x; more; b0 += stride * STAGES) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      const long long b = b0 + s * stride;
      if (b >= nbuffers) { more = false; break; }
      g.stage[s].wait_for_dma_finish();
      sc.stage[s].start_async_dma();
      pending |= 1u << s;
      ++done;
      if (done > LAG) {
        sc.stage[(s + STAGES - LAG) % STAGES].wait_for_dma_finish();
        pending &= ~(1u << ((s + STAGES - LAG) % STAGES));
        if (b + (STAGES - LAG) * stride < nbuffers) g.stage[(s + STAGES - LAG) % STAGES].start_async_dma();
      }
    }
  }
#pragma unroll
  for (int s = 0; s < STAGES; ++s)
    if ((pending >> s) & 1u) sc.stage[s].wait_for_dma_finish();
}

/* ------------------------------------------------------------------------ */
/* Indirect: buffers of RECORDS records of RECORD_BYTES bytes. A gather       */
/* object fills a shared buffer from table rows gather_idx[..], a scatter     */
/* object empties it into output slots scatter_idx[..]; one bridging warp     */
/* hands each buffer from the gather object to the scatter object and back.   */
/* Buffer b of the job is handled by CTA b % gridDim.x.                       */
/* ------------------------------------------------------------------------ */
constexpr int GS_GATHER_THREADS = 128, GS_SCATTER_THREADS = 128, GS_BRIDGE_THREADS = 32;
constexpr int GS_THREADS = GS_BRIDGE_THREADS + GS_GATHER_THREADS + GS_SCATTER_THREADS;

#ifndef GS_MIN_BLOCKS
#define GS_MIN_BLOCKS 7 /* seven CTAs of 288 threads fill an SM's 2048 thread slots: at most 32 registers. The kernel
                           is bound by how many records are in flight, and 40 registers (five CTAs) cost it 9 % */
#endif
/* BPT: the BYTES_PER_THREAD template argument of the objects (the reference's register staging budget) */
template <int RECORD_BYTES, int RECORDS, int STAGES, int BPT = 64>
__global__ void __launch_bounds__(GS_THREADS, GS_MIN_BLOCKS)
gather_scatter_kernel(char *__restrict__ out, const char *__restrict__ table, const int *__restrict__ gather_idx,
                      const int *__restrict__ scatter_idx, const long long nbuffers) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int BUF = RECORD_BYTES * RECORDS;
  typedef CudaDMAIndirect<true, true, 16, BPT, RECORD_BYTES, GS_GATHER_THREADS, RECORDS> Gather;
  typedef CudaDMAIndirect<false, true, 16, BPT, RECORD_BYTES, GS_SCATTER_THREADS, RECORDS> Scatter;
  Ring<Gather, STAGES, 0> g(GS_BRIDGE_THREADS, GS_BRIDGE_THREADS);
  Ring<Scatter, STAGES, STAGES> sc(GS_BRIDGE_THREADS, GS_BRIDGE_THREADS + GS_GATHER_THREADS);
  const long long stride = gridDim.x;

  if (g.stage[0].owns_this_thread()) {
    for (long long b0 = blockIdx.x;; b0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long b = b0 + s * stride;
        if (b >= nbuffers) return;
        g.stage[s].execute_dma(gather_idx + b * RECORDS, table, smem + s * BUF);
      }
    }
  } else if (sc.stage[0].owns_this_thread()) {
    for (long long b0 = blockIdx.x;; b0 += stride * STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const long long b = b0 + s * stride;
        if (b >= nbuffers) return;
        sc.stage[s].execute_dma(scatter_idx + b * RECORDS, smem + s * BUF, out);
      }
    }
  } else {
    bridge_gather_to_scatter<STAGES>(g, sc, nbuffers, stride);
  }
}

}  // namespace kernels
}  // namespace cudadma_b200

#endif
