/*
 * cudadma.h -- Blackwell (sm_100a) implementation of the CudaDMA object API.
 *
 * The classes keep the template and constructor surface of the CudaDMA v2
 * header (reference: include/cudaDMAv2.h, plus the v1 halo class in
 * include/cudaDMA.h:3653-4156) so that kernels written against it compile
 * unchanged, but none of the reference's machinery is kept:
 *
 *   - the named-barrier handshake (bar.sync / bar.arrive, cudaDMAv2.h:65-75)
 *     is an mbarrier pair per dmaID ("empty" counts compute threads, "full"
 *     counts DMA threads and async-copy transaction bytes);
 *   - data never passes through registers: contiguous runs move with
 *     cp.async.bulk, tiles with cp.async.bulk.tensor (TMA tensor maps,
 *     hardware zero fill outside the tensor), 16-byte-unaligned or
 *     non-specialised transfers with per-thread cp.async (4/8/16 bytes);
 *   - shared->global transfers (scatter, write-back) are bulk stores;
 *   - every wait is bounded: when a wait gives up it records a code in a
 *     device status word and the call returns, so a wrong thread count ends
 *     the kernel with an error status instead of hanging the GPU.
 *
 * Threading contract (same as the reference, cudaDMAv2.h:1316-1353):
 * every thread of the CTA constructs every object, at a point all threads
 * reach (the warp-specialised constructor contains a __syncthreads()); DMA
 * threads are threadIdx.x in [dma_threadIdx_start, +num_dma_threads).
 */
#ifndef CUDADMA_B200_CUDADMA_H
#define CUDADMA_B200_CUDADMA_H

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#ifndef CUDADMA_MAX_IDS
#define CUDADMA_MAX_IDS 16 /* dmaID range per CTA: 0 .. CUDADMA_MAX_IDS-1 (a power of two) */
#endif
#ifndef CUDADMA_WAIT_LIMIT_CYCLES
#define CUDADMA_WAIT_LIMIT_CYCLES (1ll << 31) /* about one second of SM clocks */
#endif

/* Cache qualifiers accepted as template arguments (reference: cudaDMAv2.h:50-63).
 * On this implementation loads map to an L2 eviction hint on bulk copies and
 * to .ca/.cg on cp.async; store qualifiers are accepted and ignored because
 * the destination of a load-type DMA is shared memory. */
enum CudaDMALoadQualifier {
  LOAD_CACHE_ALL = 0,
  LOAD_CACHE_GLOBAL = 1,
  LOAD_CACHE_STREAMING = 2,
  LOAD_CACHE_LAST_USE = 3,
  LOAD_CACHE_VOLATILE = 4
};
enum CudaDMAStoreQualifier {
  STORE_WRITE_BACK = 0,
  STORE_CACHE_GLOBAL = 1,
  STORE_CACHE_STREAMING = 2,
  STORE_CACHE_WRITE_THROUGH = 3
};

namespace cudadma_b200 {

/* Status word of this translation unit: 0, or the code of the first wait that
 * gave up. Layout: bit31 set | dmaID << 8 | 1 (empty wait) or 2 (full wait). */
static __device__ unsigned int g_status_word = 0;

/* Host helper: read and clear the status word (stream-ordered, then waits). */
static inline __host__ cudaError_t read_status(unsigned int *out, cudaStream_t stream = 0) {
  unsigned int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_status_word, sizeof(unsigned int), 0,
                                            cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return e;
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return e;
  if (*out != 0) e = cudaMemcpyToSymbolAsync(g_status_word, &zero, sizeof(unsigned int), 0,
                                              cudaMemcpyHostToDevice, stream);
  return e;
}

/*
 * -DCUDADMA_CHECKED: a debugging build for machines without a memory checker. The caller names the
 * ranges of global memory that transfers may touch (checked::set_windows, up to eight); every
 * transfer of the engine then tests each run of bytes it is about to move -- global addresses
 * against those ranges, shared addresses against the CTA's shared-memory size -- and a transfer
 * with a run outside is not issued at all: the first such run is recorded (checked::read_violation)
 * and the status word gets the code 0x8000B000 | dmaID-less kind (1 source, 2 destination), the
 * handshake completes as usual, and the kernel runs on with a buffer that was not filled instead
 * of faulting. Tensor-map transfers are bounded by their map and are not tested.
 */
#ifdef CUDADMA_CHECKED
namespace checked {
struct Windows { unsigned long long lo[8], hi[8]; int n; };
struct Violation { unsigned long long address, bytes; unsigned int kind, block, thread, pad; };
static __device__ Windows g_windows = {{0}, {0}, 0};
static __device__ Violation g_violation = {0, 0, 0, 0, 0, 0};

/* bases[i] .. bases[i] + bytes[i] are the ranges of global memory a transfer may read or write */
static inline __host__ cudaError_t set_windows(const void *const *bases, const size_t *bytes, int n,
                                               cudaStream_t stream = 0) {
  Windows w;
  if (n < 0 || n > 8) return cudaErrorInvalidValue;
  for (int i = 0; i < 8; ++i) {
    w.lo[i] = i < n ? (unsigned long long)reinterpret_cast<uintptr_t>(bases[i]) : 0ull;
    w.hi[i] = i < n ? w.lo[i] + bytes[i] : 0ull;
  }
  w.n = n;
  cudaError_t e = cudaMemcpyToSymbolAsync(g_windows, &w, sizeof(w), 0, cudaMemcpyHostToDevice, stream);
  return e != cudaSuccess ? e : cudaStreamSynchronize(stream);
}
/* reads and clears the record of the first refused run (kind 0 = none) */
static inline __host__ cudaError_t read_violation(Violation *out, cudaStream_t stream = 0) {
  const Violation none = {0, 0, 0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_violation, sizeof(Violation), 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess && out->kind != 0)
    e = cudaMemcpyToSymbolAsync(g_violation, &none, sizeof(none), 0, cudaMemcpyHostToDevice, stream);
  return e;
}
__device__ __forceinline__ bool run_ok(const void *p, unsigned long long bytes) {
  if (__isShared(p)) {
    unsigned int total;
    asm volatile("mov.u32 %0, %%total_smem_size;" : "=r"(total));
    const unsigned long long off = (unsigned long long)__cvta_generic_to_shared(p);
    return off + bytes <= total;
  }
  const unsigned long long a = (unsigned long long)reinterpret_cast<uintptr_t>(p);
  for (int i = 0; i < g_windows.n; ++i)
    if (a >= g_windows.lo[i] && a + bytes <= g_windows.hi[i]) return true;
  return false;
}
__device__ __forceinline__ void record(const void *p, unsigned long long bytes, unsigned int kind) {
  if (atomicCAS(&g_status_word, 0u, 0x8000B000u | kind) == 0u) {
    g_violation.address = (unsigned long long)reinterpret_cast<uintptr_t>(p);
    g_violation.bytes = bytes;
    g_violation.block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    g_violation.thread = threadIdx.x;
    g_violation.kind = kind;
  }
}
/* true when every run of the transfer lies inside what it may touch; the calling thread tests the
 * runs it would move itself and all threads of the transfer get the same answer only if they
 * all pass -- so the test is made on ALL runs by every thread (debug build: cost is not a concern) */
template <typename ROWS>
__device__ __forceinline__ bool transfer_ok(const ROWS &a, int rows, int row_bytes) {
  for (int r = 0; r < rows; ++r) {
    const void *s = a.src_row(r);
    const void *d = a.dst_row(r);
    if (!run_ok(s, (unsigned long long)row_bytes)) { record(s, (unsigned long long)row_bytes, 1u); return false; }
    if (!run_ok(d, (unsigned long long)row_bytes)) { record(d, (unsigned long long)row_bytes, 2u); return false; }
  }
  return true;
}
}  // namespace checked
#endif

namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t gmem_u64(const void *p) {
  return static_cast<uint64_t>(__cvta_generic_to_global(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
/* Arrival of the calling thread. Every thread arrives for itself: one arrival per warp with the
 * lane count (CUDADMA_WARP_AGGREGATED_ARRIVE) saves mbarrier operations but puts a warp
 * synchronisation, a vote and a population count into the release -> refill -> consume chain, and
 * measured slower wherever it made a difference (the reference's saxpy example, 1 KiB per
 * transfer: 0.78 against 0.62 ms; the stencil kernel: 3 %; the bandwidth-bound kernels: equal). */
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
#ifndef CUDADMA_WARP_AGGREGATED_ARRIVE
  mbar_arrive(bar);
#else
  const unsigned mask = __activemask();
  __syncwarp(mask);
  if ((threadIdx.x & 31u) == (unsigned)(__ffs(mask) - 1)) mbar_arrive_n(bar, (uint32_t)__popc(mask));
#endif
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
/* Arrival that fires when this thread's earlier cp.async copies have landed. */
__device__ __forceinline__ void mbar_arrive_after_cp_async(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
/* hardware (named) barriers: id 1..15, count a multiple of 32 */
__device__ __forceinline__ void named_sync(uint32_t id, uint32_t count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_arrive(uint32_t id, uint32_t count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
/* global -> shared, contiguous, size and both addresses multiples of 16 */
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(gmem_u64(src)), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(dst),
      "l"(gmem_u64(src)), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
/* shared -> global, contiguous, size and both addresses multiples of 16 */
__device__ __forceinline__ void bulk_s2g(void *dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_u64(dst)), "r"(src),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem_u64(src)), "r"(bytes) : "memory");
}
/* TMA tile loads; x is the innermost coordinate and x * element size must be a multiple of 16 bytes */
__device__ __forceinline__ void tensor_g2s_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tensor_g2s_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], "
      "[%5];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
/* TMA row gather: four rows y0..y3 of a 2-D tensor, columns [x, x + box width) */
__device__ __forceinline__ void tensor_gather4(uint32_t dst, const CUtensorMap *map, int x, int y0, int y1, int y2,
                                               int y3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
      "%4, %5, %6}], [%7];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(bar)
      : "memory");
}
/* TMA row scatter: four packed rows from shared memory to rows y0..y3 of a 2-D tensor (bulk group) */
__device__ __forceinline__ void tensor_scatter4(const CUtensorMap *map, int x, int y0, int y1, int y2, int y3,
                                                uint32_t src) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.tile::scatter4.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];" ::"l"(
          reinterpret_cast<uint64_t>(map)),
      "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(src)
      : "memory");
}
/* per-thread asynchronous copy global -> shared of UNIT = 4, 8 or 16 bytes.
 * HALF_LINE: the copy belongs to a run of at most 64 bytes whose neighbourhood nobody wants (a
 * gathered record). A miss then fetches 64 bytes from DRAM instead of the whole 128-byte line,
 * which is what a load without the .L2::64B qualifier costs on this part (measured: 2^22 random
 * 32-byte records read 533 MB of DRAM without it and 292 MB with it). */
template <int UNIT, bool L2_ONLY, bool HALF_LINE = false>
__device__ __forceinline__ void ldgsts(uint32_t dst, const void *src) {
  if (HALF_LINE) {
    if (UNIT == 16 && L2_ONLY)
      asm volatile("cp.async.cg.shared.global.L2::64B [%0], [%1], 16;" ::"r"(dst), "l"(gmem_u64(src)) : "memory");
    else
      asm volatile("cp.async.ca.shared.global.L2::64B [%0], [%1], %2;" ::"r"(dst), "l"(gmem_u64(src)), "n"(UNIT)
                   : "memory");
  } else {
    if (UNIT == 16 && L2_ONLY)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_u64(src)) : "memory");
    else
      asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(gmem_u64(src)), "n"(UNIT)
                   : "memory");
  }
}
__device__ __forceinline__ void ldgsts_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

}  // namespace ptx

namespace detail {

/* Two mbarriers per dmaID, shared by every object of the CTA. */
__device__ __forceinline__ uint32_t barrier_addr(int dmaID, int which) {
  __shared__ __align__(8) unsigned long long bars[2 * CUDADMA_MAX_IDS];
  /* an id outside 0 .. CUDADMA_MAX_IDS - 1 wraps around (and the constructor records a status code)
   * rather than addressing shared memory that belongs to somebody else */
  return ptx::smem_u32(bars) + 8u * (2u * ((unsigned)dmaID % (unsigned)CUDADMA_MAX_IDS) + (unsigned)which);
}

/* Slow half of a wait: keeps polling, gives up after CUDADMA_WAIT_LIMIT_CYCLES
 * or as soon as any earlier wait of the grid has given up. Returns whether the barrier was
 * passed. (Sleeping between polls, 32 ns to 2 us, and a suspend-time hint on the poll were both
 * measured on the stencil kernel, whose DMA warps wait most of the time, also with the GPU at its
 * power cap: no gain from the first, a 1 % loss from the second.)
 * A thread that gives up first sleeps for a few microseconds: copies that other threads issued
 * just before the failure are still on their way into this CTA's shared memory, and a thread
 * that ran on to the end of the kernel at once could take the CTA away from under them. */
inline __device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, unsigned int code) {
  const long long t0 = clock64();
  unsigned int polls = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    ++polls;
    if (polls == 16 || (polls & 1023u) == 0) {
      const bool lost = *reinterpret_cast<volatile unsigned int *>(&g_status_word) != 0;
      if (!lost && clock64() - t0 <= (long long)CUDADMA_WAIT_LIMIT_CYCLES) continue;
      if (!lost) atomicCAS(&g_status_word, 0u, code);
      __nanosleep(4000);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, unsigned int code) {
  return ptx::mbar_try_wait(bar, parity) || wait_slow(bar, parity, code);
}

template <int UNIT> struct unit_type;
template <> struct unit_type<4> { typedef unsigned int type; };
template <> struct unit_type<8> { typedef uint2 type; };
template <> struct unit_type<16> { typedef uint4 type; };

/* Addressing of a transfer made of `rows` contiguous runs of `row_bytes`. */
struct StridedRows {
  static constexpr bool SCATTERED_SOURCE = false; /* rows of one array: neighbouring rows want the rest of a line */
  const char *src; char *dst; long long src_stride; long long dst_stride;
  __device__ __forceinline__ const char *src_row(int r) const { return src + (long long)r * src_stride; }
  __device__ __forceinline__ char *dst_row(int r) const { return dst + (long long)r * dst_stride; }
};
/* gather: row r comes from src + index[r] * row_bytes, lands at dst + r * pitch */
struct GatherRows {
  static constexpr bool SCATTERED_SOURCE = true;
  const char *src; char *dst; const int *index; long long row_bytes; long long pitch;
  __device__ __forceinline__ const char *src_row(int r) const { return src + (long long)__ldg(index + r) * row_bytes; }
  __device__ __forceinline__ char *dst_row(int r) const { return dst + (long long)r * pitch; }
};
/* scatter: row r comes from src + r * pitch, lands at dst + index[r] * row_bytes */
struct ScatterRows {
  static constexpr bool SCATTERED_SOURCE = false;
  const char *src; char *dst; const int *index; long long row_bytes; long long pitch;
  __device__ __forceinline__ const char *src_row(int r) const { return src + (long long)r * pitch; }
  __device__ __forceinline__ char *dst_row(int r) const { return dst + (long long)__ldg(index + r) * row_bytes; }
};

/* Largest of 16/8/4 that divides every address, stride and length OR-ed into `mask`. */
__device__ __forceinline__ int copy_unit(unsigned long long mask) {
  if ((mask & 15) == 0) return 16;
  if ((mask & 7) == 0) return 8;
  return 4;
}

/* Walk all UNIT-sized pieces of all rows, thread `tid` of `nthreads`, and hand
 * (row, byte offset) to `op`. One division at entry, none in the loop. */
template <int UNIT, typename OP>
__device__ __forceinline__ void for_each_unit(int rows, int row_bytes, int tid, int nthreads, OP op) {
  const int upr = row_bytes / UNIT;
  if (upr <= 0 || tid < 0 || tid >= nthreads) return;
  int r = tid / upr, c = tid - r * upr;
  const int dr = nthreads / upr, dc = nthreads - dr * upr;
  while (r < rows) {
    op(r, c * UNIT);
    r += dr; c += dc;
    if (c >= upr) { c -= upr; ++r; }
  }
}

/* global -> shared with per-thread cp.async in pieces of `unit` bytes. HALF_LINE: see ptx::ldgsts;
 * set for scattered rows (gathers) of at most 64 bytes. */
template <bool L2_ONLY, bool HALF_LINE, typename ROWS>
__device__ __forceinline__ void ldgsts_rows(const ROWS &a, int rows, int row_bytes, int unit, int tid, int nthreads) {
  if (unit == 16)
    for_each_unit<16>(rows, row_bytes, tid, nthreads, [&](int r, int off) {
      ptx::ldgsts<16, L2_ONLY, HALF_LINE>(ptx::smem_u32(a.dst_row(r) + off), a.src_row(r) + off); });
  else if (unit == 8)
    for_each_unit<8>(rows, row_bytes, tid, nthreads, [&](int r, int off) {
      ptx::ldgsts<8, false, HALF_LINE>(ptx::smem_u32(a.dst_row(r) + off), a.src_row(r) + off); });
  else
    for_each_unit<4>(rows, row_bytes, tid, nthreads, [&](int r, int off) {
      ptx::ldgsts<4, false, HALF_LINE>(ptx::smem_u32(a.dst_row(r) + off), a.src_row(r) + off); });
}

/* any address space -> any address space through registers (generic ld / st) */
template <typename ROWS>
__device__ __forceinline__ void generic_rows(const ROWS &a, int rows, int row_bytes, int unit, int tid, int nthreads) {
  if (unit == 16)
    for_each_unit<16>(rows, row_bytes, tid, nthreads, [&](int r, int off) {
      *reinterpret_cast<uint4 *>(a.dst_row(r) + off) = *reinterpret_cast<const uint4 *>(a.src_row(r) + off); });
  else if (unit == 8)
    for_each_unit<8>(rows, row_bytes, tid, nthreads, [&](int r, int off) {
      *reinterpret_cast<uint2 *>(a.dst_row(r) + off) = *reinterpret_cast<const uint2 *>(a.src_row(r) + off); });
  else
    for_each_unit<4>(rows, row_bytes, tid, nthreads, [&](int r, int off) {
      *reinterpret_cast<unsigned int *>(a.dst_row(r) + off) =
          *reinterpret_cast<const unsigned int *>(a.src_row(r) + off); });
}

__device__ __forceinline__ unsigned long long addr_bits(const void *p) {
  return (unsigned long long)reinterpret_cast<uintptr_t>(p);
}

}  // namespace detail
}  // namespace cudadma_b200

/* ------------------------------------------------------------------------- */
/* Base class: ownership test and the four synchronisation calls             */
/* (reference: cudaDMAv2.h:1316-1353; the two DMA-side calls are public here  */
/* as they are in the v1 classes, cudaDMA.h:839-846).                        */
/* ------------------------------------------------------------------------- */
class CudaDMA {
 public:
  /* do_sync == false builds an object without barriers (non-specialised mode).
   * async_proxy == false: the derived class knows at compile time that none of its transfers can go
   * through the bulk-copy engine (rows too short for it), so the two calls that hand the buffer
   * over need no proxy fence; the tensor-map extensions of such a class fence for themselves.
   * hardware_barriers == true: the derived class never issues an asynchronous copy at all (it
   * moves its bytes through registers, or the caller does), so nothing has to be counted by an
   * mbarrier and the handshake can be the reference's own pair of hardware barriers
   * (bar.sync / bar.arrive, cudaDMAv2.h:65-75), whose crossing is cheaper (about 50 ns against 80).
   * Barrier ids are 2 * dmaID + 1 (empty) and 2 * dmaID + 2 (full), so id 0 (__syncthreads) stays
   * free and dmaIDs 0..6 qualify (which object does is decided by its type and its dmaID alone,
   * so with a literal dmaID the other mechanism costs no registers); objects with a higher dmaID
   * use mbarriers as all others do. As in the reference, the DMA threads and the compute threads
   * of such an object must each be whole warps (bar counts threads in units of 32), and a wait on
   * a hardware barrier is NOT bounded: it hangs when the two sides disagree about the thread
   * counts. -DCUDADMA_NO_NAMED_BARRIERS keeps every object on mbarriers and every wait bounded. */
  __device__ __forceinline__ CudaDMA(const int dmaID, const int num_dma_threads, const int num_compute_threads,
                                     const int dma_threadIdx_start, const bool do_sync = true,
                                     const bool async_proxy = true, const bool hardware_barriers = false)
      : m_dma_tid(int(threadIdx.x) - dma_threadIdx_start),
        m_num_dma_threads(num_dma_threads),
        m_is_dma_thread((int(threadIdx.x) >= dma_threadIdx_start) &&
                        (int(threadIdx.x) < (dma_threadIdx_start + num_dma_threads))),
#ifdef CUDADMA_NO_NAMED_BARRIERS
        m_named(false),
#else
        m_named(do_sync && hardware_barriers && dmaID >= 0 && dmaID <= 6),
#endif
        m_bar_empty(!do_sync ? 0u : m_named ? (uint32_t)(2 * dmaID + 1) : cudadma_b200::detail::barrier_addr(dmaID, 0)),
        m_bar_full(!do_sync ? 0u : m_named ? (uint32_t)(2 * dmaID + 2) : cudadma_b200::detail::barrier_addr(dmaID, 1)),
        m_code(0x80000000u | ((unsigned)dmaID << 8)),
        m_async_proxy(async_proxy),
        m_count((uint32_t)(num_dma_threads + num_compute_threads)),
        m_phase(0),
        m_gave_up(false) {
    if (do_sync && (dmaID < 0 || dmaID >= CUDADMA_MAX_IDS)) /* barrier_addr() wraps the id around; say so */
      atomicCAS(&cudadma_b200::g_status_word, 0u, 0x8000D000u | ((unsigned)dmaID & 0xFFu));
    if (do_sync && !m_named) {
      if (int(threadIdx.x) == dma_threadIdx_start) {
        cudadma_b200::ptx::mbar_init(m_bar_empty, (uint32_t)num_compute_threads);
        cudadma_b200::ptx::mbar_init(m_bar_full, (uint32_t)num_dma_threads);
        cudadma_b200::ptx::mbar_fence_init();
      }
      __syncthreads();
    }
  }

 public:
  /* compute threads: the buffer may be overwritten (or, for a scatter, read) by the DMA threads */
  __device__ __forceinline__ void start_async_dma(void) const {
    if (m_named) { cudadma_b200::ptx::named_arrive(m_bar_empty, m_count); return; }
    if (m_async_proxy) cudadma_b200::ptx::fence_proxy_async();
    cudadma_b200::ptx::mbar_arrive_warp(m_bar_empty);
  }
  /* Extension (not in the reference): start_async_dma() for compute threads that have only READ the
   * buffer since it was last filled. The proxy fence above exists to make a thread's own shared-memory
   * WRITES visible to the bulk-copy engine; reads are ordered before the next transfer by the arrival
   * alone, so a kernel that releases a buffer every few hundred instructions can leave the fence out. */
  __device__ __forceinline__ void start_async_dma_after_reads(void) const {
    if (m_named) { cudadma_b200::ptx::named_arrive(m_bar_empty, m_count); return; }
    cudadma_b200::ptx::mbar_arrive_warp(m_bar_empty);
  }
  /* compute threads: block until the transfer has landed */
  __device__ __forceinline__ void wait_for_dma_finish(void) const {
    if (m_named) { cudadma_b200::ptx::named_sync(m_bar_full, m_count); return; }
    cudadma_b200::detail::bounded_wait(m_bar_full, m_phase, m_code | 2u);
    m_phase ^= 1u;
  }
  __device__ __forceinline__ bool owns_this_thread(void) const { return m_is_dma_thread; }
  /* DMA threads: block until the compute threads have released the buffer. When the wait gives up
   * (or the grid has failed already) the object issues no further asynchronous copies: nothing may
   * still be on its way into shared memory when the kernel winds down with its error status. */
  __device__ __forceinline__ void wait_for_dma_start(void) const {
    if (m_named) { cudadma_b200::ptx::named_sync(m_bar_empty, m_count); return; }
    if (!cudadma_b200::detail::bounded_wait(m_bar_empty, m_phase, m_code | 1u)) m_gave_up = true;
    m_phase ^= 1u;
    if (m_async_proxy) cudadma_b200::ptx::fence_proxy_async();
  }
  /* the same wait for DMA threads that will fill the buffer with ordinary stores: no proxy fence */
  __device__ __forceinline__ void wait_for_dma_start_for_stores(void) const {
    if (m_named) { cudadma_b200::ptx::named_sync(m_bar_empty, m_count); return; }
    if (!cudadma_b200::detail::bounded_wait(m_bar_empty, m_phase, m_code | 1u)) m_gave_up = true;
    m_phase ^= 1u;
  }
  /* Extension: true once a wait of this thread on this object has given up (see wait_for_dma_start) */
  __device__ __forceinline__ bool gave_up(void) const { return m_gave_up; }
  /* DMA threads: this thread's share of the transfer is complete (or tracked by the barrier) */
  __device__ __forceinline__ void finish_async_dma(void) const {
    if (m_named) { cudadma_b200::ptx::named_arrive(m_bar_full, m_count); return; }
    cudadma_b200::ptx::mbar_arrive_warp(m_bar_full);
  }

 protected:
  const int m_dma_tid;
  const int m_num_dma_threads;
  const bool m_is_dma_thread;
  const bool m_named;         /* hardware barriers instead of mbarriers (see the constructor) */
  const uint32_t m_bar_empty; /* shared-memory address of the mbarrier, or the hardware barrier's id */
  const uint32_t m_bar_full;
  const unsigned int m_code;
  const bool m_async_proxy;
  const uint32_t m_count;     /* threads of both sides together */
  mutable uint32_t m_phase; /* parity this thread waits for next (empty for DMA threads, full for compute) */
  mutable bool m_gave_up;   /* a wait for the buffer gave up: no asynchronous copy is issued any more */
};

namespace cudadma_b200 {
namespace detail {

/*
 * The transfer engine behind every class. ROWS supplies src_row(r) and
 * dst_row(r); a transfer is `rows` runs of `row_bytes` bytes and `mask` is
 * the OR of every address, stride and length involved (it decides between
 * bulk copies, 16/8/4-byte cp.async and 16/8/4-byte register copies).
 *
 *   WS  : warp-specialised. The DMA threads call issue_rows() (any number of
 *         times) after the empty wait and then complete() exactly once:
 *         bytes moved by bulk copies are added to the full barrier's
 *         transaction count, cp.async copies trigger the thread's arrival
 *         when they land, so the DMA thread itself never waits for data.
 *   !WS : every participating thread issues cp.async copies and complete()
 *         waits for the caller's own copies; the caller's __syncthreads()
 *         then publishes them to the CTA.
 * issue_rows() returns 1 when the calling thread has cp.async copies pending.
 */
#ifndef CUDADMA_BULK_ROW_MIN
#define CUDADMA_BULK_ROW_MIN 64 /* rows shorter than this use cp.async, not one bulk copy each */
#endif

template <bool WS, int LOAD_QUAL, typename ROWS>
__device__ __forceinline__ int issue_rows(const ROWS &a, const int rows, const int row_bytes,
                                          const unsigned long long mask, const int tid, const int nthreads,
                                          const uint32_t bar_full) {
  constexpr bool L2_ONLY = (LOAD_QUAL != LOAD_CACHE_ALL);
  constexpr bool EVICT_FIRST = (LOAD_QUAL == LOAD_CACHE_STREAMING) || (LOAD_QUAL == LOAD_CACHE_LAST_USE);
  if (rows <= 0 || row_bytes <= 0) return 0;
#ifdef CUDADMA_CHECKED
  if (!checked::transfer_ok(a, rows, row_bytes)) return 0;
#endif
  const char *s0 = a.src_row(0);
  char *d0 = a.dst_row(0);
  const int unit = copy_unit(mask);
  if (__isGlobal(s0) && __isShared(d0)) {
    if (WS && unit == 16 && row_bytes >= CUDADMA_BULK_ROW_MIN) {
      /* one bulk copy per row, rows dealt round-robin to the DMA threads */
      const int mine = (rows > tid) ? (rows - tid + nthreads - 1) / nthreads : 0;
      if (mine > 0) {
        ptx::mbar_expect_tx(bar_full, (uint32_t)mine * (uint32_t)row_bytes);
        if (EVICT_FIRST) {
          const uint64_t pol = ptx::policy_evict_first();
          for (int r = tid; r < rows; r += nthreads)
            ptx::bulk_g2s_hint(ptx::smem_u32(a.dst_row(r)), a.src_row(r), (uint32_t)row_bytes, bar_full, pol);
        } else {
          for (int r = tid; r < rows; r += nthreads)
            ptx::bulk_g2s(ptx::smem_u32(a.dst_row(r)), a.src_row(r), (uint32_t)row_bytes, bar_full);
        }
      }
      return 0;
    }
    if (ROWS::SCATTERED_SOURCE && row_bytes <= 64) ldgsts_rows<L2_ONLY, true>(a, rows, row_bytes, unit, tid, nthreads);
    else ldgsts_rows<L2_ONLY, false>(a, rows, row_bytes, unit, tid, nthreads);
    return 1;
  }
  if (__isShared(s0) && __isGlobal(d0) && unit == 16 && row_bytes >= CUDADMA_BULK_ROW_MIN) {
    /* Bulk stores. The call returns once shared memory has been READ (the buffer may be refilled);
     * the global writes complete asynchronously, at the latest at kernel end: a thread that wants
     * to read the destination back inside the same kernel must first wait for the whole bulk
     * group (cp.async.bulk.wait_group 0), which the reference's plain stores did not need. */
    ptx::fence_proxy_async();
    if (tid >= 0) {
      for (int r = tid; r < rows; r += nthreads)
        ptx::bulk_s2g(a.dst_row(r), ptx::smem_u32(a.src_row(r)), (uint32_t)row_bytes);
    }
    ptx::bulk_commit();
    ptx::bulk_wait_read<0>();
    return 0;
  }
  generic_rows(a, rows, row_bytes, unit, tid, nthreads);
  return 0;
}

template <bool WS>
__device__ __forceinline__ void complete(const int cp_async_pending, const uint32_t bar_full) {
  if (WS) {
    if (cp_async_pending) ptx::mbar_arrive_after_cp_async(bar_full);
    else ptx::mbar_arrive_warp(bar_full);
  } else {
    if (cp_async_pending) ptx::ldgsts_wait_all();
  }
}

/* Contiguous run. In warp-specialised mode the 16-byte-aligned body is cut
 * into one bulk copy per DMA warp (lane 0 issues it) and a 4/8/12-byte tail
 * goes through registers; everything else takes the row engine. */
template <bool WS, int LOAD_QUAL>
__device__ __forceinline__ int issue_contiguous(const char *src, char *dst, const int bytes, const int tid,
                                                const int nthreads, const uint32_t bar_full) {
  constexpr bool EVICT_FIRST = (LOAD_QUAL == LOAD_CACHE_STREAMING) || (LOAD_QUAL == LOAD_CACHE_LAST_USE);
  const unsigned long long ends = addr_bits(src) | addr_bits(dst);
#ifdef CUDADMA_CHECKED
  {
    const StridedRows whole = {src, dst, 0, 0};
    if (bytes > 0 && !checked::transfer_ok(whole, 1, bytes)) return 0;
  }
#endif
  if (WS && (ends & 15) == 0 && bytes >= CUDADMA_BULK_ROW_MIN && __isGlobal(src) && __isShared(dst)) {
    const int body = bytes & ~15;
    const int nwarps = (nthreads + 31) >> 5;
    int piece = ((body + nwarps - 1) / nwarps + 15) & ~15;
    if (piece < 2048) piece = 2048;
    const int off = (tid >> 5) * piece;
    if (bytes > body && tid == (nthreads > 1 ? 1 : 0)) {
      for (int o = body; o < bytes; o += 4)
        *reinterpret_cast<unsigned int *>(dst + o) = *reinterpret_cast<const unsigned int *>(src + o);
    }
    if ((tid & 31) == 0 && off < body) {
      const int len = (body - off < piece) ? (body - off) : piece;
      ptx::mbar_expect_tx(bar_full, (uint32_t)len);
      if (EVICT_FIRST)
        ptx::bulk_g2s_hint(ptx::smem_u32(dst + off), src + off, (uint32_t)len, bar_full, ptx::policy_evict_first());
      else
        ptx::bulk_g2s(ptx::smem_u32(dst + off), src + off, (uint32_t)len, bar_full);
    }
    return 0;
  }
  StridedRows a = {src, dst, 0, 0};
  return issue_rows<WS, LOAD_QUAL>(a, 1, bytes, ends | (unsigned long long)bytes, tid, nthreads, bar_full);
}

/* Small warp-specialised loads are latency-bound: the copy may only start once the compute threads
 * have released the buffer, and then pays a full trip to DRAM. start_xfer_async() (which runs
 * before that wait) therefore asks for the source to be brought into L2 meanwhile, so that the
 * copy itself is an L2 hit (the reference's strided saxpy example, three rows of 1 KiB per
 * transfer: 1.80 -> 1.41 ms). Only for transfers of at most CUDADMA_SMALL_PREFETCH_BYTES in at
 * most CUDADMA_SMALL_PREFETCH_ROWS rows: larger ones are bandwidth-bound and run several buffers
 * deep anyway, and a prefetch per row of a many-row window doubles the DMA threads' work (a
 * 24-row stencil window lost 30 % with it). */
#ifndef CUDADMA_SMALL_PREFETCH_BYTES
#define CUDADMA_SMALL_PREFETCH_BYTES 4096
#endif
#ifndef CUDADMA_SMALL_PREFETCH_ROWS
#define CUDADMA_SMALL_PREFETCH_ROWS 4
#endif
__device__ __forceinline__ void prefetch_small(const char *src, const int rows, const int row_bytes,
                                               const long long src_stride, const int tid, const int nthreads) {
#ifdef CUDADMA_CHECKED
  return; /* nothing is touched before it has been tested */
#endif
  if (CUDADMA_SMALL_PREFETCH_BYTES <= 0 || rows <= 0 || row_bytes < 16 || tid < 0 || tid >= nthreads) return;
  if (rows > CUDADMA_SMALL_PREFETCH_ROWS || (long long)rows * row_bytes > CUDADMA_SMALL_PREFETCH_BYTES) return;
  if (((addr_bits(src) | (unsigned long long)row_bytes | (unsigned long long)src_stride) & 15) || !__isGlobal(src)) return;
  for (int r = tid; r < rows; r += nthreads) ptx::bulk_prefetch_l2(src + (long long)r * src_stride, (uint32_t)row_bytes);
}

/*
 * Register staging for small, fully templated transfers: ROWS rows of ROW_BYTES bytes (a multiple
 * of 16) moved by NTHREADS threads in 16-byte units, unit i = thread + k * NTHREADS of the row-major
 * list of units. The loads are issued in start_xfer_async(), i.e. BEFORE the DMA threads wait for
 * the buffer, the stores after the wait -- the reference's scheme for everything
 * (cudaDMAv2.h:1461-1475). Loops of small transfers are latency chains (compute releases, DMA
 * fills, compute consumes), and a copy that may only start once the buffer is free pays a whole
 * trip to memory per link where the early loads overlap it with the consumer's work on the
 * previous buffer (the reference's saxpy example, 1 KiB per transfer: 0.39 us per iteration
 * against 0.19). All indices are compile-time, so the staging array stays in registers.
 * A unit's offset from the base pointer is computed in 32-bit ints, as the reference's offsets
 * are: the rows of a staged transfer must lie within 2 GiB of its base pointer. (With 64-bit
 * offsets the compiler keeps one register pair per unit and pointer alive across the caller's
 * loop: the reference's warp-specialised stencil examples took 72 registers against the
 * reference header's 60 and lost a CTA per SM; with ints they take 56.)
 */
template <int ROW_BYTES, int ROWS, int NTHREADS>
struct StagedShape {
  static constexpr int UPR = ROW_BYTES / 16;                             /* units per row */
  static constexpr int TOTAL = UPR * ROWS;
  static constexpr int UNITS = NTHREADS > 0 ? (TOTAL + NTHREADS - 1) / NTHREADS : 0; /* per thread */
};
template <int ROW_BYTES, int ROWS, int NTHREADS, bool L2_ONLY, bool GLOBAL_SRC, int N>
__device__ __forceinline__ void staged_load(uint4 (&v)[N], const char *src, const int src_stride, const int tid) {
  typedef StagedShape<ROW_BYTES, ROWS, NTHREADS> S;
#pragma unroll
  for (int k = 0; k < S::UNITS; ++k) {
    const int i = tid + k * NTHREADS;
    if ((k + 1) * NTHREADS <= S::TOTAL || i < S::TOTAL) {
      const int r = i / S::UPR, c = i - r * S::UPR;
      const uint4 *g = reinterpret_cast<const uint4 *>(src + (r * src_stride + 16 * c));
      /* Which load: an explicit cache qualifier goes to L2 (ld.global.cg), everything else is a
       * plain load, which works from any address space.
       * -DCUDADMA_SOURCES_READ_ONLY (a promise: the kernel never writes what its transfer objects
       * read afterwards): global sources are read through the read-only data path (ld.global.nc),
       * as the reference does for DMA_GLOBAL_LOAD on the architecture it was tuned for
       * (cudaDMAv2.h:98-103). Such loads are not tied to the handshake's barriers, so the compiler
       * moves them: in the reference's saxpy examples it starts the next transfer's loads before
       * this one's wait (1.45 x and 1.23 x the reference header's speed instead of 0.93 x and
       * 0.95 x), in its warp-specialised double-buffer stencil it moves them behind the wait
       * (0.64 x instead of 1.09 x). Measure before keeping it.
       * Also measured: ld.global.cg for every global source gives +3 % on those saxpy loops and
       * +6 % on the portable stencil's windows, but -4 % on a streaming copy of 1 GiB. */
      if (L2_ONLY) v[k] = __ldcg(g);
#ifdef CUDADMA_SOURCES_READ_ONLY
      else if (GLOBAL_SRC) v[k] = __ldg(g);
      else v[k] = __isGlobal(g) ? __ldg(g) : *g;
#else
      else v[k] = *g;
#endif
    }
  }
}
/* direct: destination and its stride are multiples of 16 (else word by word) */
template <int ROW_BYTES, int ROWS, int NTHREADS, int N>
__device__ __forceinline__ void staged_store(const uint4 (&v)[N], char *dst, const int dst_stride, const int tid,
                                             const bool direct) {
  typedef StagedShape<ROW_BYTES, ROWS, NTHREADS> S;
#pragma unroll
  for (int k = 0; k < S::UNITS; ++k) {
    const int i = tid + k * NTHREADS;
    if ((k + 1) * NTHREADS <= S::TOTAL || i < S::TOTAL) {
      const int r = i / S::UPR, c = i - r * S::UPR;
      char *d = dst + (r * dst_stride + 16 * c);
      if (direct) {
        *reinterpret_cast<uint4 *>(d) = v[k];
      } else {
        unsigned int *w = reinterpret_cast<unsigned int *>(d);
        w[0] = v[k].x; w[1] = v[k].y; w[2] = v[k].z; w[3] = v[k].w;
      }
    }
  }
}

#ifndef CUDADMA_NAMED_MAX_DMA_THREADS
#define CUDADMA_NAMED_MAX_DMA_THREADS 1024 /* staged objects with more DMA threads hand over on mbarriers */
#endif
#ifndef CUDADMA_STAGED_SEQUENTIAL_MAX
#define CUDADMA_STAGED_SEQUENTIAL_MAX 128 /* bytes per DMA thread a CudaDMASequential object may hold in registers */
#endif

struct V1Forms {}; /* tag: constructor arguments mean what they mean in the v1 header */

/* Constructor arguments arrive as 0..8 ints whose meaning depends on the
 * template level; ArgList just holds them. */
struct ArgList {
  int v[8];
  int n;
};
template <typename... I>
__device__ __forceinline__ ArgList make_args(I... a) {
  static_assert(sizeof...(I) <= 8, "too many constructor arguments");
  const int given[sizeof...(I) + 1] = {int(a)..., 0};
  ArgList l;
  l.n = int(sizeof...(I));
#pragma unroll
  for (int i = 0; i < 8; ++i) l.v[i] = (i < int(sizeof...(I))) ? given[i < int(sizeof...(I)) ? i : 0] : 0;
  return l;
}

}  // namespace detail
}  // namespace cudadma_b200

#define CUDADMA_B200_XFER_OVERLOADS(SRC_DECL, SRC_ARGS)                                                     \
  __device__ __forceinline__ void execute_dma(SRC_DECL, void *__restrict__ dst_ptr) {                       \
    execute_impl<false, LOAD_CACHE_ALL>(SRC_ARGS, dst_ptr);                                                 \
  }                                                                                                         \
  __device__ __forceinline__ void start_xfer_async(SRC_DECL) { start_impl<false, LOAD_CACHE_ALL>(SRC_ARGS); } \
  __device__ __forceinline__ void wait_xfer_finish(void *__restrict__ dst_ptr) {                            \
    finish_impl<LOAD_CACHE_ALL>(dst_ptr);                                                                   \
  }                                                                                                         \
  template <bool DMA_GLOBAL_LOAD>                                                                           \
  __device__ __forceinline__ void execute_dma(SRC_DECL, void *__restrict__ dst_ptr) {                       \
    execute_impl<DMA_GLOBAL_LOAD, LOAD_CACHE_ALL>(SRC_ARGS, dst_ptr);                                       \
  }                                                                                                         \
  template <bool DMA_GLOBAL_LOAD>                                                                           \
  __device__ __forceinline__ void start_xfer_async(SRC_DECL) {                                              \
    start_impl<DMA_GLOBAL_LOAD, LOAD_CACHE_ALL>(SRC_ARGS);                                                  \
  }                                                                                                         \
  template <bool DMA_GLOBAL_LOAD>                                                                           \
  __device__ __forceinline__ void wait_xfer_finish(void *__restrict__ dst_ptr) {                            \
    finish_impl<LOAD_CACHE_ALL>(dst_ptr);                                                                   \
  }                                                                                                         \
  template <bool DMA_GLOBAL_LOAD, int DMA_LOAD_QUAL, int DMA_STORE_QUAL>                                    \
  __device__ __forceinline__ void execute_dma(SRC_DECL, void *__restrict__ dst_ptr) {                       \
    execute_impl<DMA_GLOBAL_LOAD, DMA_LOAD_QUAL>(SRC_ARGS, dst_ptr);                                        \
  }                                                                                                         \
  template <bool DMA_GLOBAL_LOAD, int DMA_LOAD_QUAL, int DMA_STORE_QUAL>                                    \
  __device__ __forceinline__ void start_xfer_async(SRC_DECL) {                                              \
    start_impl<DMA_GLOBAL_LOAD, DMA_LOAD_QUAL>(SRC_ARGS);                                                   \
  }                                                                                                         \
  template <bool DMA_GLOBAL_LOAD, int DMA_LOAD_QUAL, int DMA_STORE_QUAL>                                    \
  __device__ __forceinline__ void wait_xfer_finish(void *__restrict__ dst_ptr) {                            \
    finish_impl<DMA_LOAD_QUAL>(dst_ptr);                                                                    \
  }

/* ------------------------------------------------------------------------- */
/* CudaDMASequential: one contiguous run of BYTES_PER_ELMT bytes.            */
/* Template surface: cudaDMAv2.h:1367. Constructor forms, by how many of the  */
/* trailing template arguments are non-zero (cudaDMAv2.h:1848-1852,           */
/* :2265-2268, :2663-2665 warp-specialised; :2042-2044, :2449-2450, :2811 not):*/
/*   ws  L1 (dmaID, num_dma_threads, num_compute_threads, start, elmt_bytes)  */
/*   ws  L2 (dmaID, num_dma_threads, num_compute_threads, start)              */
/*   ws  L3 (dmaID, num_compute_threads, start)                               */
/*   nws L1 (elmt_bytes, num_dma_threads = 0, start = 0)                      */
/*   nws L2 (num_dma_threads = 0, start = 0)                                  */
/*   nws L3 (start = 0)                                                       */
/* BYTES_PER_THREAD bounds the register staging of fully templated objects   */
/* (see STAGED below) and is validated otherwise.                            */
/* ------------------------------------------------------------------------- */
template <bool DO_SYNC = false, int ALIGNMENT = 0, int BYTES_PER_THREAD = 4 * ALIGNMENT, int BYTES_PER_ELMT = 0,
          int DMA_THREADS = 0>
class CudaDMASequential : public CudaDMA {
  static_assert(ALIGNMENT == 4 || ALIGNMENT == 8 || ALIGNMENT == 16, "ALIGNMENT must be 4, 8 or 16");
  static_assert((BYTES_PER_THREAD / ALIGNMENT) > 0 && (BYTES_PER_THREAD % ALIGNMENT) == 0,
                "BYTES_PER_THREAD must be a positive multiple of ALIGNMENT");
  static constexpr int LEVEL = (BYTES_PER_ELMT == 0) ? 1 : ((DMA_THREADS == 0) ? 2 : 3);
  struct Params { int dmaID, ndma, ncomp, start, bytes; };
  __device__ __forceinline__ static Params decode(const cudadma_b200::detail::ArgList &l) {
    const int *a = l.v;
    Params p;
    if (DO_SYNC) {
      if (LEVEL == 1) p = {a[0], a[1], a[2], a[3], a[4]};
      else if (LEVEL == 2) p = {a[0], a[1], a[2], a[3], BYTES_PER_ELMT};
      else p = {a[0], DMA_THREADS, a[1], a[2], BYTES_PER_ELMT};
    } else {
      int nd, st, by;
      if (LEVEL == 1) { by = a[0]; nd = a[1]; st = a[2]; }
      else if (LEVEL == 2) { by = BYTES_PER_ELMT; nd = a[0]; st = a[1]; }
      else { by = BYTES_PER_ELMT; nd = DMA_THREADS; st = a[0]; }
      if (nd <= 0) nd = blockDim.x;
      p = {0, nd, nd, st, by};
    }
    return p;
  }
  /* Small, fully templated transfers are staged through registers (see detail::staged_load), with
   * plain loads and stores, so source and destination may be in any address space: at most 64 bytes
   * per DMA thread, or BYTES_PER_THREAD where the caller grants more (the reference's meaning of
   * that argument: the register budget of a DMA thread), up to 128. Loads that sit in registers
   * while the thread waits for the buffer are a buffer of their own: a streaming copy of 16 KiB
   * chunks by 128 DMA threads runs 3 % faster staged (BYTES_PER_THREAD = 128, three buffers, plain
   * stores for the write-back) than through cp.async.bulk in both directions, and within half a
   * per cent of a device-to-device cudaMemcpy. Such an object never issues an asynchronous copy, so its handshake can use
   * the hardware barriers (see class CudaDMA). With ALIGNMENT == 16 the object takes the caller's
   * word for it, as the reference does (a pointer less aligned than promised faults); with
   * ALIGNMENT 4 or 8 it looks at the pointers and, where they are not 16-byte aligned, copies
   * with smaller loads and stores after the wait instead. Larger transfers keep the asynchronous
   * copies, which take whatever alignment they find. */
  static constexpr int NT = DMA_THREADS > 0 ? DMA_THREADS : 1;
  static constexpr bool TRUST = ALIGNMENT == 16;
#if defined(CUDADMA_NO_REGISTER_STAGING) || defined(CUDADMA_CHECKED) /* checked builds move everything through the engine */
  static constexpr bool STAGED = false;
#else
  static constexpr int STAGE_BUDGET = BYTES_PER_THREAD < 64 ? 64 : (BYTES_PER_THREAD > CUDADMA_STAGED_SEQUENTIAL_MAX ? CUDADMA_STAGED_SEQUENTIAL_MAX : BYTES_PER_THREAD);
  static constexpr bool STAGED = LEVEL == 3 && BYTES_PER_ELMT % 16 == 0 && BYTES_PER_ELMT <= STAGE_BUDGET * NT;
#endif
  typedef cudadma_b200::detail::StagedShape<STAGED ? BYTES_PER_ELMT : 16, 1, NT> Shape;
  __device__ __forceinline__ CudaDMASequential(const Params &p, int)
      : CudaDMA(p.dmaID, p.ndma, p.ncomp, p.start, DO_SYNC, !STAGED, STAGED && NT <= CUDADMA_NAMED_MAX_DMA_THREADS), m_bytes(p.bytes), m_src(0),
        m_staged(false) {}

 public:
  template <typename... I>
  __device__ __forceinline__ CudaDMASequential(I... args)
      : CudaDMASequential(decode(cudadma_b200::detail::make_args(args...)), 0) {
    static_assert(DO_SYNC ? (sizeof...(I) == 6 - LEVEL) : (sizeof...(I) <= 4 - LEVEL),
                  "wrong number of constructor arguments for this template form");
  }
  CUDADMA_B200_XFER_OVERLOADS(const void *__restrict__ src_ptr, src_ptr)

 private:
  template <bool GLOBAL, int LQ>
  __device__ __forceinline__ void start_impl(const void *src) {
    m_src = static_cast<const char *>(src);
    if (STAGED) {
      m_staged = m_is_dma_thread && (TRUST || (cudadma_b200::detail::addr_bits(src) & 15) == 0);
      if (m_staged)
        cudadma_b200::detail::staged_load<STAGED ? BYTES_PER_ELMT : 16, 1, NT, GLOBAL && LQ != LOAD_CACHE_ALL, GLOBAL>(m_stage, m_src, 0, m_dma_tid);
      return;
    }
    if (DO_SYNC) cudadma_b200::detail::prefetch_small(m_src, 1, m_bytes, 0, m_dma_tid, m_num_dma_threads);
  }
  /* execute_dma: the whole transfer in one call. A staged object keeps the bytes in a local array
   * here, so that nothing of one transfer stays live into the next (the member array serves the
   * two-phase calls, where it has to). */
  template <bool GLOBAL, int LQ>
  __device__ __forceinline__ void execute_impl(const void *src, void *dst) {
    using namespace cudadma_b200::detail;
    if (STAGED) {
      const char *s = static_cast<const char *>(src);
      /* warp-specialised: only DMA threads call this (the reference's contract); otherwise every thread does */
      const bool early = (DO_SYNC || m_is_dma_thread) && (TRUST || (addr_bits(src) & 15) == 0);
      uint4 stage[Shape::UNITS > 0 ? Shape::UNITS : 1];
      if (early) staged_load<STAGED ? BYTES_PER_ELMT : 16, 1, NT, GLOBAL && LQ != LOAD_CACHE_ALL, GLOBAL>(stage, s, 0, m_dma_tid);
      if (DO_SYNC) wait_for_dma_start_for_stores();
      else if (!m_is_dma_thread) return;
      if (early) {
        staged_store<STAGED ? BYTES_PER_ELMT : 16, 1, NT>(stage, static_cast<char *>(dst), 0, m_dma_tid,
                                                          TRUST || (addr_bits(dst) & 15) == 0);
      } else if (!TRUST && m_is_dma_thread) {
        StridedRows a = {s, static_cast<char *>(dst), 0, 0};
        generic_rows(a, 1, m_bytes, copy_unit(addr_bits(s) | addr_bits(dst) | (unsigned long long)m_bytes), m_dma_tid,
                     m_num_dma_threads);
      }
      if (DO_SYNC) finish_async_dma();
      return;
    }
    start_impl<GLOBAL, LQ>(src);
    finish_impl<LQ>(dst);
  }
  template <int LQ>
  __device__ __forceinline__ void finish_impl(void *dst) {
    using namespace cudadma_b200::detail;
    if (STAGED) {
      /* all DMA threads of the object take the same branches: the tests are on the two pointers only */
      if (DO_SYNC) wait_for_dma_start_for_stores();
      else if (!m_is_dma_thread) return;
      if (m_staged) {
        staged_store<STAGED ? BYTES_PER_ELMT : 16, 1, NT>(m_stage, static_cast<char *>(dst), 0, m_dma_tid,
                                                          TRUST || (addr_bits(dst) & 15) == 0);
      } else if (!TRUST && m_is_dma_thread) {
        StridedRows a = {m_src, static_cast<char *>(dst), 0, 0};
        generic_rows(a, 1, m_bytes, copy_unit(addr_bits(m_src) | addr_bits(dst) | (unsigned long long)m_bytes), m_dma_tid,
                     m_num_dma_threads);
      }
      if (DO_SYNC) finish_async_dma();
      return;
    }
    if (DO_SYNC) wait_for_dma_start();
    else if (!m_is_dma_thread) return;
    const int pending = m_gave_up ? 0 : issue_contiguous<DO_SYNC, LQ>(m_src, static_cast<char *>(dst), m_bytes, m_dma_tid,
                                                                      m_num_dma_threads, m_bar_full);
    complete<DO_SYNC>(pending, m_bar_full);
  }
  const int m_bytes;
  const char *m_src;
  uint4 m_stage[Shape::UNITS > 0 ? Shape::UNITS : 1];
  bool m_staged;
};

/* Host-side description of what a parameter set turns into on this
 * implementation (the reference's diagnose(), cudaDMAv2.h:1402-1458, reports
 * load/store steps; here the interesting facts are the copy mechanism). */
template <bool DO_SYNC>
class CudaDMASequential<DO_SYNC, 0, 0, 0, 0> {
 public:
  __host__ static void diagnose(const int ALIGNMENT, const int BYTES_PER_THREAD, const int BYTES_PER_ELMT,
                                const int DMA_THREADS, const bool FULL_TEMPLATE, const bool verbose = false) {
    const bool bulk = (ALIGNMENT == 16) && (BYTES_PER_ELMT >= CUDADMA_BULK_ROW_MIN);
    const int warps = (DMA_THREADS + 31) / 32;
    fprintf(stdout, "CudaDMASequential on sm_100a: ALIGNMENT %d BYTES_PER_ELMT %d DMA_THREADS %d (%s)\n", ALIGNMENT,
            BYTES_PER_ELMT, DMA_THREADS, FULL_TEMPLATE ? "fully templated" : "runtime sized");
    const int budget = BYTES_PER_THREAD < 64 ? 64 : (BYTES_PER_THREAD > CUDADMA_STAGED_SEQUENTIAL_MAX ? CUDADMA_STAGED_SEQUENTIAL_MAX : BYTES_PER_THREAD);
    const bool staged = FULL_TEMPLATE && (BYTES_PER_ELMT % 16 == 0) && DMA_THREADS > 0 &&
                        (BYTES_PER_ELMT <= budget * DMA_THREADS);
    if (staged)
      fprintf(stdout, "  warp-specialised: staged through registers, %d 16-byte loads per DMA thread before the wait, "
                      "stores after it (small transfer)\n", (BYTES_PER_ELMT / 16 + DMA_THREADS - 1) / DMA_THREADS);
    else if (bulk)
      fprintf(stdout, "  warp-specialised: %d bulk copies (cp.async.bulk) of up to %d bytes, tail %d bytes via registers\n",
              warps, ((BYTES_PER_ELMT & ~15) + warps - 1) / (warps > 0 ? warps : 1), BYTES_PER_ELMT & 15);
    else
      fprintf(stdout, "  warp-specialised: per-thread cp.async of %d bytes (pointers not known to be 16-byte aligned)\n",
              ALIGNMENT);
    fprintf(stdout, "  non-specialised : per-thread cp.async, %d copies per thread\n",
            DMA_THREADS > 0 ? (BYTES_PER_ELMT / ALIGNMENT + DMA_THREADS - 1) / DMA_THREADS : 0);
    if (verbose) fprintf(stdout, "  BYTES_PER_THREAD %d: register staging up to %d bytes per DMA thread\n", BYTES_PER_THREAD, budget);
    fflush(stdout);
  }
};

/* ------------------------------------------------------------------------- */
/* CudaDMAStrided: NUM_ELMTS rows of BYTES_PER_ELMT bytes, independent source */
/* and destination row strides in bytes (cudaDMAv2.h:3193-3195).              */
/* Constructor forms (s = one stride, used for source and destination alike,  */
/* cudaDMAv2.h:5110-5127; s,d = source and destination stride):               */
/*   ws  L1 (dmaID, ndma, ncomp, start, elmt_bytes, num_elmts, s | s, d)      */
/*   ws  L2 (dmaID, ndma, ncomp, start, num_elmts, s | s, d)                  */
/*   ws  L3 (dmaID, ncomp, start, num_elmts, s | s, d)                        */
/*   ws  L4 (dmaID, ncomp, start, s | s, d)                                   */
/*   nws L1 (elmt_bytes, num_elmts, s) | (elmt_bytes, num_elmts, s, d, ndma = 0, start = 0) */
/*   nws L2 (num_elmts, s) | (num_elmts, s, d, ndma = 0, start = 0)           */
/*   nws L3 (num_elmts, s) | (num_elmts, s, d, start = 0)                     */
/*   nws L4 (s) | (s, d, start = 0)                                           */
/* (cudaDMAv2.h:5110-5144, :6300-6331, :7482-7510, :8610-8635, :5556-5585,     */
/*  :6731-6757, :7880-7904, :8993-9014).                                      */
/* ------------------------------------------------------------------------- */
template <bool DO_SYNC = false, int ALIGNMENT = 0, int BYTES_PER_THREAD = 4 * ALIGNMENT, int BYTES_PER_ELMT = 0,
          int DMA_THREADS = 0, int NUM_ELMTS = 0>
class CudaDMAStrided : public CudaDMA {
  static_assert(ALIGNMENT == 4 || ALIGNMENT == 8 || ALIGNMENT == 16, "ALIGNMENT must be 4, 8 or 16");
  static_assert((BYTES_PER_THREAD / ALIGNMENT) > 0 && (BYTES_PER_THREAD % ALIGNMENT) == 0,
                "BYTES_PER_THREAD must be a positive multiple of ALIGNMENT");
  static constexpr int LEVEL = (BYTES_PER_ELMT == 0) ? 1 : ((DMA_THREADS == 0) ? 2 : ((NUM_ELMTS == 0) ? 3 : 4));
  struct Params { int dmaID, ndma, ncomp, start, bytes, rows, sstride, dstride; };
  /* one_stride_packs: the one-stride forms leave the destination packed (rows BYTES_PER_ELMT apart),
   * which is what they mean in the v1 header (cudaDMA.h:1812-1840, "dst_stride == BYTES_PER_ELMT");
   * in the v2 header the one stride serves both sides (cudaDMAv2.h:5110-5127). */
  __device__ __forceinline__ static Params decode(const cudadma_b200::detail::ArgList &l, const bool one_stride_packs = false) {
    const int *a = l.v;
    const int n = l.n;
    Params p;
    if (DO_SYNC) {
      /* leading sync arguments, then the shape arguments, then one or two strides */
      int k;
      if (LEVEL <= 2) { p.dmaID = a[0]; p.ndma = a[1]; p.ncomp = a[2]; p.start = a[3]; k = 4; }
      else { p.dmaID = a[0]; p.ndma = DMA_THREADS; p.ncomp = a[1]; p.start = a[2]; k = 3; }
      if (LEVEL == 1) { p.bytes = a[k]; p.rows = a[k + 1]; k += 2; }
      else if (LEVEL <= 3) { p.bytes = BYTES_PER_ELMT; p.rows = a[k]; k += 1; }
      else { p.bytes = BYTES_PER_ELMT; p.rows = NUM_ELMTS; }
      p.sstride = a[k];
      p.dstride = (n - k >= 2) ? a[k + 1] : (one_stride_packs ? p.bytes : p.sstride);
    } else {
      int k = 0;
      if (LEVEL == 1) { p.bytes = a[0]; p.rows = a[1]; k = 2; }
      else if (LEVEL <= 3) { p.bytes = BYTES_PER_ELMT; p.rows = a[0]; k = 1; }
      else { p.bytes = BYTES_PER_ELMT; p.rows = NUM_ELMTS; }
      p.sstride = a[k];
      const bool two = (n - k >= 2);
      p.dstride = two ? a[k + 1] : (one_stride_packs ? p.bytes : p.sstride);
      int nd = DMA_THREADS, st = 0;
      if (two) {
        if (LEVEL <= 2) { nd = a[k + 2]; st = a[k + 3]; }
        else { st = a[k + 2]; }
      }
      if (nd <= 0) nd = blockDim.x;
      p.dmaID = 0; p.ndma = nd; p.ncomp = nd; p.start = st;
    }
    return p;
  }
  /* Small, fully templated tiles are staged through registers like small CudaDMASequential
   * transfers (see detail::staged_load): at most BYTES_PER_THREAD bytes per DMA thread, which is
   * what that parameter bounds in the reference too, and never more than 128. Such an object issues
   * no asynchronous copy, so its handshake can use the hardware barriers (see class CudaDMA). */
  static constexpr int NT = DMA_THREADS > 0 ? DMA_THREADS : 1;
  typedef cudadma_b200::detail::StagedShape<(LEVEL == 4 && BYTES_PER_ELMT % 16 == 0) ? BYTES_PER_ELMT : 16,
                                            LEVEL == 4 ? NUM_ELMTS : 1, NT> Shape;
#if defined(CUDADMA_NO_REGISTER_STAGING) || defined(CUDADMA_CHECKED)
  static constexpr bool STAGED = false;
#else
  static constexpr bool STAGED = LEVEL == 4 && BYTES_PER_ELMT % 16 == 0 &&
                                 16 * Shape::UNITS <= (BYTES_PER_THREAD < 128 ? BYTES_PER_THREAD : 128);
#endif
  static constexpr int SB = STAGED ? BYTES_PER_ELMT : 16, SR = STAGED ? NUM_ELMTS : 1; /* staged shape */
  static constexpr bool TRUST = ALIGNMENT == 16; /* pointers and strides are what the template argument says */
  __device__ __forceinline__ CudaDMAStrided(const Params &p, int)
      : CudaDMA(p.dmaID, p.ndma, p.ncomp, p.start, DO_SYNC, !STAGED, STAGED && NT <= CUDADMA_NAMED_MAX_DMA_THREADS), m_bytes(p.bytes), m_rows(p.rows),
        m_src_stride(p.sstride), m_dst_stride(p.dstride), m_src(0), m_staged(false) {}

 public:
  template <typename... I>
  __device__ __forceinline__ CudaDMAStrided(I... args)
      : CudaDMAStrided(decode(cudadma_b200::detail::make_args(args...)), 0) {
    static_assert(sizeof...(I) >= 1, "a stride argument is required");
  }
  /* the v1 spelling's constructor (see cudaDMAStrided at the end of this file) */
  template <typename... I>
  __device__ __forceinline__ CudaDMAStrided(cudadma_b200::detail::V1Forms, I... args)
      : CudaDMAStrided(decode(cudadma_b200::detail::make_args(args...), true), 0) {
    static_assert(sizeof...(I) >= 1, "a stride argument is required");
  }
  CUDADMA_B200_XFER_OVERLOADS(const void *__restrict__ src_ptr, src_ptr)

  /* Extension: tile load through a host-encoded 2-D tensor map. The map's
   * box must be m_rows rows tall; `nboxes` boxes of `box_cols` columns each,
   * side by side in x, land one after another at dst (each `box_bytes`
   * long, the map's swizzle decides the layout inside a box). dst must be
   * 128-byte aligned (1024 for the 128-byte swizzle) and x * element size a
   * multiple of 16. Warp-specialised objects only. */
  __device__ __forceinline__ void execute_dma_tensor(const CUtensorMap *map, const int x, const int y, void *dst,
                                                     const int nboxes, const int box_cols,
                                                     const uint32_t box_bytes) {
    static_assert(DO_SYNC, "tensor-map transfers need a warp-specialised object");
    static_assert(!STAGED, "this instantiation is small enough to be staged through registers and has no mbarrier "
                           "for a tensor-map transfer to count on; build with -DCUDADMA_NO_REGISTER_STAGING");
    wait_for_dma_start();
    if (m_dma_tid == 0 && !m_gave_up) {
      cudadma_b200::ptx::mbar_expect_tx(m_bar_full, box_bytes * (uint32_t)nboxes);
      const uint32_t d = cudadma_b200::ptx::smem_u32(dst);
      for (int b = 0; b < nboxes; ++b)
        cudadma_b200::ptx::tensor_g2s_2d(d + (uint32_t)b * box_bytes, map, x + b * box_cols, y, m_bar_full);
    }
    finish_async_dma();
  }

 private:
  template <bool GLOBAL, int LQ>
  __device__ __forceinline__ void start_impl(const void *src) {
    m_src = static_cast<const char *>(src);
    if (STAGED) {
      m_staged = m_is_dma_thread &&
                 (TRUST || ((cudadma_b200::detail::addr_bits(src) | (unsigned long long)(unsigned)m_src_stride) & 15) == 0);
      if (m_staged)
        cudadma_b200::detail::staged_load<SB, SR, NT, GLOBAL && LQ != LOAD_CACHE_ALL, GLOBAL>(m_stage, m_src, m_src_stride, m_dma_tid);
      return;
    }
    if (DO_SYNC)
      cudadma_b200::detail::prefetch_small(m_src, m_rows, m_bytes, m_src_stride, m_dma_tid, m_num_dma_threads);
  }
  /* execute_dma in one call; a staged object keeps the bytes in a local array (see CudaDMASequential) */
  template <bool GLOBAL, int LQ>
  __device__ __forceinline__ void execute_impl(const void *src, void *dst) {
    using namespace cudadma_b200::detail;
    if (STAGED) {
      const char *s = static_cast<const char *>(src);
      const bool early = (DO_SYNC || m_is_dma_thread) &&
                         (TRUST || ((addr_bits(src) | (unsigned long long)(unsigned)m_src_stride) & 15) == 0);
      uint4 stage[STAGED ? Shape::UNITS : 1];
      if (early) staged_load<SB, SR, NT, GLOBAL && LQ != LOAD_CACHE_ALL, GLOBAL>(stage, s, m_src_stride, m_dma_tid);
      if (DO_SYNC) wait_for_dma_start_for_stores();
      else if (!m_is_dma_thread) return;
      const unsigned long long dmask = addr_bits(dst) | (unsigned long long)(unsigned)m_dst_stride;
      if (early) {
        staged_store<SB, SR, NT>(stage, static_cast<char *>(dst), m_dst_stride, m_dma_tid, TRUST || (dmask & 15) == 0);
      } else if (!TRUST && m_is_dma_thread) {
        StridedRows a = {s, static_cast<char *>(dst), m_src_stride, m_dst_stride};
        generic_rows(a, m_rows, m_bytes,
                     copy_unit(dmask | addr_bits(s) | (unsigned long long)(unsigned)m_src_stride | (unsigned long long)m_bytes),
                     m_dma_tid, m_num_dma_threads);
      }
      if (DO_SYNC) finish_async_dma();
      return;
    }
    start_impl<GLOBAL, LQ>(src);
    finish_impl<LQ>(dst);
  }
  template <int LQ>
  __device__ __forceinline__ void finish_impl(void *dst) {
    using namespace cudadma_b200::detail;
    if (STAGED) {
      if (DO_SYNC) wait_for_dma_start_for_stores();
      else if (!m_is_dma_thread) return;
      const unsigned long long dmask = addr_bits(dst) | (unsigned long long)(unsigned)m_dst_stride;
      if (m_staged) {
        staged_store<SB, SR, NT>(m_stage, static_cast<char *>(dst), m_dst_stride, m_dma_tid, TRUST || (dmask & 15) == 0);
      } else if (!TRUST && m_is_dma_thread) {
        StridedRows a = {m_src, static_cast<char *>(dst), m_src_stride, m_dst_stride};
        generic_rows(a, m_rows, m_bytes,
                     copy_unit(dmask | addr_bits(m_src) | (unsigned long long)(unsigned)m_src_stride |
                               (unsigned long long)m_bytes),
                     m_dma_tid, m_num_dma_threads);
      }
      if (DO_SYNC) finish_async_dma();
      return;
    }
    if (DO_SYNC) wait_for_dma_start();
    else if (!m_is_dma_thread) return;
    int pending = 0;
    if (m_gave_up) {
      /* nothing is issued after a failed wait */
    } else if (m_src_stride == m_bytes && m_dst_stride == m_bytes) {
      pending = issue_contiguous<DO_SYNC, LQ>(m_src, static_cast<char *>(dst), m_bytes * m_rows, m_dma_tid,
                                              m_num_dma_threads, m_bar_full);
    } else {
      StridedRows a = {m_src, static_cast<char *>(dst), m_src_stride, m_dst_stride};
      const unsigned long long mask = addr_bits(m_src) | addr_bits(dst) | (unsigned long long)m_bytes |
                                      (unsigned long long)(unsigned)m_src_stride |
                                      (unsigned long long)(unsigned)m_dst_stride;
      pending = issue_rows<DO_SYNC, LQ>(a, m_rows, m_bytes, mask, m_dma_tid, m_num_dma_threads, m_bar_full);
    }
    complete<DO_SYNC>(pending, m_bar_full);
  }
  const int m_bytes;
  const int m_rows;
  const int m_src_stride;
  const int m_dst_stride;
  const char *m_src;
  uint4 m_stage[STAGED ? Shape::UNITS : 1];
  bool m_staged;
};

template <bool DO_SYNC>
class CudaDMAStrided<DO_SYNC, 0, 0, 0, 0, 0> {
 public:
  __host__ static void diagnose(const int ALIGNMENT, const int BYTES_PER_THREAD, const int BYTES_PER_ELMT,
                                const int DMA_THREADS, const int NUM_ELMTS, const bool FULL_TEMPLATE,
                                const bool verbose = false) {
    const bool bulk = (ALIGNMENT == 16) && (BYTES_PER_ELMT % 16 == 0) && (BYTES_PER_ELMT >= CUDADMA_BULK_ROW_MIN);
    fprintf(stdout, "CudaDMAStrided on sm_100a: ALIGNMENT %d BYTES_PER_ELMT %d NUM_ELMTS %d DMA_THREADS %d (%s)\n",
            ALIGNMENT, BYTES_PER_ELMT, NUM_ELMTS, DMA_THREADS, FULL_TEMPLATE ? "fully templated" : "runtime sized");
    if (bulk)
      fprintf(stdout, "  warp-specialised: one bulk copy per row, %d rows per DMA thread at most (strides must be multiples of 16)\n",
              DMA_THREADS > 0 ? (NUM_ELMTS + DMA_THREADS - 1) / DMA_THREADS : 0);
    else
      fprintf(stdout, "  warp-specialised: per-thread cp.async of %d bytes\n",
              (BYTES_PER_ELMT % ALIGNMENT == 0) ? ALIGNMENT : 4);
    fprintf(stdout, "  tensor-map path : execute_dma_tensor(), one TMA box of %d x %d bytes\n", NUM_ELMTS, BYTES_PER_ELMT);
    if (verbose) fprintf(stdout, "  BYTES_PER_THREAD %d is not used: no register staging\n", BYTES_PER_THREAD);
    fflush(stdout);
  }
};

/* ------------------------------------------------------------------------- */
/* CudaDMAIndirect: gather (rows at src + index[i] * BYTES_PER_ELMT, packed   */
/* destination) or scatter (packed source, rows land at dst + index[i] *      */
/* BYTES_PER_ELMT); the packed side's pitch is max(alternate_stride,          */
/* BYTES_PER_ELMT) (cudaDMAv2.h:9381-9383, :9406, :13618-13619, :14021-14025). */
/* Index arithmetic is 64-bit here (the reference multiplies in 32 bits).     */
/* Constructor forms (cudaDMAv2.h:10225-10231, :11431-11436, :12710-12714,     */
/* :13983-13986, :10628-10632, :11825-11828, :13098-13100, :14362-14363):      */
/*   ws  L1 (dmaID, ndma, ncomp, start, elmt_bytes, num_elmts, alt = 0)       */
/*   ws  L2 (dmaID, ndma, ncomp, start, num_elmts, alt = 0)                   */
/*   ws  L3 (dmaID, ncomp, start, num_elmts, alt = 0)                         */
/*   ws  L4 (dmaID, ncomp, start, alt = 0)                                    */
/*   nws L1 (elmt_bytes, num_elmts, alt = 0, ndma = 0, start = 0)             */
/*   nws L2 (num_elmts, alt = 0, ndma = 0, start = 0)                         */
/*   nws L3 (num_elmts, alt = 0, start = 0)                                   */
/*   nws L4 (alt = 0, start = 0)                                              */
/* ------------------------------------------------------------------------- */
template <bool GATHER = true, bool DO_SYNC = false, int ALIGNMENT = 0, int BYTES_PER_THREAD = 4 * ALIGNMENT,
          int BYTES_PER_ELMT = 0, int DMA_THREADS = 0, int NUM_ELMTS = 0>
class CudaDMAIndirect : public CudaDMA {
  static_assert(ALIGNMENT == 4 || ALIGNMENT == 8 || ALIGNMENT == 16, "ALIGNMENT must be 4, 8 or 16");
  static_assert((BYTES_PER_THREAD / ALIGNMENT) > 0 && (BYTES_PER_THREAD % ALIGNMENT) == 0,
                "BYTES_PER_THREAD must be a positive multiple of ALIGNMENT");
  static constexpr int LEVEL = (BYTES_PER_ELMT == 0) ? 1 : ((DMA_THREADS == 0) ? 2 : ((NUM_ELMTS == 0) ? 3 : 4));
  struct Params { int dmaID, ndma, ncomp, start, bytes, rows, alt; };
  __device__ __forceinline__ static Params decode(const cudadma_b200::detail::ArgList &l) {
    const int *a = l.v;
    Params p;
    int k;
    if (DO_SYNC) {
      if (LEVEL <= 2) { p.dmaID = a[0]; p.ndma = a[1]; p.ncomp = a[2]; p.start = a[3]; k = 4; }
      else { p.dmaID = a[0]; p.ndma = DMA_THREADS; p.ncomp = a[1]; p.start = a[2]; k = 3; }
    } else {
      k = 0;
    }
    if (LEVEL == 1) { p.bytes = a[k]; p.rows = a[k + 1]; k += 2; }
    else if (LEVEL <= 3) { p.bytes = BYTES_PER_ELMT; p.rows = a[k]; k += 1; }
    else { p.bytes = BYTES_PER_ELMT; p.rows = NUM_ELMTS; }
    p.alt = a[k];
    if (!DO_SYNC) {
      int nd = DMA_THREADS, st;
      if (LEVEL <= 2) { nd = a[k + 1]; st = a[k + 2]; }
      else { st = a[k + 1]; }
      if (nd <= 0) nd = blockDim.x;
      p.dmaID = 0; p.ndma = nd; p.ncomp = nd; p.start = st;
    }
    return p;
  }
  /* records shorter than the smallest bulk copy never meet the bulk-copy engine */
#ifdef CUDADMA_ALWAYS_FENCE
  static constexpr bool MAY_BULK = true;
#else
  static constexpr bool MAY_BULK = !(BYTES_PER_ELMT > 0 && BYTES_PER_ELMT < CUDADMA_BULK_ROW_MIN);
#endif
  __device__ __forceinline__ CudaDMAIndirect(const Params &p, int)
      : CudaDMA(p.dmaID, p.ndma, p.ncomp, p.start, DO_SYNC, MAY_BULK), m_bytes(p.bytes), m_rows(p.rows),
        m_pitch(p.alt > p.bytes ? p.alt : p.bytes), m_index(0), m_src(0) {}

 public:
  template <typename... I>
  __device__ __forceinline__ CudaDMAIndirect(I... args)
      : CudaDMAIndirect(decode(cudadma_b200::detail::make_args(args...)), 0) {}
#define CUDADMA_B200_COMMA ,
  CUDADMA_B200_XFER_OVERLOADS(const int *__restrict__ index_ptr CUDADMA_B200_COMMA const void *__restrict__ src_ptr,
                              index_ptr CUDADMA_B200_COMMA src_ptr)
#undef CUDADMA_B200_COMMA

  /* Extension (gather only): TMA row gather. `map` describes the table as a
   * 2-D tensor [table rows][row elements] whose box is one row wide; four
   * table rows are fetched per instruction. Needs m_rows % 4 == 0, the index
   * array 16-byte aligned and dst 128-byte aligned; rows land packed. */
  __device__ __forceinline__ void execute_dma_gather4(const CUtensorMap *map, const int *__restrict__ index_ptr,
                                                      void *dst) {
    static_assert(DO_SYNC && GATHER, "gather4 needs a warp-specialised gather object");
    wait_for_dma_start();
    if (!MAY_BULK) cudadma_b200::ptx::fence_proxy_async();
    const int groups = m_rows >> 2;
    const int mine = (groups > m_dma_tid && !m_gave_up) ? (groups - m_dma_tid + m_num_dma_threads - 1) / m_num_dma_threads : 0;
    if (mine > 0) {
      cudadma_b200::ptx::mbar_expect_tx(m_bar_full, (uint32_t)mine * 4u * (uint32_t)m_bytes);
      const uint32_t d = cudadma_b200::ptx::smem_u32(dst);
      for (int g = m_dma_tid; g < groups; g += m_num_dma_threads) {
        const int4 ix = __ldg(reinterpret_cast<const int4 *>(index_ptr) + g);
        cudadma_b200::ptx::tensor_gather4(d + (uint32_t)g * 4u * (uint32_t)m_bytes, map, 0, ix.x, ix.y, ix.z, ix.w,
                                          m_bar_full);
      }
    }
    finish_async_dma();
  }

  /* Extension (scatter only): TMA row scatter. `map` describes the destination as a 2-D tensor
   * [destination rows][row elements] whose box is one row wide; four packed rows of the shared
   * buffer leave per instruction. Needs m_rows % 4 == 0, the index array 16-byte aligned and
   * src 128-byte aligned, rows packed. Returns once the buffer has been read. */
  __device__ __forceinline__ void execute_dma_scatter4(const CUtensorMap *map, const int *__restrict__ index_ptr,
                                                       const void *src) {
    static_assert(DO_SYNC && !GATHER, "scatter4 needs a warp-specialised scatter object");
    wait_for_dma_start();
    if (!MAY_BULK) cudadma_b200::ptx::fence_proxy_async(); /* the rows were written by ordinary or cp.async stores */
    const int groups = m_rows >> 2;
    const uint32_t s0 = cudadma_b200::ptx::smem_u32(src);
    for (int g = m_gave_up ? groups : m_dma_tid; g < groups; g += m_num_dma_threads) {
      const int4 ix = __ldg(reinterpret_cast<const int4 *>(index_ptr) + g);
      cudadma_b200::ptx::tensor_scatter4(map, 0, ix.x, ix.y, ix.z, ix.w, s0 + (uint32_t)g * 4u * (uint32_t)m_bytes);
    }
    cudadma_b200::ptx::bulk_commit();
    cudadma_b200::ptx::bulk_wait_read<0>();
    finish_async_dma();
  }

 private:
  template <bool GLOBAL, int LQ>
  __device__ __forceinline__ void start_impl(const int *index, const void *src) {
    m_index = index;
    m_src = static_cast<const char *>(src);
  }
  template <bool GLOBAL, int LQ>
  __device__ __forceinline__ void execute_impl(const int *index, const void *src, void *dst) {
    start_impl<GLOBAL, LQ>(index, src);
    finish_impl<LQ>(dst);
  }
  template <int LQ>
  __device__ __forceinline__ void finish_impl(void *dst) {
    using namespace cudadma_b200::detail;
    if (DO_SYNC) wait_for_dma_start();
    else if (!m_is_dma_thread) return;
    const unsigned long long mask = addr_bits(m_src) | addr_bits(dst) | (unsigned long long)m_bytes |
                                    (unsigned long long)m_pitch;
    int pending = 0;
    if (m_gave_up) {
      /* nothing is issued after a failed wait */
    } else if (GATHER) {
      GatherRows a = {m_src, static_cast<char *>(dst), m_index, m_bytes, m_pitch};
      pending = issue_rows<DO_SYNC, LQ>(a, m_rows, m_bytes, mask, m_dma_tid, m_num_dma_threads, m_bar_full);
    } else {
      ScatterRows a = {m_src, static_cast<char *>(dst), m_index, m_bytes, m_pitch};
      pending = issue_rows<DO_SYNC, LQ>(a, m_rows, m_bytes, mask, m_dma_tid, m_num_dma_threads, m_bar_full);
    }
    complete<DO_SYNC>(pending, m_bar_full);
  }
  const int m_bytes;
  const int m_rows;
  const int m_pitch;
  const int *m_index;
  const char *m_src;
};

template <bool GATHER, bool DO_SYNC>
class CudaDMAIndirect<GATHER, DO_SYNC, 0, 0, 0, 0, 0> {
 public:
  __host__ static void diagnose(const int ALIGNMENT, const int BYTES_PER_THREAD, const int BYTES_PER_ELMT,
                                const int DMA_THREADS, const int NUM_ELMTS, const bool FULL_TEMPLATE,
                                const bool verbose = false) {
    const bool a16 = (ALIGNMENT == 16) && (BYTES_PER_ELMT % 16 == 0);
    fprintf(stdout, "CudaDMAIndirect (%s) on sm_100a: ALIGNMENT %d BYTES_PER_ELMT %d NUM_ELMTS %d DMA_THREADS %d (%s)\n",
            GATHER ? "gather" : "scatter", ALIGNMENT, BYTES_PER_ELMT, NUM_ELMTS, DMA_THREADS,
            FULL_TEMPLATE ? "fully templated" : "runtime sized");
    if (GATHER) {
      if (a16 && BYTES_PER_ELMT >= CUDADMA_BULK_ROW_MIN) fprintf(stdout, "  warp-specialised: one bulk copy per record\n");
      else fprintf(stdout, "  warp-specialised: %d-byte cp.async, %d per record\n", a16 ? 16 : ((BYTES_PER_ELMT % ALIGNMENT) ? 4 : ALIGNMENT),
                   BYTES_PER_ELMT / (a16 ? 16 : ((BYTES_PER_ELMT % ALIGNMENT) ? 4 : ALIGNMENT)));
      if (a16 && NUM_ELMTS % 4 == 0) fprintf(stdout, "  gather4 path    : execute_dma_gather4(), %d TMA row gathers per buffer\n", NUM_ELMTS / 4);
    } else {
      if (a16) fprintf(stdout, "  one bulk store (cp.async.bulk shared->global) per record\n");
      else fprintf(stdout, "  register copies of %d bytes\n", (BYTES_PER_ELMT % ALIGNMENT) ? 4 : ALIGNMENT);
    }
    if (verbose) fprintf(stdout, "  BYTES_PER_THREAD %d is not used: no register staging\n", BYTES_PER_THREAD);
    fflush(stdout);
  }
};

/* ------------------------------------------------------------------------- */
/* CudaDMAHalo: the ring around a dimx x dimy tile -- RADIUS rows above and   */
/* below (dimx wide, dimx + 2*RADIUS with CORNERS) and RADIUS-wide panels on  */
/* either side -- from an array of row pitch `pitch` elements into a buffer   */
/* of row pitch dimx + 2*RADIUS elements. Both pointers address the interior  */
/* origin. Constructor and calls follow the v1 class, cudaDMA.h:3686-3692,    */
/* :3853-3860; ring geometry cudaDMA.h:3616-3649, :3718-3727.                 */
/* execute_dma_tile() is the tensor-map form: whole tile, ring and interior,  */
/* in one TMA box with zero fill outside the array.                           */
/* ------------------------------------------------------------------------- */
template <typename ELMT_TYPE, int RADIUS, bool CORNERS, int ALIGNMENT>
class CudaDMAHalo : public CudaDMA {
  struct RingRows {   /* item i: rows above (i < RADIUS) then rows below */
    static constexpr bool SCATTERED_SOURCE = false;
    const char *src; char *dst; int dimy; long long spitch, dpitch;
    __device__ __forceinline__ long long row(int i) const { return (i < RADIUS) ? (i - RADIUS) : (dimy + i - RADIUS); }
    __device__ __forceinline__ const char *src_row(int i) const { return src + row(i) * spitch; }
    __device__ __forceinline__ char *dst_row(int i) const { return dst + row(i) * dpitch; }
  };
  struct RingSides {  /* item i: row i/2, left panel (even) or right panel (odd) */
    static constexpr bool SCATTERED_SOURCE = false;
    const char *src; char *dst; long long right; long long spitch, dpitch;
    __device__ __forceinline__ const char *src_row(int i) const { return src + (i >> 1) * spitch + ((i & 1) ? right : 0); }
    __device__ __forceinline__ char *dst_row(int i) const { return dst + (i >> 1) * dpitch + ((i & 1) ? right : 0); }
  };

 public:
  __device__ __forceinline__ CudaDMAHalo(const int dmaID, const int num_dma_threads, const int num_compute_threads,
                                         const int dma_threadIdx_start, const int dimx, const int dimy,
                                         const int pitch)
      : CudaDMA(dmaID, num_dma_threads, num_compute_threads, dma_threadIdx_start, true),
        m_dimx(dimx), m_dimy(dimy), m_pitch(pitch) {}

  __device__ __forceinline__ void execute_dma(const void *__restrict__ src_origin, void *__restrict__ dst_origin) const {
    wait_for_dma_start();
    const int pending = m_gave_up ? 0 : issue_ring<true>(src_origin, dst_origin);
    cudadma_b200::detail::complete<true>(pending, m_bar_full);
  }
  /* same copy without either barrier; the data is in place when the call returns */
  __device__ __forceinline__ void execute_dma_no_sync(const void *__restrict__ src_origin,
                                                      void *__restrict__ dst_origin) const {
    const int pending = issue_ring<false>(src_origin, dst_origin);
    cudadma_b200::detail::complete<false>(pending, m_bar_full);
  }
  /* Tensor-map form: the (dimx + 2R) x (dimy + 2R) tile whose interior origin
   * is element (x0, y0) of plane z, one TMA box, zero outside the tensor.
   * `tile` is the start of the buffer (not the interior origin), 128-byte
   * aligned; (x0 - RADIUS) * sizeof(ELMT_TYPE) must be a multiple of 16. */
  __device__ __forceinline__ void execute_dma_tile(const CUtensorMap *map, const int x0, const int y0, const int z,
                                                   void *tile) const {
    wait_for_dma_start();
    if (m_dma_tid == 0 && !m_gave_up) {
      cudadma_b200::ptx::mbar_expect_tx(
          m_bar_full, (uint32_t)((m_dimx + 2 * RADIUS) * (m_dimy + 2 * RADIUS)) * (uint32_t)sizeof(ELMT_TYPE));
      cudadma_b200::ptx::tensor_g2s_3d(cudadma_b200::ptx::smem_u32(tile), map, x0 - RADIUS, y0 - RADIUS, z,
                                       m_bar_full);
    }
    finish_async_dma();
  }

 private:
  template <bool WS>
  __device__ __forceinline__ int issue_ring(const void *src_origin, void *dst_origin) const {
    using namespace cudadma_b200::detail;
    const long long sz = (long long)sizeof(ELMT_TYPE);
    const long long spitch = (long long)m_pitch * sz, dpitch = (long long)(m_dimx + 2 * RADIUS) * sz;
    const long long lead = CORNERS ? (long long)RADIUS * sz : 0;
    const int row_bytes = (m_dimx + (CORNERS ? 2 * RADIUS : 0)) * (int)sz;
    const int side_bytes = RADIUS * (int)sz;
    const char *s = static_cast<const char *>(src_origin);
    char *d = static_cast<char *>(dst_origin);
    const unsigned long long strides = (unsigned long long)spitch | (unsigned long long)dpitch;
    RingRows rows = {s - lead, d - lead, m_dimy, spitch, dpitch};
    int pending = issue_rows<WS, LOAD_CACHE_ALL>(
        rows, 2 * RADIUS, row_bytes,
        addr_bits(rows.src) | addr_bits(rows.dst) | strides | (unsigned long long)row_bytes, m_dma_tid,
        m_num_dma_threads, m_bar_full);
    RingSides sides = {s - side_bytes, d - side_bytes, (long long)side_bytes + (long long)m_dimx * sz, spitch, dpitch};
    pending |= issue_rows<WS, LOAD_CACHE_ALL>(
        sides, 2 * m_dimy, side_bytes,
        addr_bits(sides.src) | addr_bits(sides.dst) | strides | (unsigned long long)side_bytes |
            (unsigned long long)sides.right,
        m_dma_tid, m_num_dma_threads, m_bar_full);
    return pending;
  }
  const int m_dimx, m_dimy, m_pitch;
};
template <typename ELMT_TYPE, int RADIUS, bool CORNERS, int ALIGNMENT>
using cudaDMAHalo = CudaDMAHalo<ELMT_TYPE, RADIUS, CORNERS, ALIGNMENT>;

/* ------------------------------------------------------------------------- */
/* CudaDMACustom: only the handshake, for hand-written copy loops             */
/* (v1 cudaDMACustom, cudaDMA.h:4184-4208). The caller's loop fills the buffer */
/* with ordinary stores, so the handshake is a pair of hardware barriers where */
/* dmaID and thread counts allow it (see class CudaDMA). A caller that fills   */
/* the buffer with asynchronous copies of its own must wait for them before    */
/* finish_async_dma().                                                         */
/* ------------------------------------------------------------------------- */
class CudaDMACustom : public CudaDMA {
 public:
  __device__ __forceinline__ CudaDMACustom(const int dmaID, const int num_dma_threads, const int num_compute_threads,
                                           const int dma_threadIdx_start)
      : CudaDMA(dmaID, num_dma_threads, num_compute_threads, dma_threadIdx_start, true, false, true) {}
};
typedef CudaDMACustom cudaDMACustom;

/* ------------------------------------------------------------------------- */
/* v1 spellings (include/cudaDMA.h:644, :1977, :2891): the same classes        */
/* without the BYTES_PER_THREAD parameter. v1 moved 4 * ALIGNMENT bytes per     */
/* thread and pass, in as many passes as the transfer needed; this header       */
/* stages a transfer at once or not at all, so the v1 names get twice that       */
/* budget (128 bytes per DMA thread with ALIGNMENT 16): the reference's sgemv    */
/* example's matrix panels, 128 bytes per thread, run 1.7 x the reference header */
/* staged and 0.48 x through bulk copies. Constructor argument orders of the v1  */
/* forms are those of the v2 forms above (cudaDMA.h:651-653, :916-920,           */
/* :1037-1040, :1985-1996), so kernels written for v1 (the saxpy and sgemv       */
/* examples of the reference) name these and construct them as before.           */
/* ------------------------------------------------------------------------- */
#ifndef CUDADMA_V1_BYTES_PER_THREAD
#define CUDADMA_V1_BYTES_PER_THREAD(ALIGNMENT) (8 * (ALIGNMENT))
#endif
template <bool DO_SYNC, int ALIGNMENT, int BYTES_PER_ELMT = 0, int DMA_THREADS = 0>
using cudaDMASequential = CudaDMASequential<DO_SYNC, ALIGNMENT, CUDADMA_V1_BYTES_PER_THREAD(ALIGNMENT), BYTES_PER_ELMT, DMA_THREADS>;
/* cudaDMAStrided is a class of its own because one constructor form means something else in v1: with
 * ONE stride argument the destination rows are packed (BYTES_PER_ELMT apart, cudaDMA.h:1981,
 * :1812-1840), where the v2 class uses that stride on both sides. The reference's sgemv example
 * depends on it (src/examples/sgemv/sgemv_dma.cu:340-341: matrix panels with the matrix pitch as
 * their one stride, into a dense shared array). */
template <bool DO_SYNC, int ALIGNMENT, int BYTES_PER_ELMT = 0, int DMA_THREADS = 0, int NUM_ELMTS = 0>
class cudaDMAStrided : public CudaDMAStrided<DO_SYNC, ALIGNMENT, CUDADMA_V1_BYTES_PER_THREAD(ALIGNMENT), BYTES_PER_ELMT, DMA_THREADS, NUM_ELMTS> {
 public:
  template <typename... I>
  __device__ __forceinline__ cudaDMAStrided(I... args)
      : CudaDMAStrided<DO_SYNC, ALIGNMENT, CUDADMA_V1_BYTES_PER_THREAD(ALIGNMENT), BYTES_PER_ELMT, DMA_THREADS, NUM_ELMTS>(
            cudadma_b200::detail::V1Forms(), args...) {}
};
template <bool GATHER, bool DO_SYNC, int ALIGNMENT, int BYTES_PER_ELMT = 0, int DMA_THREADS = 0, int NUM_ELMTS = 0>
using cudaDMAIndirect = CudaDMAIndirect<GATHER, DO_SYNC, ALIGNMENT, CUDADMA_V1_BYTES_PER_THREAD(ALIGNMENT), BYTES_PER_ELMT, DMA_THREADS, NUM_ELMTS>;

#undef CUDADMA_B200_XFER_OVERLOADS
#endif /* CUDADMA_B200_CUDADMA_H */
