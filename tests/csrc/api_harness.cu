/*
 * api_harness.cu -- single-CTA test kernels for the CudaDMA object API.
 *
 * Every kernel follows the shape of the reference's own tests
 * (src/tests/test_sequential/cudaDMA_test_sequential_v2.cu:52-405,
 *  src/tests/test_strided/cudaDMA_test_strided_v2.cu:52-537,
 *  src/tests/test_indirect/cudaDMA_test_indirect_v2.cu:54-537,
 *  src/tests/test_halo/cudaDMA_test_halo.cu:180-231): the compute threads zero
 * a shared buffer, the object under test fills it, the compute threads copy
 * the whole buffer out, the host compares. What differs is that sizes the
 * template form leaves open are run-time arguments, so one binary serves a
 * randomised sweep.
 *
 * The file is written against the common object API and is built three times
 * with the same source:
 *   default                  "cudaDMAv2.h" resolves to this repository's header
 *   -DAPITEST_REFERENCE_V2   the reference's cudaDMAv2.h (Sequential/Strided/Indirect)
 *   -DAPITEST_REFERENCE_V1   the reference's cudaDMA.h   (halo only; the two
 *                            reference headers cannot share a translation unit)
 * Entry points are prefixed with APITEST_PREFIX. Return value: 0 ok, -1 bad
 * argument / shape not instantiated, -2 CUDA error, 1 device wait gave up.
 */
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#if defined(APITEST_REFERENCE_V1)
#include "cudaDMA.h"
#define HAVE_V2 0
#define HAVE_HALO 1
#elif defined(APITEST_REFERENCE_V2)
#include "cudaDMAv2.h"
#define HAVE_V2 1
#define HAVE_HALO 0
#else
#include "cudaDMAv2.h"
#define HAVE_V2 1
#define HAVE_HALO 1
#define HAVE_STATUS 1
#endif

#ifndef APITEST_PREFIX
#define APITEST_PREFIX apitest_
#endif
#define CAT2(a, b) a##b
#define CAT(a, b) CAT2(a, b)
#define ENTRY(name) CAT(APITEST_PREFIX, name)

#define BPT 64 /* BYTES_PER_THREAD used everywhere: a multiple of every ALIGNMENT */

namespace {

int finish() {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { fprintf(stderr, "apitest: %s\n", cudaGetErrorString(e)); return -2; }
#ifdef HAVE_STATUS
  unsigned int w = 0;
  if (cudadma_b200::read_status(&w, 0) != cudaSuccess) return -2;
  if (w) return 1;
#endif
  return 0;
}

/* device buffers for one experiment: input copied down, output zeroed */
struct Buffers {
  float *d_in = nullptr, *d_out = nullptr;
  int *d_idx = nullptr;
  size_t out_bytes = 0;
  int init(const float *h_in, size_t in_floats, size_t out_floats, const int *h_idx = nullptr, size_t nidx = 0) {
    out_bytes = out_floats * 4;
    if (cudaMalloc(&d_in, in_floats * 4 + 64) != cudaSuccess) return -2;
    if (cudaMalloc(&d_out, out_bytes + 64) != cudaSuccess) return -2;
    if (cudaMemcpy(d_in, h_in, in_floats * 4, cudaMemcpyHostToDevice) != cudaSuccess) return -2;
    if (cudaMemset(d_out, 0, out_bytes + 64) != cudaSuccess) return -2;
    if (h_idx) {
      if (cudaMalloc(&d_idx, nidx * 4 + 64) != cudaSuccess) return -2;
      if (cudaMemcpy(d_idx, h_idx, nidx * 4, cudaMemcpyHostToDevice) != cudaSuccess) return -2;
    }
    return 0;
  }
  int fetch(float *h_out) {
    int r = finish();
    if (r == 0 && cudaMemcpy(h_out, d_out, out_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) r = -2;
    return r;
  }
  ~Buffers() { cudaFree(d_in); cudaFree(d_out); cudaFree(d_idx); }
};

template <typename K>
int big_smem(K k, size_t bytes) {
  /* the header under test may add a little static shared memory of its own: opt in early */
  if (bytes > 40 * 1024 &&
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
    return -2;
  return 0;
}

__device__ __forceinline__ void zero_buffer(float *buffer, int n, int tid, int nthreads) {
  for (int i = tid; i < n; i += nthreads) buffer[i] = 0.0f;
}
__device__ __forceinline__ void copy_out(float *odata, const float *buffer, int n, int tid, int nthreads) {
  for (int i = tid; i < n; i += nthreads) odata[i] = buffer[i];
}

/* The four ways the reference tests call a transfer: one or two phases,
 * plain or with the global-load flag and cache qualifiers. */
#define RUN_XFER(obj, two_phase, qualified, SRC_ARGS, dst)                                                   \
  do {                                                                                                       \
    if (!(two_phase)) {                                                                                      \
      if (qualified) obj.template execute_dma<true, LOAD_CACHE_GLOBAL, STORE_CACHE_GLOBAL>(SRC_ARGS, dst);   \
      else obj.execute_dma(SRC_ARGS, dst);                                                                   \
    } else {                                                                                                 \
      if (qualified) {                                                                                       \
        obj.template start_xfer_async<true, LOAD_CACHE_STREAMING, STORE_CACHE_STREAMING>(SRC_ARGS);          \
        obj.template wait_xfer_finish<true, LOAD_CACHE_STREAMING, STORE_CACHE_STREAMING>(dst);               \
      } else {                                                                                               \
        obj.start_xfer_async(SRC_ARGS);                                                                      \
        obj.wait_xfer_finish(dst);                                                                           \
      }                                                                                                      \
    }                                                                                                        \
  } while (0)

#if HAVE_V2
/* ---------------------------------------------------------------- sequential */
template <bool WS, typename MAKE>
__global__ void __launch_bounds__(1024, 1)
seq_kernel(const float *idata, float *odata, int offset, int buffer_floats, int ncompute, int ndma, int bytes,
           bool two_phase, bool qualified) {
  extern __shared__ float buffer[];
  typename MAKE::type dma = MAKE::make(ncompute, ndma, bytes);
  if (WS) {
    if (dma.owns_this_thread()) {
      RUN_XFER(dma, two_phase, qualified, idata + offset, buffer + offset);
    } else {
      zero_buffer(buffer, buffer_floats, threadIdx.x, ncompute);
      dma.start_async_dma();
      dma.wait_for_dma_finish();
      copy_out(odata, buffer, buffer_floats, threadIdx.x, ncompute);
    }
  } else {
    zero_buffer(buffer, buffer_floats, threadIdx.x, blockDim.x);
    __syncthreads();
    RUN_XFER(dma, two_phase, qualified, idata + offset, buffer + offset);
    __syncthreads();
    copy_out(odata, buffer, buffer_floats, threadIdx.x, blockDim.x);
  }
}
/* object factories: warp-specialised objects use dmaID 1 and put the DMA threads after the compute threads */
template <bool WS, int A> struct SeqL1 {
  typedef CudaDMASequential<WS, A, BPT> type;
  __device__ static type make(int nc, int nd, int bytes) { return make_(nc, nd, bytes, (char (*)[WS ? 1 : 2])0); }
  __device__ static type make_(int nc, int nd, int bytes, char (*)[1]) { return type(1, nd, nc, nc, bytes); }
  __device__ static type make_(int nc, int nd, int bytes, char (*)[2]) { return type(bytes); }
};
template <bool WS, int A, int E> struct SeqL2 {
  typedef CudaDMASequential<WS, A, BPT, E> type;
  __device__ static type make(int nc, int nd, int bytes) { return make_(nc, nd, (char (*)[WS ? 1 : 2])0); }
  __device__ static type make_(int nc, int nd, char (*)[1]) { return type(1, nd, nc, nc); }
  __device__ static type make_(int nc, int nd, char (*)[2]) { return type(); }
};
template <bool WS, int A, int E, int T> struct SeqL3 {
  typedef CudaDMASequential<WS, A, BPT, E, T> type;
  __device__ static type make(int nc, int nd, int bytes) { return make_(nc, (char (*)[WS ? 1 : 2])0); }
  __device__ static type make_(int nc, char (*)[1]) { return type(1, nc, nc); }
  __device__ static type make_(int nc, char (*)[2]) { return type(); }
};

template <bool WS, typename MAKE>
int seq_run(int two_phase, int qualified, int offset, int bytes, int ndma, const float *h_in, float *h_out,
            int buffer_floats) {
  Buffers b;
  if (int r = b.init(h_in, buffer_floats, buffer_floats)) return r;
  const int ncompute = 32;
  const int threads = WS ? ncompute + ndma : ndma;
  auto k = seq_kernel<WS, MAKE>;
  if (int r = big_smem(k, (size_t)buffer_floats * 4)) return r;
  k<<<1, threads, buffer_floats * 4>>>(b.d_in, b.d_out, offset, buffer_floats, ncompute, ndma, bytes, two_phase != 0,
                                       qualified != 0);
  return b.fetch(h_out);
}

/* shapes instantiated for the template forms that fix sizes at compile time */
#define SEQ_SHAPES(X) X(16, 16384, 128) X(8, 1000, 64) X(4, 2532, 96)

template <bool WS>
int seq_dispatch(int level, int two_phase, int qualified, int alignment, int offset, int bytes, int ndma,
                 const float *h_in, float *h_out, int buffer_floats) {
  if (level == 1) {
    switch (alignment) {
      case 4: return seq_run<WS, SeqL1<WS, 4>>(two_phase, qualified, offset, bytes, ndma, h_in, h_out, buffer_floats);
      case 8: return seq_run<WS, SeqL1<WS, 8>>(two_phase, qualified, offset, bytes, ndma, h_in, h_out, buffer_floats);
      case 16: return seq_run<WS, SeqL1<WS, 16>>(two_phase, qualified, offset, bytes, ndma, h_in, h_out, buffer_floats);
    }
    return -1;
  }
#define SEQ_CASE(A, E, T)                                                                                         \
  if (alignment == A && bytes == E) {                                                                             \
    if (level == 2) return seq_run<WS, SeqL2<WS, A, E>>(two_phase, qualified, offset, bytes, ndma, h_in, h_out, buffer_floats); \
    if (level == 3 && ndma == T)                                                                                  \
      return seq_run<WS, SeqL3<WS, A, E, T>>(two_phase, qualified, offset, bytes, ndma, h_in, h_out, buffer_floats);   \
  }
  SEQ_SHAPES(SEQ_CASE)
#undef SEQ_CASE
  return -1;
}

/* ------------------------------------------------------------------- strided */
template <bool WS, typename MAKE>
__global__ void __launch_bounds__(1024, 1)
strided_kernel(const float *idata, float *odata, int offset, int buffer_floats, int ncompute, int ndma, int bytes,
               int rows, int sstride, int dstride, bool two_phase, bool qualified) {
  extern __shared__ float buffer[];
  typename MAKE::type dma = MAKE::make(ncompute, ndma, bytes, rows, sstride, dstride);
  if (WS) {
    if (dma.owns_this_thread()) {
      RUN_XFER(dma, two_phase, qualified, idata + offset, buffer + offset);
    } else {
      zero_buffer(buffer, buffer_floats, threadIdx.x, ncompute);
      dma.start_async_dma();
      dma.wait_for_dma_finish();
      copy_out(odata, buffer, buffer_floats, threadIdx.x, ncompute);
    }
  } else {
    zero_buffer(buffer, buffer_floats, threadIdx.x, blockDim.x);
    __syncthreads();
    RUN_XFER(dma, two_phase, qualified, idata + offset, buffer + offset);
    __syncthreads();
    copy_out(odata, buffer, buffer_floats, threadIdx.x, blockDim.x);
  }
}
/* dstride < 0 selects the one-stride constructor (the same stride on both sides) */
#define STRIDED_FACTORY(NAME, TYPE, WS_ARGS, NWS_ARGS)                                                       \
  struct NAME {                                                                                              \
    typedef TYPE type;                                                                                       \
    __device__ static type make(int nc, int nd, int bytes, int rows, int s, int d) {                         \
      return make_(nc, nd, bytes, rows, s, d, (char (*)[WS ? 1 : 2])0);                                      \
    }                                                                                                        \
    __device__ static type make_(int nc, int nd, int bytes, int rows, int s, int d, char (*)[1]) {           \
      if (d < 0) return type(WS_ARGS s);                                                                     \
      return type(WS_ARGS s, d);                                                                             \
    }                                                                                                        \
    __device__ static type make_(int nc, int nd, int bytes, int rows, int s, int d, char (*)[2]) {           \
      if (d < 0) return type(NWS_ARGS s);                                                                    \
      return type(NWS_ARGS s, d);                                                                            \
    }                                                                                                        \
  }
#define COMMA ,
template <bool WS, int A>
STRIDED_FACTORY(StrL1, CudaDMAStrided<WS COMMA A COMMA BPT>, 1 COMMA nd COMMA nc COMMA nc COMMA bytes COMMA rows COMMA,
                bytes COMMA rows COMMA);
template <bool WS, int A, int E>
STRIDED_FACTORY(StrL2, CudaDMAStrided<WS COMMA A COMMA BPT COMMA E>, 1 COMMA nd COMMA nc COMMA nc COMMA rows COMMA,
                rows COMMA);
template <bool WS, int A, int E, int T>
STRIDED_FACTORY(StrL3, CudaDMAStrided<WS COMMA A COMMA BPT COMMA E COMMA T>, 1 COMMA nc COMMA nc COMMA rows COMMA,
                rows COMMA);
template <bool WS, int A, int E, int T, int N>
STRIDED_FACTORY(StrL4, CudaDMAStrided<WS COMMA A COMMA BPT COMMA E COMMA T COMMA N>, 1 COMMA nc COMMA nc COMMA, );

template <bool WS, typename MAKE>
int strided_run(int two_phase, int qualified, int offset, int bytes, int rows, int sstride, int dstride, int ndma,
                const float *h_in, int in_floats, float *h_out, int buffer_floats) {
  Buffers b;
  if (int r = b.init(h_in, in_floats, buffer_floats)) return r;
  const int ncompute = 32;
  const int threads = WS ? ncompute + ndma : ndma;
  auto k = strided_kernel<WS, MAKE>;
  if (int r = big_smem(k, (size_t)buffer_floats * 4)) return r;
  k<<<1, threads, buffer_floats * 4>>>(b.d_in, b.d_out, offset, buffer_floats, ncompute, ndma, bytes, rows, sstride,
                                       dstride, two_phase != 0, qualified != 0);
  return b.fetch(h_out);
}

#define STRIDED_SHAPES(X) X(16, 256, 128, 128) X(8, 320, 32, 24) X(4, 100, 64, 7)

template <bool WS>
int strided_dispatch(int level, int two_phase, int qualified, int alignment, int offset, int bytes, int rows,
                     int sstride, int dstride, int ndma, const float *h_in, int in_floats, float *h_out,
                     int buffer_floats) {
#define ARGS two_phase, qualified, offset, bytes, rows, sstride, dstride, ndma, h_in, in_floats, h_out, buffer_floats
  if (level == 1) {
    switch (alignment) {
      case 4: return strided_run<WS, StrL1<WS, 4>>(ARGS);
      case 8: return strided_run<WS, StrL1<WS, 8>>(ARGS);
      case 16: return strided_run<WS, StrL1<WS, 16>>(ARGS);
    }
    return -1;
  }
#define STR_CASE(A, E, T, N)                                                                    \
  if (alignment == A && bytes == E) {                                                           \
    if (level == 2) return strided_run<WS, StrL2<WS, A, E>>(ARGS);                              \
    if (level == 3 && ndma == T) return strided_run<WS, StrL3<WS, A, E, T>>(ARGS);              \
    if (level == 4 && ndma == T && rows == N) return strided_run<WS, StrL4<WS, A, E, T, N>>(ARGS); \
  }
  STRIDED_SHAPES(STR_CASE)
#undef STR_CASE
#undef ARGS
  return -1;
}

/* ------------------------------------------------------------------ indirect */
/* gather: global rows -> packed shared buffer -> copied out whole */
template <bool WS, typename MAKE>
__global__ void __launch_bounds__(1024, 1)
gather_kernel(const float *idata, float *odata, const int *index, int offset, int buffer_floats, int ncompute,
              int ndma, int bytes, int rows, int alt, bool two_phase, bool qualified) {
  extern __shared__ float buffer[];
  typename MAKE::type dma = MAKE::make(ncompute, ndma, bytes, rows, alt);
  if (WS) {
    if (dma.owns_this_thread()) {
      RUN_XFER(dma, two_phase, qualified, index COMMA idata + offset, buffer + offset);
    } else {
      zero_buffer(buffer, buffer_floats, threadIdx.x, ncompute);
      dma.start_async_dma();
      dma.wait_for_dma_finish();
      copy_out(odata, buffer, buffer_floats, threadIdx.x, ncompute);
    }
  } else {
    zero_buffer(buffer, buffer_floats, threadIdx.x, blockDim.x);
    __syncthreads();
    RUN_XFER(dma, two_phase, qualified, index COMMA idata + offset, buffer + offset);
    __syncthreads();
    copy_out(odata, buffer, buffer_floats, threadIdx.x, blockDim.x);
  }
}
/* scatter: the compute threads load the packed shared buffer, the object writes its rows to global */
template <bool WS, typename MAKE>
__global__ void __launch_bounds__(1024, 1)
scatter_kernel(const float *idata, float *odata, const int *index, int offset, int buffer_floats, int ncompute,
               int ndma, int bytes, int rows, int alt, bool two_phase, bool qualified) {
  extern __shared__ float buffer[];
  typename MAKE::type dma = MAKE::make(ncompute, ndma, bytes, rows, alt);
  if (WS) {
    if (dma.owns_this_thread()) {
      RUN_XFER(dma, two_phase, qualified, index COMMA buffer + offset, odata + offset);
    } else {
      copy_out(buffer, idata, buffer_floats, threadIdx.x, ncompute);
      dma.start_async_dma();
      dma.wait_for_dma_finish();
    }
  } else {
    copy_out(buffer, idata, buffer_floats, threadIdx.x, blockDim.x);
    __syncthreads();
    RUN_XFER(dma, two_phase, qualified, index COMMA buffer + offset, odata + offset);
    __syncthreads();
  }
}
#define INDIRECT_FACTORY(NAME, TYPE, WS_ARGS, NWS_ARGS)                                          \
  struct NAME {                                                                                  \
    typedef TYPE type;                                                                           \
    __device__ static type make(int nc, int nd, int bytes, int rows, int alt) {                  \
      return make_(nc, nd, bytes, rows, alt, (char (*)[WS ? 1 : 2])0);                           \
    }                                                                                            \
    __device__ static type make_(int nc, int nd, int bytes, int rows, int alt, char (*)[1]) {    \
      return type(WS_ARGS alt);                                                                  \
    }                                                                                            \
    __device__ static type make_(int nc, int nd, int bytes, int rows, int alt, char (*)[2]) {    \
      return type(NWS_ARGS alt);                                                                 \
    }                                                                                            \
  }
template <bool G, bool WS, int A>
INDIRECT_FACTORY(IndL1, CudaDMAIndirect<G COMMA WS COMMA A COMMA BPT>,
                 1 COMMA nd COMMA nc COMMA nc COMMA bytes COMMA rows COMMA, bytes COMMA rows COMMA);
template <bool G, bool WS, int A, int E>
INDIRECT_FACTORY(IndL2, CudaDMAIndirect<G COMMA WS COMMA A COMMA BPT COMMA E>,
                 1 COMMA nd COMMA nc COMMA nc COMMA rows COMMA, rows COMMA);
template <bool G, bool WS, int A, int E, int T>
INDIRECT_FACTORY(IndL3, CudaDMAIndirect<G COMMA WS COMMA A COMMA BPT COMMA E COMMA T>,
                 1 COMMA nc COMMA nc COMMA rows COMMA, rows COMMA);
template <bool G, bool WS, int A, int E, int T, int N>
INDIRECT_FACTORY(IndL4, CudaDMAIndirect<G COMMA WS COMMA A COMMA BPT COMMA E COMMA T COMMA N>,
                 1 COMMA nc COMMA nc COMMA, );

template <bool G, bool WS, typename MAKE>
int indirect_run(int two_phase, int qualified, int offset, int bytes, int rows, int alt, int ndma, const int *h_idx,
                 const float *h_in, int in_floats, float *h_out, int out_floats, int buffer_floats) {
  Buffers b;
  if (int r = b.init(h_in, in_floats, out_floats, h_idx, rows)) return r;
  const int ncompute = 32;
  const int threads = WS ? ncompute + ndma : ndma;
  if (G) {
    auto k = gather_kernel<WS, MAKE>;
    if (int r = big_smem(k, (size_t)buffer_floats * 4)) return r;
    k<<<1, threads, buffer_floats * 4>>>(b.d_in, b.d_out, b.d_idx, offset, buffer_floats, ncompute, ndma, bytes, rows,
                                         alt, two_phase != 0, qualified != 0);
  } else {
    auto k = scatter_kernel<WS, MAKE>;
    if (int r = big_smem(k, (size_t)buffer_floats * 4)) return r;
    k<<<1, threads, buffer_floats * 4>>>(b.d_in, b.d_out, b.d_idx, offset, buffer_floats, ncompute, ndma, bytes, rows,
                                         alt, two_phase != 0, qualified != 0);
  }
  return b.fetch(h_out);
}

#define INDIRECT_SHAPES(X) X(16, 32, 128, 128) X(8, 40, 32, 9) X(4, 12, 64, 20)

template <bool G, bool WS>
int indirect_dispatch(int level, int two_phase, int qualified, int alignment, int offset, int bytes, int rows,
                      int alt, int ndma, const int *h_idx, const float *h_in, int in_floats, float *h_out,
                      int out_floats, int buffer_floats) {
#define ARGS two_phase, qualified, offset, bytes, rows, alt, ndma, h_idx, h_in, in_floats, h_out, out_floats, buffer_floats
  if (level == 1) {
    switch (alignment) {
      case 4: return indirect_run<G, WS, IndL1<G, WS, 4>>(ARGS);
      case 8: return indirect_run<G, WS, IndL1<G, WS, 8>>(ARGS);
      case 16: return indirect_run<G, WS, IndL1<G, WS, 16>>(ARGS);
    }
    return -1;
  }
#define IND_CASE(A, E, T, N)                                                                            \
  if (alignment == A && bytes == E) {                                                                   \
    if (level == 2) return indirect_run<G, WS, IndL2<G, WS, A, E>>(ARGS);                               \
    if (level == 3 && ndma == T) return indirect_run<G, WS, IndL3<G, WS, A, E, T>>(ARGS);               \
    if (level == 4 && ndma == T && rows == N) return indirect_run<G, WS, IndL4<G, WS, A, E, T, N>>(ARGS); \
  }
  INDIRECT_SHAPES(IND_CASE)
#undef IND_CASE
#undef ARGS
  return -1;
}
#endif /* HAVE_V2 */

#if HAVE_HALO
/* ---------------------------------------------------------------------- halo */
template <typename ELMT, int RADIUS, bool CORNERS, int ALIGNMENT>
__global__ void __launch_bounds__(1024, 1)
halo_kernel(const ELMT *idata, ELMT *odata, int offset, int dimx, int dimy, int pitch, int buffer_elems,
            int ncompute, int ndma) {
  extern __shared__ float share[];
  ELMT *buffer = reinterpret_cast<ELMT *>(share);
  cudaDMAHalo<ELMT, RADIUS, CORNERS, ALIGNMENT> dma(1, ndma, ncompute, ncompute, dimx, dimy, pitch);
  if (dma.owns_this_thread()) {
    dma.execute_dma(idata + offset + RADIUS + RADIUS * pitch, buffer + offset + RADIUS + RADIUS * (dimx + 2 * RADIUS));
  } else {
    zero_buffer(share, buffer_elems * (int)(sizeof(ELMT) / 4), threadIdx.x, ncompute);
    dma.start_async_dma();
    dma.wait_for_dma_finish();
    copy_out(reinterpret_cast<float *>(odata), share, buffer_elems * (int)(sizeof(ELMT) / 4), threadIdx.x, ncompute);
  }
}
template <typename ELMT, int RADIUS, bool CORNERS, int ALIGNMENT>
int halo_run(int offset, int dimx, int dimy, int pitch, int ndma, const float *h_in, float *h_out) {
  const int elems = (dimx + 2 * RADIUS) * (dimy + 2 * RADIUS) + offset;
  const int in_elems = pitch * (dimy + 2 * RADIUS) + offset;
  const int w = sizeof(ELMT) / 4;
  Buffers b;
  if (int r = b.init(h_in, (size_t)in_elems * w, (size_t)elems * w)) return r;
  const int ncompute = 32;
  auto k = halo_kernel<ELMT, RADIUS, CORNERS, ALIGNMENT>;
  if (int r = big_smem(k, (size_t)elems * sizeof(ELMT))) return r;
  k<<<1, ncompute + ndma, elems * sizeof(ELMT)>>>(reinterpret_cast<const ELMT *>(b.d_in),
                                                  reinterpret_cast<ELMT *>(b.d_out), offset, dimx, dimy, pitch, elems,
                                                  ncompute, ndma);
  return b.fetch(h_out);
}
template <typename ELMT, int ALIGNMENT>
int halo_dispatch(int radius, int corners, int offset, int dimx, int dimy, int pitch, int ndma, const float *h_in,
                  float *h_out) {
#define HALO_CASE(R)                                                                                             \
  if (radius == R)                                                                                               \
    return corners ? halo_run<ELMT, R, true, ALIGNMENT>(offset, dimx, dimy, pitch, ndma, h_in, h_out)            \
                   : halo_run<ELMT, R, false, ALIGNMENT>(offset, dimx, dimy, pitch, ndma, h_in, h_out);
  HALO_CASE(1) HALO_CASE(2) HALO_CASE(4) HALO_CASE(8)
#undef HALO_CASE
  return -1;
}
#endif /* HAVE_HALO */

}  // namespace

#ifdef HAVE_STATUS
/* A transfer whose start signal never comes: the compute threads leave without calling
 * start_async_dma, so the DMA threads' wait runs out, records its code and returns. */
__global__ void starved_kernel(const float *idata, int ncompute, int ndma) {
  extern __shared__ float buffer[];
  CudaDMASequential<true, 16, BPT> dma(3, ndma, ncompute, ncompute, 256);
  if (dma.owns_this_thread()) dma.execute_dma(idata, buffer);
}
#endif

#ifdef HAVE_STATUS
/* CudaDMACustom (v1 cudaDMACustom, include/cudaDMA.h:4184-4208): only the handshake; the DMA
 * threads fill the buffer with a copy loop of their own, ordinary loads and stores, between
 * wait_for_dma_start() and finish_async_dma(). `iters` buffers of nfloats floats go through one
 * shared buffer. PLAIN_WAIT selects wait_for_dma_start_for_stores(), the same wait without the
 * fence that only asynchronous copies need. */
template <bool PLAIN_WAIT>
__global__ void custom_copy_kernel(const float *__restrict__ idata, float *__restrict__ odata, int nfloats, int iters,
                                   int ncompute, int ndma) {
  extern __shared__ float buffer[];
  CudaDMACustom dma(2, ndma, ncompute, ncompute);
  if (dma.owns_this_thread()) {
    const int t = threadIdx.x - ncompute;
    for (int it = 0; it < iters; ++it) {
      if (PLAIN_WAIT) dma.wait_for_dma_start_for_stores();
      else dma.wait_for_dma_start();
      for (int i = t; i < nfloats; i += ndma) buffer[i] = idata[(size_t)it * nfloats + i];
      dma.finish_async_dma();
    }
  } else {
    for (int it = 0; it < iters; ++it) {
      dma.start_async_dma();
      dma.wait_for_dma_finish();
      for (int i = threadIdx.x; i < nfloats; i += ncompute) odata[(size_t)it * nfloats + i] = buffer[i];
    }
  }
}
#endif

extern "C" {

#ifdef HAVE_STATUS
/* h_in, h_out: iters * nfloats floats. Returns 0, a negative argument / CUDA code, or the status
 * word of a wait that gave up. */
long long ENTRY(custom_copy)(int plain_wait, int nfloats, int iters, int ncompute, int ndma, const float *h_in,
                             float *h_out) {
  if (!h_in || !h_out || nfloats <= 0 || nfloats > 12000 || iters <= 0 || ncompute <= 0 || (ncompute & 31) || ndma <= 0 ||
      (ndma & 31) || ncompute + ndma > 1024)
    return -1;
  const size_t bytes = (size_t)nfloats * iters * sizeof(float);
  float *d_in = nullptr, *d_out = nullptr;
  cudaError_t e = cudaMalloc(&d_in, bytes);
  if (e == cudaSuccess) e = cudaMalloc(&d_out, bytes);
  if (e == cudaSuccess) e = cudaMemcpy(d_in, h_in, bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(d_out, 0, bytes);
  if (e == cudaSuccess) {
    if (plain_wait) custom_copy_kernel<true><<<1, ncompute + ndma, nfloats * sizeof(float)>>>(d_in, d_out, nfloats, iters, ncompute, ndma);
    else custom_copy_kernel<false><<<1, ncompute + ndma, nfloats * sizeof(float)>>>(d_in, d_out, nfloats, iters, ncompute, ndma);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(h_out, d_out, bytes, cudaMemcpyDeviceToHost);
  unsigned int w = 0;
  if (e == cudaSuccess) e = cudadma_b200::read_status(&w, 0);
  cudaFree(d_in);
  cudaFree(d_out);
  return e == cudaSuccess ? (long long)w : -2;
}

/* Runs starved_kernel; returns the status word it left (0 would mean the wait never gave up),
 * negative on a CUDA error. The context stays usable. */
long long ENTRY(starved_wait)(void) {
  float *d = nullptr;
  if (cudaMalloc(&d, 1024) != cudaSuccess) return -2;
  starved_kernel<<<1, 64, 1024>>>(d, 32, 32);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  unsigned int w = 0;
  if (e == cudaSuccess) e = cudadma_b200::read_status(&w, 0);
  cudaFree(d);
  return e == cudaSuccess ? (long long)w : -2;
}
#endif

/* which families this build contains: bit 0 sequential/strided/indirect, bit 1 halo */
int ENTRY(families)(void) { return (HAVE_V2 ? 1 : 0) | (HAVE_HALO ? 2 : 0); }

#if HAVE_V2
/* h_in, h_out: buffer_floats floats; the element starts at float `offset` of both */
int ENTRY(sequential)(int ws, int level, int two_phase, int qualified, int alignment, int offset, int bytes, int ndma,
                      const float *h_in, float *h_out, int buffer_floats) {
  if (!h_in || !h_out || bytes <= 0 || (bytes & 3) || ndma <= 0 || (ndma & 31) || ndma > 992 ||
      offset * 4 + bytes > buffer_floats * 4)
    return -1;
  return ws ? seq_dispatch<true>(level, two_phase, qualified, alignment, offset, bytes, ndma, h_in, h_out, buffer_floats)
            : seq_dispatch<false>(level, two_phase, qualified, alignment, offset, bytes, ndma, h_in, h_out, buffer_floats);
}

/* h_in: in_floats floats (rows sstride bytes apart from float `offset`); h_out: the shared buffer,
 * buffer_floats floats (rows dstride bytes apart from float `offset`); dstride < 0: one-stride form,
 * rows sstride bytes apart on both sides */
int ENTRY(strided)(int ws, int level, int two_phase, int qualified, int alignment, int offset, int bytes, int rows,
                   int sstride, int dstride, int ndma, const float *h_in, int in_floats, float *h_out,
                   int buffer_floats) {
  if (!h_in || !h_out || bytes <= 0 || (bytes & 3) || rows <= 0 || ndma <= 0 || (ndma & 31) || ndma > 992) return -1;
  const long long dpitch = dstride < 0 ? sstride : dstride;
  if (offset * 4ll + (rows - 1ll) * sstride + bytes > in_floats * 4ll) return -1;
  if (offset * 4ll + (rows - 1ll) * dpitch + bytes > buffer_floats * 4ll) return -1;
  return ws ? strided_dispatch<true>(level, two_phase, qualified, alignment, offset, bytes, rows, sstride, dstride,
                                     ndma, h_in, in_floats, h_out, buffer_floats)
            : strided_dispatch<false>(level, two_phase, qualified, alignment, offset, bytes, rows, sstride, dstride,
                                      ndma, h_in, in_floats, h_out, buffer_floats);
}

/* gather != 0: h_in is the table (in_floats), h_out the shared buffer (out_floats == buffer_floats).
 * gather == 0: h_in is the packed shared buffer (in_floats == buffer_floats), h_out the table (out_floats).
 * h_idx: `rows` record numbers. */
int ENTRY(indirect)(int gather, int ws, int level, int two_phase, int qualified, int alignment, int offset, int bytes,
                    int rows, int alt, int ndma, const int *h_idx, const float *h_in, int in_floats, float *h_out,
                    int out_floats, int buffer_floats) {
  if (!h_in || !h_out || !h_idx || bytes <= 0 || (bytes & 3) || rows <= 0 || ndma <= 0 || (ndma & 31) || ndma > 992)
    return -1;
  const long long pitch = alt > bytes ? alt : bytes;
  if (offset * 4ll + (rows - 1ll) * pitch + bytes > buffer_floats * 4ll) return -1;
  const long long table_bytes = (gather ? in_floats : out_floats) * 4ll;
  for (int i = 0; i < rows; ++i)
    if (h_idx[i] < 0 || offset * 4ll + (h_idx[i] + 1ll) * bytes > table_bytes) return -1;
  if (gather)
    return ws ? indirect_dispatch<true, true>(level, two_phase, qualified, alignment, offset, bytes, rows, alt, ndma,
                                              h_idx, h_in, in_floats, h_out, out_floats, buffer_floats)
              : indirect_dispatch<true, false>(level, two_phase, qualified, alignment, offset, bytes, rows, alt, ndma,
                                               h_idx, h_in, in_floats, h_out, out_floats, buffer_floats);
  return ws ? indirect_dispatch<false, true>(level, two_phase, qualified, alignment, offset, bytes, rows, alt, ndma,
                                             h_idx, h_in, in_floats, h_out, out_floats, buffer_floats)
            : indirect_dispatch<false, false>(level, two_phase, qualified, alignment, offset, bytes, rows, alt, ndma,
                                              h_idx, h_in, in_floats, h_out, out_floats, buffer_floats);
}
#endif

#if HAVE_HALO
/* h_in: (pitch * (dimy + 2 radius) + offset) elements; h_out: ((dimx + 2 radius)(dimy + 2 radius) + offset)
 * elements; elmt_floats = 1, 2 or 4 (float, float2, float4); offset in elements */
int ENTRY(halo)(int elmt_floats, int radius, int corners, int alignment, int offset, int dimx, int dimy, int pitch,
                int ndma, const float *h_in, float *h_out) {
  if (!h_in || !h_out || dimx <= 0 || dimy <= 0 || pitch < dimx + 2 * radius || ndma <= 0 || (ndma & 31) || ndma > 992)
    return -1;
#define HALO_TYPE(W, T)                                                                                \
  if (elmt_floats == W) {                                                                              \
    if (alignment == 4) return halo_dispatch<T, 4>(radius, corners, offset, dimx, dimy, pitch, ndma, h_in, h_out);   \
    if (alignment == 8) return halo_dispatch<T, 8>(radius, corners, offset, dimx, dimy, pitch, ndma, h_in, h_out);   \
    if (alignment == 16) return halo_dispatch<T, 16>(radius, corners, offset, dimx, dimy, pitch, ndma, h_in, h_out); \
  }
  HALO_TYPE(1, float) HALO_TYPE(2, float2) HALO_TYPE(4, float4)
#undef HALO_TYPE
  return -1;
}
#endif

} /* extern "C" */
