/*
 * capi.cu -- host side of libcudadma_b200.so: argument checks, tensor-map
 * encoding, launches, the host-buffer forms and their device workspace.
 * Declarations and the reference programs each entry point replaces are in
 * include/cudadma_b200.h.
 */
#include "cudadma_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

/* tuning knobs (compile-time): stages in flight per CTA and CTAs per SM of each kernel */
#ifndef SEQ_STAGES
#define SEQ_STAGES 4
#endif
#ifndef SEQ_CTAS_PER_SM
#define SEQ_CTAS_PER_SM 3
#endif
#ifndef SEQ_BULK_STORE
#define SEQ_BULK_STORE false /* register-staged loads and plain stores; true: bulk copies both ways (dma_kernels.cuh) */
#endif

#ifndef P_SEQ_BPT
#define P_SEQ_BPT 128 /* BYTES_PER_THREAD of the portable sequential copy's objects: staged through registers, 2 % over 64 */
#endif

#ifndef TR_STAGES
#define TR_STAGES 3
#endif
#ifndef TR_CTAS_PER_SM
#define TR_CTAS_PER_SM 2
#endif
#ifndef TR_SUPER
#define TR_SUPER 2 /* tile numbering of the transpose, see dma_kernels.cuh: 2 measured 0.8 % over 1, 4 to 16 below it */
#endif
#ifndef HOST_PIPE_CHUNK_BYTES
#define HOST_PIPE_CHUNK_BYTES ((size_t)128 << 20) /* piece of the field per upload in the overlapped host run */
#endif
#ifndef GS_STAGES
#define GS_STAGES 4 /* buffers per CTA and direction; 8 measured 2 % slower at the same number of CTAs */
#endif
#ifndef GS_CTAS_PER_SM
#define GS_CTAS_PER_SM 8 /* upper bound; the launch takes what is resident (five per SM at 40 registers) */
#endif
#ifndef STENCIL25_L2PROMO
#define STENCIL25_L2PROMO CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif
#ifndef STENCIL_CTAS_TARGET
#define STENCIL_CTAS_TARGET 8 /* CTAs per SM the automatic z_chunk aims for (two are resident) */
#endif
#ifndef STENCIL_MAX_RUN
#define STENCIL_MAX_RUN 128 /* longest run of planes the automatic z_chunk gives one CTA (see plan_chunks) */
#endif

/* Waits inside this library's kernels give up after about four seconds; the wait of a sharded
 * rank for its neighbours (SLAB_WAIT_LIMIT_CYCLES, about two) is the shorter one, so that a
 * neighbour that is late is reported as that and not as a starved buffer. */
#define CUDADMA_WAIT_LIMIT_CYCLES (1ll << 33)
#include "cudadma.h"
#include "common_kernels.cuh"
#include "dma_kernels.cuh"
#include "portable_kernels.cuh"
#include "stencil25.cuh"

namespace {

thread_local int t_last_cuda_error = 0;
std::atomic<unsigned long long> g_launches{0};

#define CK(call)                                   \
  do {                                             \
    cudaError_t e_ = (call);                       \
    if (e_ != cudaSuccess) {                       \
      t_last_cuda_error = (int)e_;                 \
      return CUDADMA_ERR_CUDA;                     \
    }                                              \
  } while (0)

int launched() {
  ++g_launches;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    t_last_cuda_error = (int)e;
    return CUDADMA_ERR_CUDA;
  }
  return CUDADMA_OK;
}

/* What the library remembers per device (a process may drive several): values are looked up on
 * first use with that device current. Races between threads only repeat a lookup. */
constexpr int MAX_DEVICES = 64;
struct DeviceState {
  std::atomic<int> sms{0};
  std::atomic<bool> stencil_smem{false};   /* tensor_kernel may use its dynamic shared memory */
  std::atomic<int> gather_fit[4] = {{0}, {0}, {0}, {0}}; /* resident CTAs per SM of gather_scatter_kernel, by record size */
};
DeviceState g_dev[MAX_DEVICES];

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
  return dev;
}

int sm_count() {
  const int dev = current_device();
  if (dev < 0) return 0;
  int n = g_dev[dev].sms.load();
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 0;
    g_dev[dev].sms.store(n);
  }
  return n;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

/* cuTensorMapEncodeTiled is fetched through the runtime so that the library
 * has no link-time dependency on the driver library and loads on a machine
 * without a GPU. */
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

/* fp32 tensor map, `rank` dims (x fastest), zero fill outside the tensor */
int make_map_f32(CUtensorMap *map, const void *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides_bytes,
                 const cuuint32_t *box, CUtensorMapSwizzle swizzle,
                 CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) { t_last_cuda_error = (int)cudaErrorNotSupported; return CUDADMA_ERR_CUDA; }
  cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void *>(base), dims,
                  strides_bytes, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { t_last_cuda_error = (int)cudaErrorInvalidValue; return CUDADMA_ERR_CUDA; }
  return CUDADMA_OK;
}

template <typename K>
int allow_smem(K kernel, int bytes) {
  CK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return CUDADMA_OK;
}

/* ---- grow-only device workspace for the host-buffer forms ----
 * One workspace per process, on the device that was current when it was last used: a call made
 * with another device current drops it (arrays, streams, events) and starts a new one there. */
std::recursive_mutex g_ws_mutex;
void *g_ws[4] = {nullptr, nullptr, nullptr, nullptr};
size_t g_ws_bytes[4] = {0, 0, 0, 0};
int g_ws_device = -1;
cudaStream_t g_ws_stream = nullptr;
cudaStream_t g_ws_up = nullptr, g_ws_down = nullptr;          /* copy streams of the overlapped host run */
cudaEvent_t g_ws_ev_up = nullptr, g_ws_ev_step = nullptr;

void ws_drop() {
  for (int i = 0; i < 4; ++i) {
    if (g_ws[i]) cudaFree(g_ws[i]);
    g_ws[i] = nullptr; g_ws_bytes[i] = 0;
  }
  if (g_ws_stream) cudaStreamDestroy(g_ws_stream);
  if (g_ws_up) cudaStreamDestroy(g_ws_up);
  if (g_ws_down) cudaStreamDestroy(g_ws_down);
  if (g_ws_ev_up) cudaEventDestroy(g_ws_ev_up);
  if (g_ws_ev_step) cudaEventDestroy(g_ws_ev_step);
  g_ws_stream = g_ws_up = g_ws_down = nullptr;
  g_ws_ev_up = g_ws_ev_step = nullptr;
}
int ws_bind_device() {
  int dev = -1;
  CK(cudaGetDevice(&dev));
  if (dev != g_ws_device) {
    if (g_ws_device >= 0) ws_drop();
    g_ws_device = dev;
  }
  return CUDADMA_OK;
}
int ws_get(int slot, size_t bytes, void **out) {
  if (int r = ws_bind_device()) return r;
  if (g_ws_bytes[slot] < bytes) {
    if (g_ws[slot]) cudaFree(g_ws[slot]);
    g_ws[slot] = nullptr; g_ws_bytes[slot] = 0;
    cudaError_t e = cudaMalloc(&g_ws[slot], bytes);
    if (e != cudaSuccess) { t_last_cuda_error = (int)e; cudaGetLastError(); return CUDADMA_ERR_NOMEM; }
    g_ws_bytes[slot] = bytes;
  }
  *out = g_ws[slot];
  return CUDADMA_OK;
}
int ws_stream(cudaStream_t *s) {
  if (int r = ws_bind_device()) return r;
  if (!g_ws_stream) CK(cudaStreamCreateWithFlags(&g_ws_stream, cudaStreamNonBlocking));
  *s = g_ws_stream;
  return CUDADMA_OK;
}

int finish_status(cudaStream_t s) {
  unsigned int w = 0;
  CK(cudadma_b200::read_status(&w, s));
  return w ? CUDADMA_ERR_TIMEOUT : CUDADMA_OK;
}

/* The last few stencil tensor maps of the calling thread, by what they were encoded from: a time
 * loop alternates between two arrays, so it encodes twice and then only looks up. */
struct MapKey { const void *base; int nx, ny, nz; };
struct MapSlot { MapKey key; CUtensorMap map; };
thread_local MapSlot t_maps[4];
thread_local int t_maps_next = 0;

int stencil_map(const CUtensorMap **out, const float *in, int nx, int ny, int nz) {
  for (int i = 0; i < 4; ++i) {
    const MapKey &k = t_maps[i].key;
    if (k.base == in && k.nx == nx && k.ny == ny && k.nz == nz) { *out = &t_maps[i].map; return CUDADMA_OK; }
  }
  MapSlot &slot = t_maps[t_maps_next];
  t_maps_next = (t_maps_next + 1) & 3;
  slot.key = MapKey{nullptr, 0, 0, 0};
  const cuuint64_t dims[3] = {(cuuint64_t)nx, (cuuint64_t)ny, (cuuint64_t)nz};
  const cuuint64_t strides[2] = {(cuuint64_t)nx * 4, (cuuint64_t)nx * ny * 4};
  const cuuint32_t box[3] = {stencil25::WIN_X, stencil25::WIN_Y, 1};
  if (int r = make_map_f32(&slot.map, in, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, STENCIL25_L2PROMO)) return r;
  slot.key = MapKey{in, nx, ny, nz};
  *out = &slot.map;
  return CUDADMA_OK;
}

/* How the output planes of a launch are cut into runs, one run per CTA and tile (see tensor_kernel). */
struct ChunkPlan { int z_chunk, z_edge, zc; };

ChunkPlan plan_chunks(int depth, long long tiles, int sms, int z_chunk, int z_edge) {
  ChunkPlan p;
  if (z_edge > 0 && depth < 2 * z_edge + 1) z_edge = 0;
  const int inner = depth - 2 * (z_edge > 0 ? z_edge : 0); /* z_edge < 0: equal runs, highest first */
  if (z_chunk <= 0) {
    /* Enough CTAs for a few waves over the SMs, but runs of at least 32 planes so that the eight
     * lead-in/lead-out planes of a run stay a small share of its loads -- and of at most
     * STENCIL_MAX_RUN planes: the CTAs of a wave start on the same plane and read each other's
     * halo cells out of L2, but over a long run they drift apart in z until those cells come from
     * DRAM a second time. On a rested GPU, 1024 x 1024 x 2048: 747 Gpts/s with runs of 128 planes,
     * 721 with 64, 625 with 256, 585 with 512 or 1024. */
    const long long want = (long long)STENCIL_CTAS_TARGET * sms - (z_edge > 0 ? 2 * tiles : 0);
    long long chunks = (want + tiles - 1) / tiles;
    const long long least = ((long long)inner + STENCIL_MAX_RUN - 1) / STENCIL_MAX_RUN;
    if (chunks < least) chunks = least;
    if (chunks < 1) chunks = 1;
    z_chunk = (int)((inner + chunks - 1) / chunks);
    if (z_chunk < 32) z_chunk = 32;
  }
  if (z_chunk > inner) z_chunk = inner;
  p.z_chunk = z_chunk;
  p.z_edge = z_edge;
  p.zc = (inner + z_chunk - 1) / z_chunk + (z_edge > 0 ? 2 : 0);
  return p;
}

/* CTAs of a launch whose run of planes reaches into a pushed range (same rule as the kernel's) */
unsigned int boundary_ctas(const ChunkPlan &p, long long tiles, const stencil25::Peers &peer, int z_begin, int z_end) {
  long long n = 0;
  for (int bz = 0; bz < p.zc; ++bz) {
    int z0, depth;
    if (p.z_edge > 0) {
      if (bz == 0) { z0 = z_begin; depth = p.z_edge; }
      else if (bz == 1) { z0 = z_end - p.z_edge; depth = p.z_edge; }
      else {
        z0 = z_begin + p.z_edge + (bz - 2) * p.z_chunk;
        depth = (z_end - p.z_edge - z0 < p.z_chunk) ? (z_end - p.z_edge - z0) : p.z_chunk;
      }
    } else {
      z0 = z_begin + bz * p.z_chunk;
      depth = (z_end - z0 < p.z_chunk) ? (z_end - z0) : p.z_chunk;
    }
    if ((peer.lo && z0 < peer.lo_end) || (peer.hi && z0 + depth > peer.hi_begin)) n += tiles;
  }
  return (unsigned int)n;
}

const stencil25::Sync NO_SYNC = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0u, 0u, 0};

/* Launch of the tensor-map stencil kernel on output planes [z_begin, z_end); `peer` names second
 * destinations for the lowest and highest planes (see stencil25::Peers), `sync` the handshake with
 * the neighbour ranks (its boundary_ctas is filled in here), z_edge the depth of the two boundary
 * runs (0: equal runs). */
int launch_stencil_native(float *out, const stencil25::Peers &peer, stencil25::Sync sync, const float *in, int nx, int ny,
                          int nz, int z_begin, int z_end, const float coeff[5], int z_chunk, int z_edge, cudaStream_t s) {
  const int sms = sm_count();
  const int dev = current_device();
  if (sms <= 0 || dev < 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  stencil25::Coeffs k;
  for (int i = 0; i < 5; ++i) k.c[i] = coeff[i];
  const int tiles_x = (nx + stencil25::TILE_X - 1) / stencil25::TILE_X;
  const int tiles_y = (ny + stencil25::TILE_Y - 1) / stencil25::TILE_Y;
  const long long tiles = (long long)tiles_x * tiles_y;
  const ChunkPlan plan = plan_chunks(z_end - z_begin, tiles, sms, z_chunk, z_edge);
  if (plan.zc > 65535 || tiles_y > 65535) return CUDADMA_ERR_ARG;
  if (sync.ticket) {
    sync.boundary_ctas = boundary_ctas(plan, tiles, peer, z_begin, z_end);
    if (sync.boundary_ctas == 0) sync.ticket = nullptr;
  }
  const CUtensorMap *map = nullptr;
  if (int r = stencil_map(&map, in, nx, ny, nz)) return r;
  dim3 grid(tiles_x, tiles_y, plan.zc);
  if (stencil25::SMEM_BYTES > 47 * 1024 && !g_dev[dev].stencil_smem.load()) {
    /* dynamic shared memory above the default limit: asked for once per device */
    if (int r = allow_smem(stencil25::tensor_kernel, stencil25::SMEM_BYTES)) return r;
    g_dev[dev].stencil_smem.store(true);
  }
  stencil25::tensor_kernel<<<grid, stencil25::COMPUTE_THREADS + stencil25::DMA_THREADS, stencil25::SMEM_BYTES, s>>>(
      *map, out, peer, sync, nx, ny, z_begin, z_end, plan.z_chunk, plan.z_edge, k);
  return launched();
}

/* copy between a plain nx x ny x nz array and one padded by four cells on every side */
int pad_copy(float *padded, float *plain, int nx, int ny, int nz, int z_begin, int z_end, bool to_padded,
             cudaStream_t s) {
  const int px = nx + 8, py = ny + 8;
  cudaMemcpy3DParms p;
  memset(&p, 0, sizeof(p));
  cudaPitchedPtr a = make_cudaPitchedPtr(plain, (size_t)nx * 4, (size_t)nx * 4, (size_t)ny);
  cudaPitchedPtr b = make_cudaPitchedPtr(padded, (size_t)px * 4, (size_t)px * 4, (size_t)py);
  const cudaPos pa = make_cudaPos(0, 0, (size_t)z_begin), pb = make_cudaPos(16, 4, (size_t)z_begin + 4);
  p.srcPtr = to_padded ? a : b; p.srcPos = to_padded ? pa : pb;
  p.dstPtr = to_padded ? b : a; p.dstPos = to_padded ? pb : pa;
  p.extent = make_cudaExtent((size_t)nx * 4, (size_t)ny, (size_t)(z_end - z_begin));
  p.kind = cudaMemcpyDeviceToDevice;
  CK(cudaMemcpy3DAsync(&p, s));
  return CUDADMA_OK;
}

/* `steps` steps of the portable kernel on padded copies of the field kept in the workspace */
int portable_stencil(float *a, float *b, int nx, int ny, int nz, int z_begin, int z_end, const float coeff[5],
                     int steps, int z_chunk, cudaStream_t s) {
  if (nx % portable::PS_TX || ny % portable::PS_TY) return CUDADMA_ERR_ARG;
  const size_t bytes = (size_t)(nx + 8) * (ny + 8) * (nz + 8) * 4;
  std::lock_guard<std::recursive_mutex> lock(g_ws_mutex);
  void *pa, *pb;
  if (int r = ws_get(2, bytes, &pa)) return r;
  if (int r = ws_get(3, bytes, &pb)) return r;
  CK(cudaMemsetAsync(pa, 0, bytes, s));
  CK(cudaMemsetAsync(pb, 0, bytes, s));
  if (int r = pad_copy((float *)pa, a, nx, ny, nz, 0, nz, true, s)) return r;
  float *cur = (float *)pa, *nxt = (float *)pb;
  for (int t = 0; t < steps; ++t) {
    if (int e = portable::launch_stencil_padded(nxt, cur, nx, ny, nz, z_begin, z_end, coeff, z_chunk, sm_count(), s)) {
      t_last_cuda_error = e;
      return CUDADMA_ERR_CUDA;
    }
    ++g_launches;
    float *tmp = cur; cur = nxt; nxt = tmp;
  }
  return pad_copy(cur, (steps & 1) ? b : a, nx, ny, nz, z_begin, z_end, false, s);
}

/* ---- host-buffer stencil run with copies and steps overlapped ----
 * The field goes up in pieces of `chunk` planes on one stream while a second stream steps and a
 * third brings finished planes down. After planes [0, Z) have arrived, step 1 can produce planes
 * below Z - 4, step 2 planes below Z - 8 and so on (each step needs four planes above its
 * output from the step before); once the whole field is up, every step runs on to the top.
 * Two arrays suffice: step t writes array t mod 2 only below the planes that step t - 1 still
 * has to read from it. Every plane is computed by the same kernel with the same operands as in
 * the plain run, so the result is bit-identical to it. */
int pipelined_stencil_host(float *h_out, const float *h_in, float *da, float *db, int nx, int ny, int nz,
                           const float coeff[5], int steps, int chunk, cudaStream_t s) {
  if (!g_ws_up) CK(cudaStreamCreateWithFlags(&g_ws_up, cudaStreamNonBlocking));
  if (!g_ws_down) CK(cudaStreamCreateWithFlags(&g_ws_down, cudaStreamNonBlocking));
  if (!g_ws_ev_up) CK(cudaEventCreateWithFlags(&g_ws_ev_up, cudaEventDisableTiming));
  if (!g_ws_ev_step) CK(cudaEventCreateWithFlags(&g_ws_ev_step, cudaEventDisableTiming));
  const size_t plane = (size_t)nx * ny;
  float *buf[2] = {da, db};
  const float *result = buf[steps & 1];
  const stencil25::Peers none{nullptr, 0, nullptr, 0};
  std::vector<int> done((size_t)steps + 1, 0); /* done[t]: planes [0, done[t]) hold the field after t steps */
  int down = 0;                               /* planes [0, down) are on their way to the host */
  while (done[0] < nz) {
    const int z0 = done[0], z1 = (nz - z0 < chunk) ? nz : z0 + chunk;
    CK(cudaMemcpyAsync(da + z0 * plane, h_in + z0 * plane, (size_t)(z1 - z0) * plane * 4, cudaMemcpyHostToDevice, g_ws_up));
    CK(cudaEventRecord(g_ws_ev_up, g_ws_up));
    CK(cudaStreamWaitEvent(s, g_ws_ev_up, 0));
    done[0] = z1;
    for (int t = 1; t <= steps; ++t) {
      int reach = done[t - 1] == nz ? nz : done[t - 1] - stencil25::R;
      if (reach <= done[t]) break; /* nothing new for this step, so nothing for the later ones */
      if (int r = launch_stencil_native(buf[t & 1], none, NO_SYNC, buf[(t - 1) & 1], nx, ny, nz, done[t], reach, coeff, 0, 0, s)) return r;
      done[t] = reach;
    }
    if (done[steps] > down) {
      CK(cudaEventRecord(g_ws_ev_step, s));
      CK(cudaStreamWaitEvent(g_ws_down, g_ws_ev_step, 0));
      CK(cudaMemcpyAsync(h_out + down * plane, result + down * plane, (size_t)(done[steps] - down) * plane * 4,
                         cudaMemcpyDeviceToHost, g_ws_down));
      down = done[steps];
    }
  }
  CK(cudaStreamSynchronize(g_ws_down));
  return finish_status(s);
}

}  // namespace

namespace {
/* One launch of the gather + scatter pipeline for records of RB bytes, 128 records per buffer. */
template <int RB, int STAGES>
int launch_gather_scatter(char *out, const char *table, const int32_t *gidx, const int32_t *sidx, long long nbuf,
                          int ctas_per_sm, int sms, cudaStream_t s) {
  using namespace cudadma_b200::kernels;
  constexpr int SMEM = STAGES * 128 * RB;
  auto k = gather_scatter_kernel<RB, 128, STAGES>;
  if (int r = allow_smem(k, SMEM)) return r;
  const int dev = current_device();
  if (dev < 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  std::atomic<int> &slot = g_dev[dev].gather_fit[RB == 16 ? 0 : RB == 32 ? 1 : RB == 64 ? 2 : 3];
  int fit = slot.load(); /* resident CTAs per SM of this instantiation on this device, asked once */
  if (fit == 0) {
    int f = 0;
    CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&f, k, GS_THREADS, SMEM));
    fit = f < 1 ? 1 : f;
    slot.store(fit);
  }
  const long long want = (long long)(fit < ctas_per_sm ? fit : ctas_per_sm) * sms;
  const int grid = (int)(nbuf < want ? nbuf : want);
  k<<<grid, GS_THREADS, SMEM, s>>>(out, table, gidx, sidx, nbuf);
  return launched();
}
}  // namespace

namespace {
/* Seeded synthetic inputs, stateless: element i is a function of seed + i (splitmix64), so a
 * field can be made in pieces, on any device, and comes out the same everywhere. */
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__global__ void fill_uniform_kernel(float *__restrict__ dst, const size_t n, const unsigned long long seed,
                                    const float lo, const float scale) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float u = (float)(splitmix64(seed + i) >> 40) * (1.0f / 16777216.0f);
    dst[i] = __fadd_rn(lo, __fmul_rn(scale, u)); /* two roundings, as the host generator does it */
  }
}
__global__ void fill_index_kernel(int32_t *__restrict__ dst, const size_t n, const unsigned long long seed,
                                  const unsigned int modulo) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = (int32_t)(splitmix64(seed + i) % modulo);
}
/* One thread spins for spin_ns of wall time and reports the SM cycles and nanoseconds that
 * passed: the SM clock under whatever runs beside it. */
__global__ void clock_probe_kernel(unsigned long long *out, const long long spin_ns) {
  unsigned long long t0, t1;
  const long long c0 = clock64();
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  do {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
  } while ((long long)(t1 - t0) < spin_ns);
  out[0] = (unsigned long long)(clock64() - c0);
  out[1] = t1 - t0;
}
}  // namespace

extern "C" {

int cudadma_version(void) { return 101; }

const char *cudadma_status_string(int status) {
  switch (status) {
    case CUDADMA_OK: return "ok";
    case CUDADMA_ERR_ARG: return "invalid argument";
    case CUDADMA_ERR_CUDA: return "CUDA call failed";
    case CUDADMA_ERR_UNSUPPORTED: return "implementation not available";
    case CUDADMA_ERR_NOMEM: return "out of device or pinned memory";
    case CUDADMA_ERR_TIMEOUT: return "a bounded wait inside the kernel gave up";
    case CUDADMA_ERR_TOO_LARGE: return "grid larger than the built-in scratch of the entry point that allocates nothing";
    default: return "unknown status";
  }
}
int cudadma_last_cuda_error(void) { return t_last_cuda_error; }
unsigned long long cudadma_launch_count(void) { return g_launches.load(); }

int cudadma_device_status(void *stream, unsigned int *out) {
  if (!out) return CUDADMA_ERR_ARG;
  CK(cudadma_b200::read_status(out, (cudaStream_t)stream));
  return CUDADMA_OK;
}

int cudadma_make_tensor_map_2d(void *out_map, const void *base, unsigned long long cols, unsigned long long rows,
                               unsigned long long row_pitch_bytes, unsigned int box_cols, unsigned int box_rows,
                               int swizzle_128b) {
  if (!out_map || !base || cols == 0 || rows == 0 || box_cols == 0 || box_rows == 0 || box_cols > 256 || box_rows > 256 ||
      !aligned16(base) || (row_pitch_bytes & 15) || row_pitch_bytes < cols * 4 || ((box_cols * 4) & 15) ||
      (swizzle_128b && box_cols * 4 > 128))
    return CUDADMA_ERR_ARG;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  return make_map_f32(static_cast<CUtensorMap *>(out_map), base, 2, dims, strides, box,
                      swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

int cudadma_make_tensor_map_3d(void *out_map, const void *base, unsigned long long nx, unsigned long long ny,
                               unsigned long long nz, unsigned long long row_pitch_bytes,
                               unsigned long long plane_pitch_bytes, unsigned int box_x, unsigned int box_y,
                               unsigned int box_z) {
  if (!out_map || !base || nx == 0 || ny == 0 || nz == 0 || box_x == 0 || box_y == 0 || box_z == 0 || box_x > 256 ||
      box_y > 256 || box_z > 256 || !aligned16(base) || (row_pitch_bytes & 15) || (plane_pitch_bytes & 15) ||
      row_pitch_bytes < nx * 4 || plane_pitch_bytes < row_pitch_bytes * ny || ((box_x * 4) & 15))
    return CUDADMA_ERR_ARG;
  const cuuint64_t dims[3] = {nx, ny, nz};
  const cuuint64_t strides[2] = {row_pitch_bytes, plane_pitch_bytes};
  const cuuint32_t box[3] = {box_x, box_y, box_z};
  return make_map_f32(static_cast<CUtensorMap *>(out_map), base, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

int cudadma_fill_uniform(float *dst, size_t n, unsigned long long seed, unsigned long long first_index, float lo,
                         float hi, void *stream) {
  if (!dst && n) return CUDADMA_ERR_ARG;
  if (n == 0) return CUDADMA_OK;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  fill_uniform_kernel<<<8 * sms, 256, 0, (cudaStream_t)stream>>>(dst, n, seed + first_index, lo, hi - lo);
  return launched();
}

int cudadma_fill_index(int32_t *dst, size_t n, unsigned long long seed, unsigned long long first_index,
                       unsigned int modulo, void *stream) {
  if ((!dst && n) || modulo == 0 || modulo > 0x80000000u) return CUDADMA_ERR_ARG;
  if (n == 0) return CUDADMA_OK;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  fill_index_kernel<<<8 * sms, 256, 0, (cudaStream_t)stream>>>(dst, n, seed + first_index, modulo);
  return launched();
}

int cudadma_clock_probe(unsigned long long *out, long long spin_ns, void *stream) {
  if (!out || spin_ns <= 0 || spin_ns > 100000000ll) return CUDADMA_ERR_ARG;
  clock_probe_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(out, spin_ns);
  return launched();
}

int cudadma_seq_copy(void *dst, const void *src, size_t bytes, int chunk_bytes, int impl, void *stream) {
  using namespace cudadma_b200::kernels;
  if (!dst || !src || (bytes & 3) || chunk_bytes < 16 || chunk_bytes > 16384 || (chunk_bytes & 15) ||
      !aligned16(dst) || !aligned16(src))
    return CUDADMA_ERR_ARG;
  if (bytes == 0) return CUDADMA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  const long long nfull = (long long)(bytes / (size_t)chunk_bytes);
  const int tail = (int)(bytes - (size_t)nfull * chunk_bytes);
  char *d = static_cast<char *>(dst);
  const char *p = static_cast<const char *>(src);
  if (nfull > 0) {
    if (impl == CUDADMA_IMPL_NATIVE && chunk_bytes == 16384) {
      constexpr int STAGES = SEQ_STAGES;
      auto k = seq_copy_kernel<16384, STAGES, SEQ_BULK_STORE>;
      if (int r = allow_smem(k, STAGES * 16384)) return r;
      const long long want = (long long)SEQ_CTAS_PER_SM * sms;
      const int grid = (int)(nfull < want ? nfull : want);
      k<<<grid, SEQ_DMA_THREADS + SEQ_COMPUTE_THREADS, STAGES * 16384, s>>>(d, p, nfull);
      if (int r = launched()) return r;
    } else if (impl == CUDADMA_IMPL_PORTABLE && chunk_bytes == 16384) {
      if (int r = portable::launch_seq_copy<P_SEQ_BPT>(d, p, nfull, sms, s)) { t_last_cuda_error = r; return CUDADMA_ERR_CUDA; }
      ++g_launches;
    } else if (impl == CUDADMA_IMPL_NATIVE || impl == CUDADMA_IMPL_PORTABLE) {
      const long long want = 4ll * sms;
      const int grid = (int)(nfull < want ? nfull : want);
      seq_copy_runtime_kernel<<<grid, SEQ_DMA_THREADS + SEQ_COMPUTE_THREADS, chunk_bytes, s>>>(d, p, nfull, chunk_bytes);
      if (int r = launched()) return r;
    } else {
      return CUDADMA_ERR_UNSUPPORTED;
    }
  }
  if (tail > 0) {
    seq_copy_runtime_kernel<<<1, SEQ_DMA_THREADS + SEQ_COMPUTE_THREADS, tail, s>>>(
        d + (size_t)nfull * chunk_bytes, p + (size_t)nfull * chunk_bytes, 1, tail);
    if (int r = launched()) return r;
  }
  return CUDADMA_OK;
}

int cudadma_strided_transpose(float *dst, const float *src, int rows, int cols, int impl, void *stream) {
  using namespace cudadma_b200::kernels;
  if (!dst || !src || rows <= 0 || cols <= 0 || (rows % TR_TILE_ROWS) || (cols % TR_TILE_COLS) || !aligned16(dst) ||
      !aligned16(src))
    return CUDADMA_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  const long long ntiles = (long long)(rows / TR_TILE_ROWS) * (cols / TR_TILE_COLS);
  if (impl == CUDADMA_IMPL_NATIVE) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
    const cuuint32_t box[2] = {TR_BOX_COLS, TR_TILE_ROWS};
    if (int r = make_map_f32(&map, src, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return r;
    constexpr int STAGES = TR_STAGES;
    constexpr int SMEM = STAGES * TR_TILE_BYTES + 1024;
    auto k = transpose_kernel<STAGES>;
    if (int r = allow_smem(k, SMEM)) return r;
    const long long want = (long long)TR_CTAS_PER_SM * sms;
    const int grid = (int)(ntiles < want ? ntiles : want);
    k<<<grid, TR_DMA_THREADS + TR_COMPUTE_THREADS, SMEM, s>>>(map, dst, rows, cols, cols * 4);
    return launched();
  }
  if (impl == CUDADMA_IMPL_PORTABLE) {
    if (int r = portable::launch_transpose(dst, src, rows, cols, sms, s)) { t_last_cuda_error = r; return CUDADMA_ERR_CUDA; }
    ++g_launches;
    return CUDADMA_OK;
  }
  return CUDADMA_ERR_UNSUPPORTED;
}

int cudadma_gather_scatter(void *out, const void *table, const int32_t *gather_idx, const int32_t *scatter_idx,
                           size_t n, int record_bytes, int impl, void *stream) {
  const bool size_ok = record_bytes == 16 || record_bytes == 32 || record_bytes == 64 || record_bytes == 128;
  if (!out || !table || !gather_idx || !scatter_idx || !size_ok || (n % 128) || !aligned16(out) ||
      !aligned16(table) || !aligned16(gather_idx) || !aligned16(scatter_idx))
    return CUDADMA_ERR_ARG;
  if (impl != CUDADMA_IMPL_NATIVE && impl != CUDADMA_IMPL_PORTABLE) return CUDADMA_ERR_UNSUPPORTED;
  if (n == 0) return CUDADMA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  const long long nbuf = (long long)(n / 128);
  char *o = static_cast<char *>(out);
  const char *t = static_cast<const char *>(table);
  if (impl == CUDADMA_IMPL_NATIVE) {
    /* ring depth: GS_STAGES buffers while a buffer is at most 8 KiB, half of that (at least two) for 16 KiB buffers */
    switch (record_bytes) {
      case 16: return launch_gather_scatter<16, GS_STAGES>(o, t, gather_idx, scatter_idx, nbuf, GS_CTAS_PER_SM, sms, s);
      case 32: return launch_gather_scatter<32, GS_STAGES>(o, t, gather_idx, scatter_idx, nbuf, GS_CTAS_PER_SM, sms, s);
      case 64: return launch_gather_scatter<64, GS_STAGES>(o, t, gather_idx, scatter_idx, nbuf, GS_CTAS_PER_SM, sms, s);
      default: return launch_gather_scatter<128, (GS_STAGES / 2 < 2 ? 2 : GS_STAGES / 2)>(o, t, gather_idx, scatter_idx, nbuf, GS_CTAS_PER_SM, sms, s);
    }
  }
  int r;
  switch (record_bytes) {
    case 16: r = portable::launch_gather_scatter<16>(o, t, gather_idx, scatter_idx, nbuf, sms, s); break;
    case 32: r = portable::launch_gather_scatter<32>(o, t, gather_idx, scatter_idx, nbuf, sms, s); break;
    case 64: r = portable::launch_gather_scatter<64>(o, t, gather_idx, scatter_idx, nbuf, sms, s); break;
    default: r = portable::launch_gather_scatter<128>(o, t, gather_idx, scatter_idx, nbuf, sms, s); break;
  }
  if (r) { t_last_cuda_error = r; return CUDADMA_ERR_CUDA; }
  ++g_launches;
  return CUDADMA_OK;
}

int cudadma_gather_scatter_tma(void *out, size_t out_records, const void *table, size_t table_records,
                               const int32_t *gather_idx, const int32_t *scatter_idx, size_t n, int record_bytes,
                               int mode, void *stream) {
  using namespace cudadma_b200::kernels;
  if (!out || !table || !gather_idx || !scatter_idx || record_bytes != 32 || (n % 128) || table_records == 0 ||
      table_records > 0x7fffffffull || out_records == 0 || out_records > 0x7fffffffull || mode < 1 || mode > 3 ||
      !aligned16(out) || !aligned16(table) || !aligned16(gather_idx) || !aligned16(scatter_idx))
    return CUDADMA_ERR_ARG;
  if (n == 0) return CUDADMA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  const long long nbuf = (long long)(n / 128);
  /* table and output as 2-D tensors [records][8 floats] whose box is one record: each TMA
   * instruction of the gather (scatter) object names four records */
  CUtensorMap tmap, omap;
  const cuuint64_t tdims[2] = {8, (cuuint64_t)table_records}, odims[2] = {8, (cuuint64_t)out_records};
  const cuuint64_t strides[1] = {32};
  const cuuint32_t box[2] = {8, 1};
  if (int r = make_map_f32(&tmap, table, 2, tdims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE))
    return r;
  if (int r = make_map_f32(&omap, out, 2, odims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE))
    return r;
  constexpr int STAGES = GS_STAGES;
  constexpr int SMEM = STAGES * 128 * 32;
  const long long want = (long long)GS_CTAS_PER_SM * sms;
  const int grid = (int)(nbuf < want ? nbuf : want);
  char *o = static_cast<char *>(out);
  const char *t = static_cast<const char *>(table);
#define CUDADMA_LAUNCH_G4S4(G4, S4)                                                                     \
  do {                                                                                                  \
    auto k = gather4_scatter_kernel<32, 128, STAGES, G4, S4>;                                           \
    if (int r = allow_smem(k, SMEM)) return r;                                                          \
    k<<<grid, GS_THREADS, SMEM, s>>>(tmap, omap, o, t, gather_idx, scatter_idx, nbuf);                  \
  } while (0)
  if (mode == 1) CUDADMA_LAUNCH_G4S4(true, false);
  else if (mode == 2) CUDADMA_LAUNCH_G4S4(false, true);
  else CUDADMA_LAUNCH_G4S4(true, true);
#undef CUDADMA_LAUNCH_G4S4
  return launched();
}

int cudadma_stencil25_step(float *out, const float *in, int nx, int ny, int nz, int z_begin, int z_end,
                           const float coeff[5], int z_chunk, int impl, void *stream) {
  if (!out || !in || !coeff || nx <= 0 || ny <= 0 || nz <= 0 || (nx & 3) || z_begin < 0 || z_end > nz ||
      z_begin > z_end || !aligned16(out) || !aligned16(in) || out == in)
    return CUDADMA_ERR_ARG;
  if (z_begin == z_end) return CUDADMA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  if (impl == CUDADMA_IMPL_PORTABLE)
    return portable_stencil(const_cast<float *>(in), out, nx, ny, nz, z_begin, z_end, coeff, 1, z_chunk, s);
  if (impl != CUDADMA_IMPL_NATIVE) return CUDADMA_ERR_UNSUPPORTED;
  return launch_stencil_native(out, stencil25::Peers{nullptr, 0, nullptr, 0}, NO_SYNC, in, nx, ny, nz, z_begin, z_end, coeff,
                               z_chunk, 0, s);
}

int cudadma_stencil25_run(float *a, float *b, int nx, int ny, int nz, const float coeff[5], int steps, int impl,
                          void *stream) {
  if (steps < 0) return CUDADMA_ERR_ARG;
  if (impl == CUDADMA_IMPL_PORTABLE) {
    if (!a || !b || !coeff || nx <= 0 || ny <= 0 || nz <= 0) return CUDADMA_ERR_ARG;
    if (sm_count() <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
    return portable_stencil(a, b, nx, ny, nz, 0, nz, coeff, steps, 0, (cudaStream_t)stream);
  }
  float *cur = a, *nxt = b;
  for (int t = 0; t < steps; ++t) {
    if (int r = cudadma_stencil25_step(nxt, cur, nx, ny, nz, 0, nz, coeff, 0, impl, stream)) return r;
    float *tmp = cur; cur = nxt; nxt = tmp;
  }
  return CUDADMA_OK;
}

int cudadma_stencil25_step_padded(float *out, const float *in, int nx, int ny, int nz, int z_begin, int z_end,
                                  const float coeff[5], int z_chunk, int impl, void *stream) {
  if (!out || !in || !coeff || nx <= 0 || ny <= 0 || nz <= 0 || (nx % portable::PS_TX) || (ny % portable::PS_TY) ||
      z_begin < 0 || z_end > nz || z_begin > z_end || !aligned16(out) || !aligned16(in) || out == in)
    return CUDADMA_ERR_ARG;
  if (impl != CUDADMA_IMPL_PORTABLE) return CUDADMA_ERR_UNSUPPORTED;
  if (z_begin == z_end) return CUDADMA_OK;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  if (int e = portable::launch_stencil_padded(out, in, nx, ny, nz, z_begin, z_end, coeff, z_chunk, sms,
                                              (cudaStream_t)stream)) {
    t_last_cuda_error = e;
    return CUDADMA_ERR_CUDA;
  }
  ++g_launches;
  return CUDADMA_OK;
}

/* ---- z-sharded stencil with halo planes pushed straight into the neighbour GPUs ---- */

}  /* extern "C" */

namespace {

struct SlabHandles {            /* what a rank publishes to its z-neighbours */
  cudaIpcMemHandle_t buf[2];
  cudaIpcMemHandle_t flags;
  int nzl;
};

constexpr long long SLAB_WAIT_LIMIT_CYCLES = 1ll << 32; /* about two seconds */
constexpr int SLAB_EDGE_PLANES = 32;                    /* depth of the two boundary runs of a slab step */
#ifndef SLAB_HIGHEST_FIRST
#define SLAB_HIGHEST_FIRST true
#endif
#ifndef CUDADMA_SLAB_SIGNAL_DEFAULT
#define CUDADMA_SLAB_SIGNAL_DEFAULT CUDADMA_SLAB_SIGNAL_TRAILING
#endif

/* CUDADMA_SLAB_SIGNAL_TRAILING: one thread, launched behind the step's kernel, publishes the step
 * count. Everything the kernel wrote -- its own planes and the copies stored into the neighbours'
 * ghost planes -- is complete when this launch starts; the system-scope fence and release stores
 * order it before the flags. After a wait of the step gave up nothing is published. */
__global__ void slab_signal_kernel(unsigned int *peer_lo, unsigned int *peer_hi, const unsigned int value,
                                   unsigned int *failed) {
  const unsigned int w = *reinterpret_cast<volatile unsigned int *>(&cudadma_b200::g_status_word);
  if (w != 0u) { atomicCAS(failed, 0u, w); return; }
  if (*reinterpret_cast<volatile unsigned int *>(failed) != 0u) return;
  __threadfence_system();
  if (peer_lo) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_lo), "r"(value) : "memory");
  if (peer_hi) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_hi), "r"(value) : "memory");
}

struct Slab {
  int device;
  int nx, ny, nzl;
  bool has_lo, has_hi;
  float *buf[2];                /* (nzl + 8) planes each: four ghost planes, the owned planes, four ghost planes */
  unsigned int *flags;          /* [0] steps finished by the lower neighbour, [1] by the upper one (they write);
                                   [2] ticket of the boundary CTAs; [3] this rank's failure word */
  float *lo_buf[2], *hi_buf[2]; /* the neighbours' arrays, mapped into this process (or theirs, same process) */
  unsigned int *lo_flags, *hi_flags;
  bool lo_ipc, hi_ipc;          /* mapped with CUDA IPC (to be closed), or plain pointers of this process */
  int nzl_lo;                   /* planes the lower neighbour owns */
  int cur;                      /* buf[cur] holds the current field */
  unsigned int step;            /* steps finished */
  long long wait_limit;         /* SM cycles a boundary CTA waits for a neighbour */
  int edge;                     /* depth of the two boundary runs of a step (0: equal runs) */
  int signal_mode;              /* CUDADMA_SLAB_SIGNAL_*: who publishes the step count */
  bool highest_first;           /* trailing mode: dispatch the runs of planes from the top down */
  bool failed;                  /* a failure word was read back: no further steps */
};

}  // namespace

extern "C" {

int cudadma_slab_create(void **out, int nx, int ny, int nzl, int has_lower, int has_upper) {
  if (!out || nx <= 0 || ny <= 0 || (nx & 3) || nzl <= 0 || ((has_lower || has_upper) && nzl < 8)) return CUDADMA_ERR_ARG;
  const int dev = current_device();
  if (dev < 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  Slab *sl = new Slab();
  sl->device = dev;
  sl->nx = nx; sl->ny = ny; sl->nzl = nzl;
  sl->has_lo = has_lower != 0; sl->has_hi = has_upper != 0;
  sl->wait_limit = SLAB_WAIT_LIMIT_CYCLES;
  sl->edge = SLAB_EDGE_PLANES;
  sl->signal_mode = CUDADMA_SLAB_SIGNAL_DEFAULT;
  sl->highest_first = SLAB_HIGHEST_FIRST;
  const size_t bytes = (size_t)nx * ny * (nzl + 8) * sizeof(float);
  cudaError_t e = cudaMalloc(&sl->buf[0], bytes);
  if (e == cudaSuccess) e = cudaMalloc(&sl->buf[1], bytes);
  if (e == cudaSuccess) e = cudaMalloc(&sl->flags, 256);
  if (e == cudaSuccess) e = cudaMemset(sl->buf[0], 0, bytes);
  if (e == cudaSuccess) e = cudaMemset(sl->buf[1], 0, bytes);
  if (e == cudaSuccess) e = cudaMemset(sl->flags, 0, 256);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    t_last_cuda_error = (int)e;
    cudaFree(sl->buf[0]); cudaFree(sl->buf[1]); cudaFree(sl->flags);
    delete sl;
    cudaGetLastError();
    return e == cudaErrorMemoryAllocation ? CUDADMA_ERR_NOMEM : CUDADMA_ERR_CUDA;
  }
  *out = sl;
  return CUDADMA_OK;
}

size_t cudadma_slab_handle_bytes(void) { return sizeof(SlabHandles); }

int cudadma_slab_export(void *slab, void *handles) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || !handles) return CUDADMA_ERR_ARG;
  SlabHandles h;
  memset(&h, 0, sizeof(h));
  CK(cudaIpcGetMemHandle(&h.buf[0], sl->buf[0]));
  CK(cudaIpcGetMemHandle(&h.buf[1], sl->buf[1]));
  CK(cudaIpcGetMemHandle(&h.flags, sl->flags));
  h.nzl = sl->nzl;
  memcpy(handles, &h, sizeof(h));
  return CUDADMA_OK;
}

int cudadma_slab_connect(void *slab, const void *lower_handles, const void *upper_handles) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || (sl->has_lo && !lower_handles) || (sl->has_hi && !upper_handles)) return CUDADMA_ERR_ARG;
  if (sl->has_lo) {
    SlabHandles h;
    memcpy(&h, lower_handles, sizeof(h));
    CK(cudaIpcOpenMemHandle((void **)&sl->lo_buf[0], h.buf[0], cudaIpcMemLazyEnablePeerAccess));
    CK(cudaIpcOpenMemHandle((void **)&sl->lo_buf[1], h.buf[1], cudaIpcMemLazyEnablePeerAccess));
    CK(cudaIpcOpenMemHandle((void **)&sl->lo_flags, h.flags, cudaIpcMemLazyEnablePeerAccess));
    sl->nzl_lo = h.nzl;
    sl->lo_ipc = true;
  }
  if (sl->has_hi) {
    SlabHandles h;
    memcpy(&h, upper_handles, sizeof(h));
    CK(cudaIpcOpenMemHandle((void **)&sl->hi_buf[0], h.buf[0], cudaIpcMemLazyEnablePeerAccess));
    CK(cudaIpcOpenMemHandle((void **)&sl->hi_buf[1], h.buf[1], cudaIpcMemLazyEnablePeerAccess));
    CK(cudaIpcOpenMemHandle((void **)&sl->hi_flags, h.flags, cudaIpcMemLazyEnablePeerAccess));
    sl->hi_ipc = true;
  }
  return CUDADMA_OK;
}

int cudadma_slab_connect_local(void *slab, void *lower_slab, void *upper_slab) {
  Slab *sl = static_cast<Slab *>(slab);
  Slab *lo = static_cast<Slab *>(lower_slab), *hi = static_cast<Slab *>(upper_slab);
  if (!sl || (sl->has_lo && !lo) || (sl->has_hi && !hi)) return CUDADMA_ERR_ARG;
  if ((sl->has_lo && (lo->nx != sl->nx || lo->ny != sl->ny)) || (sl->has_hi && (hi->nx != sl->nx || hi->ny != sl->ny)))
    return CUDADMA_ERR_ARG;
  int before = -1;
  CK(cudaGetDevice(&before));
  CK(cudaSetDevice(sl->device));
  Slab *nb[2] = {sl->has_lo ? lo : nullptr, sl->has_hi ? hi : nullptr};
  for (int i = 0; i < 2; ++i) {
    if (!nb[i] || nb[i]->device == sl->device) continue;
    int can = 0;
    cudaError_t e = cudaDeviceCanAccessPeer(&can, sl->device, nb[i]->device);
    if (e == cudaSuccess && !can) e = cudaErrorPeerAccessUnsupported;
    if (e == cudaSuccess) {
      e = cudaDeviceEnablePeerAccess(nb[i]->device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) { e = cudaSuccess; cudaGetLastError(); }
    }
    if (e != cudaSuccess) { t_last_cuda_error = (int)e; cudaSetDevice(before); return CUDADMA_ERR_CUDA; }
  }
  if (sl->has_lo) {
    sl->lo_buf[0] = lo->buf[0]; sl->lo_buf[1] = lo->buf[1]; sl->lo_flags = lo->flags; sl->nzl_lo = lo->nzl;
    sl->lo_ipc = false;
  }
  if (sl->has_hi) {
    sl->hi_buf[0] = hi->buf[0]; sl->hi_buf[1] = hi->buf[1]; sl->hi_flags = hi->flags;
    sl->hi_ipc = false;
  }
  CK(cudaSetDevice(before));
  return CUDADMA_OK;
}

int cudadma_slab_set_wait_limit(void *slab, long long sm_cycles) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || sm_cycles <= 0) return CUDADMA_ERR_ARG;
  sl->wait_limit = sm_cycles;
  return CUDADMA_OK;
}

int cudadma_slab_set_edge_planes(void *slab, int planes) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || planes < 0 || (planes > 0 && planes < 8)) return CUDADMA_ERR_ARG;
  sl->edge = planes;
  return CUDADMA_OK;
}

int cudadma_slab_set_run_order(void *slab, int highest_first) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || highest_first < 0 || highest_first > 1) return CUDADMA_ERR_ARG;
  sl->highest_first = highest_first != 0;
  return CUDADMA_OK;
}

int cudadma_slab_set_signal_mode(void *slab, int mode) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || (mode != CUDADMA_SLAB_SIGNAL_TRAILING && mode != CUDADMA_SLAB_SIGNAL_FUSED)) return CUDADMA_ERR_ARG;
  sl->signal_mode = mode;
  return CUDADMA_OK;
}

int cudadma_slab_buffer(void *slab, int which, float **ptr) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || !ptr || which < 0 || which > 1) return CUDADMA_ERR_ARG;
  *ptr = sl->buf[which ? (sl->cur ^ 1) : sl->cur];
  return CUDADMA_OK;
}

int cudadma_slab_step(void *slab, const float coeff[5], void *stream) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl || !coeff) return CUDADMA_ERR_ARG;
  if (sl->failed) return CUDADMA_ERR_TIMEOUT;
  cudaStream_t s = (cudaStream_t)stream;
  const int nx = sl->nx, ny = sl->ny, nzl = sl->nzl, nzt = nzl + 8;
  const long long pz = (long long)nx * ny;
  float *cur = sl->buf[sl->cur], *nxt = sl->buf[sl->cur ^ 1];
  const int first = 4, last = 4 + nzl;
  /* One launch for all owned planes. The first and last four are stored twice, here and in the
   * neighbour's ghost planes: plane z of this rank is plane z + nzl_lo of the lower neighbour
   * (its upper ghost planes) and plane z - nzl of the upper neighbour (its lower ghost planes).
   * The CTAs at a shared boundary first wait until that neighbour has finished the previous step
   * (its copies of it are in this rank's ghost planes, and it no longer reads the ghost planes
   * this step overwrites); the last of them to finish publishes this rank's step count. */
  stencil25::Peers peer = {nullptr, 0, nullptr, 0};
  stencil25::Sync sync = NO_SYNC;
  if (sl->has_lo) { peer.lo = sl->lo_buf[sl->cur ^ 1] + (long long)sl->nzl_lo * pz; peer.lo_end = first + 4; }
  if (sl->has_hi) { peer.hi = sl->hi_buf[sl->cur ^ 1] - (long long)nzl * pz; peer.hi_begin = last - 4; }
  const bool sharded = sl->has_lo || sl->has_hi;
  const bool fused = sl->signal_mode == CUDADMA_SLAB_SIGNAL_FUSED;
  if (sharded) {
    sync.wait_lo = sl->has_lo ? sl->flags + 0 : nullptr;
    sync.wait_hi = sl->has_hi ? sl->flags + 1 : nullptr;
    sync.signal_lo = sl->has_lo ? sl->lo_flags + 1 : nullptr;
    sync.signal_hi = sl->has_hi ? sl->hi_flags + 0 : nullptr;
    sync.ticket = fused ? sl->flags + 2 : nullptr;
    sync.failed = sl->flags + 3;
    sync.step = sl->step;
    sync.wait_limit = sl->wait_limit;
  }
  /* boundary runs of their own only pay where they let the step count go out early */
  if (int r = launch_stencil_native(nxt, peer, sync, cur, nx, ny, nzt, first, last, coeff, 0,
                                    !sharded ? 0 : fused ? sl->edge : (sl->highest_first ? -1 : 0), s))
    return r;
  if (sharded && !fused) {
    slab_signal_kernel<<<1, 1, 0, s>>>(sync.signal_lo, sync.signal_hi, sl->step + 1, sl->flags + 3);
    if (int r = launched()) return r;
  }
  sl->cur ^= 1;
  sl->step += 1;
  return CUDADMA_OK;
}

int cudadma_slab_status(void *slab, void *stream) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl) return CUDADMA_ERR_ARG;
  unsigned int w = 0;
  CK(cudaMemcpyAsync(&w, sl->flags + 3, sizeof(w), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  CK(cudaStreamSynchronize((cudaStream_t)stream));
  if (w != 0) sl->failed = true;
  return sl->failed ? CUDADMA_ERR_TIMEOUT : CUDADMA_OK;
}

int cudadma_slab_destroy(void *slab) {
  Slab *sl = static_cast<Slab *>(slab);
  if (!sl) return CUDADMA_OK;
  int before = -1;
  cudaGetDevice(&before);
  cudaSetDevice(sl->device);
  cudaDeviceSynchronize();
  if (sl->has_lo && sl->lo_ipc) { cudaIpcCloseMemHandle(sl->lo_buf[0]); cudaIpcCloseMemHandle(sl->lo_buf[1]); cudaIpcCloseMemHandle(sl->lo_flags); }
  if (sl->has_hi && sl->hi_ipc) { cudaIpcCloseMemHandle(sl->hi_buf[0]); cudaIpcCloseMemHandle(sl->hi_buf[1]); cudaIpcCloseMemHandle(sl->hi_flags); }
  cudaFree(sl->buf[0]); cudaFree(sl->buf[1]); cudaFree(sl->flags);
  delete sl;
  cudaGetLastError();
  if (before >= 0) cudaSetDevice(before);
  return CUDADMA_OK;
}

/* ---- the sharded stencil driven from one process: one slab and one stream per GPU ---- */

}  /* extern "C" */

namespace {
struct Multi {
  int n, nx, ny, nz;
  std::vector<int> device, z_lo, z_hi;
  std::vector<Slab *> slab;
  std::vector<cudaStream_t> stream;   /* one per distinct device: slabs that share a GPU share its stream */
};

/* planes [lo, hi) of part r of n: as even as possible, earlier parts take the remainder */
void even_cut(int nz, int n, int r, int *lo, int *hi) {
  const int base = nz / n, rem = nz % n;
  *lo = r * base + (r < rem ? r : rem);
  *hi = *lo + base + (r < rem ? 1 : 0);
}

struct DeviceGuard {   /* puts the caller's current device back */
  int before;
  DeviceGuard() : before(-1) { cudaGetDevice(&before); }
  ~DeviceGuard() { if (before >= 0) cudaSetDevice(before); }
};
}  // namespace

extern "C" {

int cudadma_stencil25_multi_destroy(void *handle) {
  Multi *m = static_cast<Multi *>(handle);
  if (!m) return CUDADMA_OK;
  DeviceGuard guard;
  for (size_t i = 0; i < m->slab.size(); ++i) {
    if (m->stream[i]) { cudaSetDevice(m->device[i]); cudaStreamSynchronize(m->stream[i]); }
  }
  for (size_t i = 0; i < m->slab.size(); ++i) cudadma_slab_destroy(m->slab[i]);
  for (size_t i = 0; i < m->stream.size(); ++i) {
    bool first = true;
    for (size_t j = 0; j < i; ++j) if (m->stream[j] == m->stream[i]) first = false;
    if (first && m->stream[i]) { cudaSetDevice(m->device[i]); cudaStreamDestroy(m->stream[i]); }
  }
  delete m;
  cudaGetLastError();
  return CUDADMA_OK;
}

int cudadma_stencil25_multi_create(void **out, int n_gpus, const int *devices, int nx, int ny, int nz) {
  if (!out || n_gpus < 1 || n_gpus > MAX_DEVICES || nx <= 0 || ny <= 0 || nz <= 0 || (nx & 3) ||
      (n_gpus > 1 && nz / n_gpus < 8))
    return CUDADMA_ERR_ARG;
  DeviceGuard guard;
  Multi *m = new Multi();
  m->n = n_gpus; m->nx = nx; m->ny = ny; m->nz = nz;
  int status = CUDADMA_OK;
  for (int r = 0; r < n_gpus && status == CUDADMA_OK; ++r) {
    const int dev = devices ? devices[r] : r;
    int lo, hi;
    even_cut(nz, n_gpus, r, &lo, &hi);
    cudaError_t e = cudaSetDevice(dev);
    if (e != cudaSuccess) { t_last_cuda_error = (int)e; status = CUDADMA_ERR_CUDA; break; }
    void *sl = nullptr;
    status = cudadma_slab_create(&sl, nx, ny, hi - lo, r > 0, r < n_gpus - 1);
    if (status != CUDADMA_OK) break;
    cudaStream_t st = nullptr;
    for (int j = 0; j < r; ++j) if (m->device[j] == dev) st = m->stream[j];
    if (!st) {
      e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
      if (e != cudaSuccess) { t_last_cuda_error = (int)e; status = CUDADMA_ERR_CUDA; cudadma_slab_destroy(sl); break; }
    }
    m->device.push_back(dev); m->z_lo.push_back(lo); m->z_hi.push_back(hi);
    m->slab.push_back(static_cast<Slab *>(sl)); m->stream.push_back(st);
  }
  for (int r = 0; r < n_gpus && status == CUDADMA_OK; ++r)
    status = cudadma_slab_connect_local(m->slab[r], r > 0 ? m->slab[r - 1] : nullptr, r < n_gpus - 1 ? m->slab[r + 1] : nullptr);
  if (status != CUDADMA_OK) { cudadma_stencil25_multi_destroy(m); return status; }
  *out = m;
  return CUDADMA_OK;
}

int cudadma_stencil25_multi_load(void *handle, const float *h_field) {
  Multi *m = static_cast<Multi *>(handle);
  if (!m || !h_field) return CUDADMA_ERR_ARG;
  DeviceGuard guard;
  const size_t plane = (size_t)m->nx * m->ny;
  for (int r = 0; r < m->n; ++r) {
    Slab *sl = m->slab[r];
    CK(cudaSetDevice(m->device[r]));
    CK(cudaStreamSynchronize(m->stream[r]));
    const size_t bytes = plane * (sl->nzl + 8) * sizeof(float);
    CK(cudaMemsetAsync(sl->buf[0], 0, bytes, m->stream[r]));
    CK(cudaMemsetAsync(sl->buf[1], 0, bytes, m->stream[r]));
    CK(cudaMemsetAsync(sl->flags, 0, 256, m->stream[r]));
    /* owned planes and the ghost planes that lie inside the grid, straight from the whole field */
    const int g0 = m->z_lo[r] - 4 < 0 ? 0 : m->z_lo[r] - 4, g1 = m->z_hi[r] + 4 > m->nz ? m->nz : m->z_hi[r] + 4;
    CK(cudaMemcpyAsync(sl->buf[0] + (size_t)(g0 - (m->z_lo[r] - 4)) * plane, h_field + (size_t)g0 * plane,
                       (size_t)(g1 - g0) * plane * sizeof(float), cudaMemcpyHostToDevice, m->stream[r]));
    sl->cur = 0; sl->step = 0; sl->failed = false;
  }
  for (int r = 0; r < m->n; ++r) { CK(cudaSetDevice(m->device[r])); CK(cudaStreamSynchronize(m->stream[r])); }
  return CUDADMA_OK;
}

int cudadma_stencil25_multi_run(void *handle, const float coeff[5], int steps) {
  Multi *m = static_cast<Multi *>(handle);
  if (!m || !coeff || steps < 0) return CUDADMA_ERR_ARG;
  DeviceGuard guard;
  for (int t = 0; t < steps; ++t)
    for (int r = 0; r < m->n; ++r) {
      CK(cudaSetDevice(m->device[r]));
      if (int e = cudadma_slab_step(m->slab[r], coeff, m->stream[r])) return e;
    }
  int status = CUDADMA_OK;
  for (int r = 0; r < m->n; ++r) {
    CK(cudaSetDevice(m->device[r]));
    const int e = cudadma_slab_status(m->slab[r], m->stream[r]);
    const int w = finish_status(m->stream[r]); /* waits inside the objects (the device's status word) */
    if (e != CUDADMA_OK && status == CUDADMA_OK) status = e;
    if (w != CUDADMA_OK && status == CUDADMA_OK) status = w;
  }
  return status;
}

int cudadma_stencil25_multi_store(void *handle, float *h_field) {
  Multi *m = static_cast<Multi *>(handle);
  if (!m || !h_field) return CUDADMA_ERR_ARG;
  DeviceGuard guard;
  const size_t plane = (size_t)m->nx * m->ny;
  for (int r = 0; r < m->n; ++r) {
    Slab *sl = m->slab[r];
    CK(cudaSetDevice(m->device[r]));
    CK(cudaMemcpyAsync(h_field + (size_t)m->z_lo[r] * plane, sl->buf[sl->cur] + 4 * plane,
                       (size_t)sl->nzl * plane * sizeof(float), cudaMemcpyDeviceToHost, m->stream[r]));
  }
  for (int r = 0; r < m->n; ++r) { CK(cudaSetDevice(m->device[r])); CK(cudaStreamSynchronize(m->stream[r])); }
  return CUDADMA_OK;
}

int cudadma_stencil25_multi_slab(void *handle, int rank, void **slab, int *z_lo, int *z_hi) {
  Multi *m = static_cast<Multi *>(handle);
  if (!m || rank < 0 || rank >= m->n) return CUDADMA_ERR_ARG;
  if (slab) *slab = m->slab[rank];
  if (z_lo) *z_lo = m->z_lo[rank];
  if (z_hi) *z_hi = m->z_hi[rank];
  return CUDADMA_OK;
}

/* ---- host-buffer forms ---- */

int cudadma_seq_copy_host(void *h_dst, const void *h_src, size_t bytes, int chunk_bytes, int impl) {
  if (!h_dst || !h_src) return CUDADMA_ERR_ARG;
  std::lock_guard<std::recursive_mutex> lock(g_ws_mutex);
  cudaStream_t s; void *din, *dout;
  if (int r = ws_stream(&s)) return r;
  if (int r = ws_get(0, bytes, &din)) return r;
  if (int r = ws_get(1, bytes, &dout)) return r;
  CK(cudaMemcpyAsync(din, h_src, bytes, cudaMemcpyHostToDevice, s));
  if (int r = cudadma_seq_copy(dout, din, bytes, chunk_bytes, impl, s)) return r;
  CK(cudaMemcpyAsync(h_dst, dout, bytes, cudaMemcpyDeviceToHost, s));
  return finish_status(s);
}

int cudadma_strided_transpose_host(float *h_dst, const float *h_src, int rows, int cols, int impl) {
  if (!h_dst || !h_src || rows <= 0 || cols <= 0) return CUDADMA_ERR_ARG;
  const size_t bytes = (size_t)rows * cols * 4;
  std::lock_guard<std::recursive_mutex> lock(g_ws_mutex);
  cudaStream_t s; void *din, *dout;
  if (int r = ws_stream(&s)) return r;
  if (int r = ws_get(0, bytes, &din)) return r;
  if (int r = ws_get(1, bytes, &dout)) return r;
  CK(cudaMemcpyAsync(din, h_src, bytes, cudaMemcpyHostToDevice, s));
  if (int r = cudadma_strided_transpose((float *)dout, (const float *)din, rows, cols, impl, s)) return r;
  CK(cudaMemcpyAsync(h_dst, dout, bytes, cudaMemcpyDeviceToHost, s));
  return finish_status(s);
}

int cudadma_gather_scatter_host(void *h_out, size_t out_records, const void *h_table, size_t table_records,
                                const int32_t *h_gather_idx, const int32_t *h_scatter_idx, size_t n,
                                int record_bytes, int impl) {
  if (!h_out || !h_table || !h_gather_idx || !h_scatter_idx || record_bytes <= 0) return CUDADMA_ERR_ARG;
  std::lock_guard<std::recursive_mutex> lock(g_ws_mutex);
  cudaStream_t s; void *dtab, *dout, *dg, *ds;
  if (int r = ws_stream(&s)) return r;
  if (int r = ws_get(0, table_records * record_bytes, &dtab)) return r;
  if (int r = ws_get(1, out_records * record_bytes, &dout)) return r;
  if (int r = ws_get(2, n * 4, &dg)) return r;
  if (int r = ws_get(3, n * 4, &ds)) return r;
  CK(cudaMemcpyAsync(dtab, h_table, table_records * record_bytes, cudaMemcpyHostToDevice, s));
  CK(cudaMemcpyAsync(dg, h_gather_idx, n * 4, cudaMemcpyHostToDevice, s));
  CK(cudaMemcpyAsync(ds, h_scatter_idx, n * 4, cudaMemcpyHostToDevice, s));
  /* slots no index names keep the caller's bytes */
  CK(cudaMemcpyAsync(dout, h_out, out_records * record_bytes, cudaMemcpyHostToDevice, s));
  if (int r = cudadma_gather_scatter(dout, dtab, (const int32_t *)dg, (const int32_t *)ds, n, record_bytes, impl, s))
    return r;
  CK(cudaMemcpyAsync(h_out, dout, out_records * record_bytes, cudaMemcpyDeviceToHost, s));
  return finish_status(s);
}

int cudadma_stencil25_run_host(float *h_out, const float *h_in, int nx, int ny, int nz, const float coeff[5],
                               int steps, int impl) {
  return cudadma_stencil25_run_host_pipelined(h_out, h_in, nx, ny, nz, coeff, steps, impl, 0);
}

int cudadma_stencil25_run_host_pipelined(float *h_out, const float *h_in, int nx, int ny, int nz,
                                         const float coeff[5], int steps, int impl, int chunk_planes) {
  if (!h_out || !h_in || !coeff || nx <= 0 || ny <= 0 || nz <= 0 || steps < 0 || chunk_planes < 0) return CUDADMA_ERR_ARG;
  if (impl != CUDADMA_IMPL_NATIVE && impl != CUDADMA_IMPL_PORTABLE) return CUDADMA_ERR_UNSUPPORTED;
  const size_t plane_bytes = (size_t)nx * ny * 4;
  const size_t bytes = plane_bytes * nz;
  std::lock_guard<std::recursive_mutex> lock(g_ws_mutex);
  cudaStream_t s; void *da, *db;
  if (int r = ws_stream(&s)) return r;
  if (int r = ws_get(0, bytes, &da)) return r;
  if (int r = ws_get(1, bytes, &db)) return r;
  bool pipeline = impl == CUDADMA_IMPL_NATIVE && steps > 0 && !(nx & 3);
  if (pipeline && chunk_planes == 0) {
    /* the library's choice: pieces of HOST_PIPE_CHUNK_BYTES, and only where the wave of steps
     * (four planes behind the upload per step) is short against the grid, so that copies and
     * steps can overlap at all */
    size_t c = HOST_PIPE_CHUNK_BYTES / plane_bytes;
    chunk_planes = c < 16 ? 16 : (int)c;
    pipeline = (long long)nz >= 4ll * chunk_planes && 8ll * steps <= nz;
  }
  if (!pipeline) {
    CK(cudaMemcpyAsync(da, h_in, bytes, cudaMemcpyHostToDevice, s));
    if (int r = cudadma_stencil25_run((float *)da, (float *)db, nx, ny, nz, coeff, steps, impl, s)) return r;
    CK(cudaMemcpyAsync(h_out, (steps & 1) ? db : da, bytes, cudaMemcpyDeviceToHost, s));
    return finish_status(s);
  }
  const int r = pipelined_stencil_host(h_out, h_in, (float *)da, (float *)db, nx, ny, nz, coeff, steps, chunk_planes, s);
  if (r < 0) { /* leave nothing of this call in flight behind an error */
    cudaStreamSynchronize(g_ws_up); cudaStreamSynchronize(s); cudaStreamSynchronize(g_ws_down);
  }
  return r;
}

/* ---- the entry point that allocates nothing ---- */

}  /* extern "C" */

namespace {
/* Scratch of cudadma_stencil25_step_noalloc: two padded copies of the field, side by side.
 * It is part of the library image, so every GPU that loads the library holds these 16 MiB
 * until the process exits, used or not. */
constexpr size_t NOALLOC_MAX_FLOATS = (size_t)1 << 21; /* per padded array */
static __device__ __align__(256) float g_noalloc_scratch[2 * NOALLOC_MAX_FLOATS];

/* In host code the name g_noalloc_scratch is only a handle for the runtime, not a device
 * address: the address is asked for once per device, with that device current. */
constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mutex;
float *g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

int noalloc_scratch(float **out) {
  int dev = -1;
  CK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return CUDADMA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void *p = nullptr;
    CK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    g_noalloc_ptr[dev] = static_cast<float *>(p);
  }
  *out = g_noalloc_ptr[dev];
  return CUDADMA_OK;
}
}  // namespace

extern "C" {

int cudadma_stencil25_step_noalloc(float *out, const float *in, int nx, int ny, int nz, const float coeff[5],
                                   void *stream) {
  if (!out || !in || !coeff || nx <= 0 || ny <= 0 || nz <= 0 || (nx % portable::PS_TX) || (ny % portable::PS_TY) ||
      !aligned16(out) || !aligned16(in) || out == in)
    return CUDADMA_ERR_ARG;
  const size_t padded = (size_t)(nx + 8) * (size_t)(ny + 8) * (size_t)(nz + 8);
  if (padded > NOALLOC_MAX_FLOATS) return CUDADMA_ERR_TOO_LARGE;
  const int sms = sm_count();
  if (sms <= 0) { t_last_cuda_error = (int)cudaErrorNoDevice; return CUDADMA_ERR_CUDA; }
  float *scratch = nullptr;
  if (int r = noalloc_scratch(&scratch)) return r;
  cudaStream_t s = (cudaStream_t)stream;
  float *pin = scratch, *pout = scratch + NOALLOC_MAX_FLOATS;
  /* the array still holds the previous call's field: the zero border of both copies is re-made every time */
  CK(cudaMemsetAsync(pin, 0, padded * sizeof(float), s));
  CK(cudaMemsetAsync(pout, 0, padded * sizeof(float), s));
  if (int r = pad_copy(pin, const_cast<float *>(in), nx, ny, nz, 0, nz, true, s)) return r;
  if (int e = portable::launch_stencil_padded(pout, pin, nx, ny, nz, 0, nz, coeff, 0, sms, s)) {
    t_last_cuda_error = e;
    return CUDADMA_ERR_CUDA;
  }
  ++g_launches;
  return pad_copy(pout, out, nx, ny, nz, 0, nz, false, s);
}

int cudadma_release_workspace(void) {
  std::lock_guard<std::recursive_mutex> lock(g_ws_mutex);
  ws_drop();
  g_ws_device = -1;
  return CUDADMA_OK;
}

}  /* extern "C" */
