/*
 * stencil25.cuh -- radius-4, 25-point finite-difference step on an fp32 grid,
 *   out = c0*u + sum_{r=1..4} c_r*(u[x-r]+u[x+r]+u[y-r]+u[y+r]+u[z-r]+u[z+r]),
 * zero outside the grid, as a z-marching kernel fed by CudaDMAHalo objects.
 *
 * One CTA owns a 64 x 16 xy tile and a run of z planes. Its DMA warp streams
 * the tile plus its radius-4 halo (72 x 24 floats, one TMA box per plane, zero
 * fill outside the grid) into a ring of shared-memory buffers. The compute
 * threads (128) each own a 4 (x) by 2 (y) patch of the tile. Every plane is read from
 * shared memory exactly once, when it arrives, and is pushed forward into the
 * nine output planes it contributes to:
 *   - its in-plane (x and y) neighbours go to the output plane of the same z;
 *   - its own value times c_|d| goes to the output planes z + d, d = -4..4.
 * The nine partial output planes of a patch live in registers; the slot of
 * output plane z is z mod 9, so the plane loop is unrolled nine times and every
 * register index is static. An output plane is complete, and stored, once the
 * plane four above it has been folded in. Every output sums its 25 products in
 * the same order whatever z range a CTA or a GPU owns, so results do not
 * depend on how the grid is cut.
 *
 * The buffering scheme is the reference's warp-specialised stencil example
 * (src/examples/stencil/warp_specialized_manual_buffer.h:46-112) with a ring of
 * buffers instead of two; the arithmetic replaces its in-plane average
 * (src/examples/stencil/stencil_math.h:28-86) by the 25-point operator.
 */
#ifndef CUDADMA_B200_STENCIL25_CUH
#define CUDADMA_B200_STENCIL25_CUH

#include <type_traits>
#include <utility>

namespace stencil25 {

constexpr int R = 4;
#ifndef STENCIL25_TILE_Y
#define STENCIL25_TILE_Y 16 /* 64 x 16 tile: 128 compute threads */
#endif
#ifndef STENCIL25_TILE_X
#define STENCIL25_TILE_X 64 /* 32 x 32 measured 0.6 to 1.5 % slower; 32 x 16 with twice the CTAs 6 % slower, 64 x 32 (one CTA per SM) slower */
#endif
constexpr int TILE_X = STENCIL25_TILE_X, TILE_Y = STENCIL25_TILE_Y;
constexpr int WIN_X = TILE_X + 2 * R, WIN_Y = TILE_Y + 2 * R; /* 72 x 24 */
constexpr int PLANE_BYTES = WIN_X * WIN_Y * 4;                /* 6912 */
constexpr int SLOTS = 2 * R + 1;                              /* 9 partial output planes */
#ifndef STENCIL25_STAGES
#define STENCIL25_STAGES 9 /* must divide SLOTS; nine keeps eight planes of loads in flight per CTA */
#endif
constexpr int STAGES = STENCIL25_STAGES;
static_assert(SLOTS % STAGES == 0, "the ring size must divide nine so that stage indices stay static");
constexpr int PY = 2; /* rows of a thread's patch (the patch is four points wide) */
constexpr int COMPUTE_THREADS = (TILE_X / 4) * (TILE_Y / PY), DMA_THREADS = 32;
constexpr int SMEM_BYTES = STAGES * PLANE_BYTES;

struct Coeffs { float c[5]; };
/* second destinations of the lowest and highest output planes (see tensor_kernel) */
struct Peers {
  float *lo; int lo_end;
  float *hi; int hi_begin;
};
/* Handshake of a z-sharded rank with its neighbours, folded into the step's one launch (all null:
 * none). Flag words count finished steps. wait_lo / wait_hi live in this GPU's memory and are
 * written by the neighbours; signal_lo / signal_hi live in the neighbours' memory. Only the CTAs
 * at a shared boundary take part: they read the ghost planes a neighbour filled during its last
 * step and they store into the neighbour's ghost planes, so before their first load they wait
 * (bounded) until that neighbour's flag has reached `step`, and the last of them to retire
 * (ticket counts them, `boundary_ctas` in all) publishes step + 1 (with a null ticket nobody in
 * the launch publishes: the caller does it with a launch of its own behind this one). The wait gives up after
 * `wait_limit` SM cycles: it then records a code in the status word, nothing more is stored into a
 * neighbour and the step count is not published, so the neighbours' own waits run out too instead
 * of taking over a wrong plane. */
struct Sync {
  const unsigned int *wait_lo, *wait_hi;
  unsigned int *signal_lo, *signal_hi;
  unsigned int *ticket;
  unsigned int *failed;      /* this rank's sticky failure word (0 = fine) */
  unsigned int step;
  unsigned int boundary_ctas;
  long long wait_limit;
};

/* Arithmetic is done two points at a time with the packed fp32 FMA of sm_100
 * (fma.rn.f32x2 through __ffma2_rn): one issue slot for two fused multiply-adds,
 * each bit-identical to fmaf. A patch row of four points is two such pairs. The
 * x neighbours at odd distances are the exception (see fold_plane): scalar fmaf. */
struct Row { float2 p[2]; };

__device__ __forceinline__ Row ld_row(const float *p) {
  const float4 v = *reinterpret_cast<const float4 *>(p);
  Row r;
  r.p[0] = make_float2(v.x, v.y);
  r.p[1] = make_float2(v.z, v.w);
  return r;
}

template <typename F, int... I>
__device__ __forceinline__ void static_for(F &&f, std::integer_sequence<int, I...>) {
  (f(std::integral_constant<int, I>{}), ...);
}

/* Fold the plane in slot position KK (plane number mod 9) into the partial outputs.
 * win: this thread's patch origin inside the plane's window (window row 2*ty + R,
 * window column 4*tx + R). in_plane: the plane is itself an output plane of this
 * CTA, so its x/y neighbours are needed. c2[r] = (c_r, c_r). */
template <int KK>
__device__ __forceinline__ void fold_plane(const float *__restrict__ win, float2 (&acc)[SLOTS][2][2],
                                           const float2 (&c2)[R + 1], const bool in_plane) {
  Row u[2];
  u[0] = ld_row(win);
  u[1] = ld_row(win + WIN_X);
  /* z direction: output plane KK + d gets c_|d| * u; the output plane four ahead starts here */
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      acc[(KK + R) % SLOTS][j][h] = make_float2(c2[R].x * u[j].p[h].x, c2[R].y * u[j].p[h].y);
#pragma unroll
      for (int d = -R; d < R; ++d) {
        const int cr = d < 0 ? -d : d;
        float2 &a = acc[(KK + d + SLOTS) % SLOTS][j][h];
        a = __ffma2_rn(c2[cr], u[j].p[h], a);
      }
    }
  if (in_plane) {
    float2(&o)[2][2] = acc[KK % SLOTS];
    /* x direction: row cells x-4 .. x+7; e[] are the pairs that start at even cells */
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const Row l = ld_row(win + j * WIN_X - 4), r = ld_row(win + j * WIN_X + 4);
      const float2 e[6] = {l.p[0], l.p[1], u[j].p[0], u[j].p[1], r.p[0], r.p[1]};
      const float cell[12] = {e[0].x, e[0].y, e[1].x, e[1].y, e[2].x, e[2].y,
                              e[3].x, e[3].y, e[4].x, e[4].y, e[5].x, e[5].y};
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int rr = 1; rr <= R; ++rr) {
          const int kl = 4 + 2 * h - rr, kr = 4 + 2 * h + rr; /* first cell of the left / right neighbour pair */
          if (rr & 1) {
            /* The pair starts at an odd cell, so it sits in no even-aligned register pair and a
             * packed FMA would first need two moves to build its operand. Two scalar FMAs on the
             * cells themselves give the same bits; leaving the five shuffled pairs out also takes ten
             * registers out of the tightest part of the loop (measured: 6 to 9 % for the kernel). */
            o[j][h].x = fmaf(c2[rr].x, cell[kl], o[j][h].x);
            o[j][h].y = fmaf(c2[rr].y, cell[kl + 1], o[j][h].y);
            o[j][h].x = fmaf(c2[rr].x, cell[kr], o[j][h].x);
            o[j][h].y = fmaf(c2[rr].y, cell[kr + 1], o[j][h].y);
          } else {
            o[j][h] = __ffma2_rn(c2[rr], e[kl >> 1], o[j][h]);
            o[j][h] = __ffma2_rn(c2[rr], e[kr >> 1], o[j][h]);
          }
        }
    }
    /* y direction: own rows feed each other, the eight rows around the patch are streamed */
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      o[0][h] = __ffma2_rn(c2[1], u[1].p[h], o[0][h]);
      o[1][h] = __ffma2_rn(c2[1], u[0].p[h], o[1][h]);
    }
#pragma unroll
    for (int d = 1; d <= R; ++d) {
      const Row up = ld_row(win - d * WIN_X);       /* row y0 - d: distance d from row 0, d + 1 from row 1 */
      const Row dn = ld_row(win + (d + 1) * WIN_X); /* row y1 + d: distance d from row 1, d + 1 from row 0 */
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        o[0][h] = __ffma2_rn(c2[d], up.p[h], o[0][h]);
        o[1][h] = __ffma2_rn(c2[d], dn.p[h], o[1][h]);
        if (d < R) {
          o[1][h] = __ffma2_rn(c2[d + 1], up.p[h], o[1][h]);
          o[0][h] = __ffma2_rn(c2[d + 1], dn.p[h], o[0][h]);
        }
      }
    }
  }
}

#ifdef CUDADMA_B200_CUDADMA_H
/* Compute side of a CTA: folds planes kp = 0 .. depth + 7 (numbered from first output plane - 4)
 * and stores output plane kp - 8 at step kp. PUSH: afterwards, planes below peer.lo_end / from
 * peer.hi_begin on are stored a second time through peer.lo / peer.hi. */
template <bool PUSH, typename RING>
__device__ __forceinline__ void compute_side(RING &ring, const unsigned char *smem, float *__restrict__ out,
                                             const Peers &peer, const Sync &sync, const int nx, const int ny,
                                             const int x0, const int y0, const int z0, const int depth,
                                             const Coeffs &k) {
  const int nplanes = depth + 2 * R;
  const int tx = threadIdx.x % (TILE_X / 4), ty = threadIdx.x / (TILE_X / 4);
  const long long py = nx, pz = (long long)nx * ny;
  const long long cell0 = (long long)z0 * pz + (long long)(y0 + PY * ty) * py + x0 + 4 * tx;
  float *o = out + cell0;
  const bool row0_ok = (x0 + 4 * tx < nx) && (y0 + PY * ty < ny);
  const bool row1_ok = (x0 + 4 * tx < nx) && (y0 + PY * ty + 1 < ny);
  const int win_off = (PY * ty + R) * WIN_X + 4 * tx + R;
  float2 acc[SLOTS][PY][2];
  float2 c2[R + 1];
#pragma unroll
  for (int r = 0; r <= R; ++r) c2[r] = make_float2(k.c[r], k.c[r]);
#pragma unroll
  for (int s = 0; s < STAGES; ++s) ring.stage[s].start_async_dma_after_reads();
  for (int k0 = 0; k0 < nplanes; k0 += SLOTS) {
    static_for(
        [&](auto kk_c) {
          constexpr int kk = decltype(kk_c)::value;
          const int kp = k0 + kk;
          if (kp < nplanes) {
            ring.stage[kk % STAGES].wait_for_dma_finish();
            const float *win = reinterpret_cast<const float *>(smem + (kk % STAGES) * PLANE_BYTES) + win_off;
            fold_plane<kk>(win, acc, c2, kp >= R && kp < depth + R);
            ring.stage[kk % STAGES].start_async_dma_after_reads(); /* this side never writes the ring */
            if (kp >= 2 * R) {
              /* output plane kp - 8 of this CTA is complete: it sits in slot (kk - 4) mod 9 */
              const float2(&r)[2][2] = acc[(kk + SLOTS - R) % SLOTS];
              const long long plane = (long long)(kp - 2 * R) * pz;
              const float4 v0 = make_float4(r[0][0].x, r[0][0].y, r[0][1].x, r[0][1].y);
              const float4 v1 = make_float4(r[1][0].x, r[1][0].y, r[1][1].x, r[1][1].y);
              if (row0_ok) *reinterpret_cast<float4 *>(o + plane) = v0;
              if (row1_ok) *reinterpret_cast<float4 *>(o + plane + py) = v1;
            }
          }
        },
        std::make_integer_sequence<int, SLOTS>{});
  }
  if (PUSH) {
    /* Second destinations. Kept out of the plane loop, which is tight on registers: every thread
     * reads back the cells it has just stored itself (its own stores are visible to it, and
     * still in cache) for the few planes of this CTA that lie in a pushed range, and stores
     * them again through the peer pointer. Not after a wait of the grid has given up: what this
     * CTA computed may then rest on planes that never arrived. */
    const bool sound = *reinterpret_cast<volatile unsigned int *>(&cudadma_b200::g_status_word) == 0u;
#pragma unroll 1
    for (int side = 0; side < 2; ++side) {
      float *const pb = side ? peer.hi : peer.lo;
      if (!pb || !sound) continue;
      const int zb = side ? (peer.hi_begin > z0 ? peer.hi_begin : z0) : z0;
      const int ze = side ? z0 + depth : (peer.lo_end < z0 + depth ? peer.lo_end : z0 + depth);
      /* at most R planes, two at a time: the loads of a pair first, then its stores, so that the
       * read-backs (L2 hits) overlap instead of each plane's stores waiting for that plane's loads
       * (all four planes at once made the compiler spill inside the kernel) */
#pragma unroll 1
      for (int z = zb; z < ze; z += 2) {
        const long long plane = (long long)(z - z0) * pz;
        const bool two = z + 1 < ze;
        float4 a0, a1, b0, b1;
        if (row0_ok) a0 = *reinterpret_cast<const float4 *>(o + plane);
        if (row1_ok) a1 = *reinterpret_cast<const float4 *>(o + plane + py);
        if (two && row0_ok) b0 = *reinterpret_cast<const float4 *>(o + plane + pz);
        if (two && row1_ok) b1 = *reinterpret_cast<const float4 *>(o + plane + pz + py);
        if (row0_ok) *reinterpret_cast<float4 *>(pb + cell0 + plane) = a0;
        if (row1_ok) *reinterpret_cast<float4 *>(pb + cell0 + plane + py) = a1;
        if (two && row0_ok) *reinterpret_cast<float4 *>(pb + cell0 + plane + pz) = b0;
        if (two && row1_ok) *reinterpret_cast<float4 *>(pb + cell0 + plane + pz + py) = b1;
      }
    }
    if (sync.ticket) {
      /* This CTA is done with the ghost planes and with its stores into the neighbours. All its
       * compute threads meet at hardware barrier 1 (the objects of this kernel are on mbarriers); thread 0 then
       * makes their stores visible system-wide (the fence is cumulative over what the barrier
       * ordered before it) and takes a ticket; the last boundary CTA of the launch publishes. */
      asm volatile("bar.sync 1, %0;" ::"n"(COMPUTE_THREADS) : "memory");
      if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int t = atomicAdd(sync.ticket, 1u);
        if (t + 1u == sync.boundary_ctas) {
          *sync.ticket = 0u; /* for the next launch, which the stream orders after this one */
          __threadfence_system();
          const unsigned int w = *reinterpret_cast<volatile unsigned int *>(&cudadma_b200::g_status_word);
          if (w != 0u) {
            atomicCAS(sync.failed, 0u, w);
          } else if (*reinterpret_cast<volatile unsigned int *>(sync.failed) == 0u) {
            const unsigned int done = sync.step + 1u;
            if (sync.signal_lo) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(sync.signal_lo), "r"(done) : "memory");
            if (sync.signal_hi) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(sync.signal_hi), "r"(done) : "memory");
          }
        }
      }
    }
  }
}

/* DMA side of a boundary CTA, before its first load: wait until the neighbour on that side has
 * finished `step` steps (see Sync). One lane polls with system-scope acquire loads; the fence
 * afterwards orders the TMA loads of the ghost planes (asynchronous proxy) behind the acquire. */
__device__ __noinline__ bool poll_neighbour(const unsigned int *flag, const Sync &sync, const unsigned int side) {
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= sync.step) return true;
    if (*reinterpret_cast<volatile unsigned int *>(&cudadma_b200::g_status_word) != 0u ||
        *reinterpret_cast<volatile unsigned int *>(sync.failed) != 0u)
      return false; /* the step is lost already: do not sit out another limit */
    if (clock64() - t0 > sync.wait_limit) {
      atomicCAS(&cudadma_b200::g_status_word, 0u, 0x80000000u | 0xE000u | side);
      return false;
    }
    __nanosleep(100);
  }
}
/* whole warp; returns whether the neighbours asked for have arrived */
__device__ __forceinline__ bool wait_for_neighbours(const Sync &sync, const bool lo, const bool hi) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    if (lo && sync.wait_lo) ok = poll_neighbour(sync.wait_lo, sync, 0u);
    if (ok && hi && sync.wait_hi) ok = poll_neighbour(sync.wait_hi, sync, 1u);
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

/* in_map: 3-D tensor map over the nx x ny x nz input (x fastest), box 72 x 24 x 1.
 * Output planes [z_begin, z_end) are produced; input planes outside [0, nz) read as zero. Planes
 * of a CTA are numbered kp = 0 .. depth + 7 from (first output plane - 4); output plane kp - 8 is
 * stored at step kp.
 * Runs of planes per CTA: z_edge == 0: blockIdx.z takes planes [z_begin + blockIdx.z * z_chunk, + z_chunk).
 * z_edge < 0: the same runs, highest first (run gridDim.z - 1 - blockIdx.z). A sharded rank whose step
 * count goes out behind the kernel uses this: the CTAs that wait for the LOWER neighbour before their
 * first load then start in the second half of the launch, and those of the top run wait for the upper
 * neighbour only before their last four planes, so neither wait is met at the start of the kernel
 * and two GPUs can drift against each other by a good part of a step without either of them idling.
 * z_edge > 0 (sharded ranks): blockIdx.z == 0 takes the lowest z_edge planes, blockIdx.z == 1 the
 * highest z_edge planes, and blockIdx.z >= 2 runs of z_chunk planes of what lies between. CTAs are
 * dispatched in blockIdx order, so both boundary runs start first and the step count can go out
 * to the neighbours while the interior is still being computed.
 * Peers: output planes below peer.lo_end are stored a second time through peer.lo, planes from
 * peer.hi_begin on through peer.hi, at the same plane index (null pointers switch this off).
 * The sharded driver points them into the z-neighbour GPUs' ghost planes (plain stores over
 * NVLink), shifted so that this rank's plane numbers land on the neighbour's. Sync: see above. */
#ifndef STENCIL25_MIN_BLOCKS
#define STENCIL25_MIN_BLOCKS 2 /* two CTAs of 160 threads per SM: eight compute warps, 167 registers */
#endif
__global__ void __launch_bounds__(COMPUTE_THREADS + DMA_THREADS, STENCIL25_MIN_BLOCKS)
tensor_kernel(const __grid_constant__ CUtensorMap in_map, float *__restrict__ out, const Peers peer,
              const __grid_constant__ Sync sync, const int nx, const int ny, const int z_begin, const int z_end,
              const int z_chunk, const int z_edge, const Coeffs k) {
  extern __shared__ __align__(128) unsigned char smem[];
  typedef CudaDMAHalo<float, R, true, 16> Halo;
  cudadma_b200::kernels::Ring<Halo, STAGES> ring(DMA_THREADS, COMPUTE_THREADS, COMPUTE_THREADS, TILE_X, TILE_Y, nx);
  const int x0 = blockIdx.x * TILE_X, y0 = blockIdx.y * TILE_Y;
  int z0, depth;
  if (z_edge > 0) {
    if (blockIdx.z == 0) { z0 = z_begin; depth = z_edge; }
    else if (blockIdx.z == 1) { z0 = z_end - z_edge; depth = z_edge; }
    else {
      z0 = z_begin + z_edge + ((int)blockIdx.z - 2) * z_chunk;
      depth = (z_end - z_edge - z0 < z_chunk) ? (z_end - z_edge - z0) : z_chunk;
    }
  } else {
    const int run = z_edge < 0 ? (int)(gridDim.z - 1 - blockIdx.z) : (int)blockIdx.z;
    z0 = z_begin + run * z_chunk;
    depth = (z_end - z0 < z_chunk) ? (z_end - z0) : z_chunk;
  }
  const int nplanes = depth + 2 * R;
  /* CTAs whose planes reach into a pushed range are the ones that touch a shared boundary */
  const bool at_lo = peer.lo && z0 < peer.lo_end, at_hi = peer.hi && z0 + depth > peer.hi_begin;
  if (ring.stage[0].owns_this_thread()) {
    /* The ghost planes of the lower neighbour are the first planes this CTA loads, those of the upper
     * neighbour the last four: each wait comes directly before the first load that needs it. A
     * neighbour that did not arrive: no further plane is loaded, so nothing can still be on its way
     * into shared memory when this CTA's compute threads, whose own waits now give up at once,
     * have run through their planes and the CTA retires. */
    if (at_lo && sync.wait_lo && !wait_for_neighbours(sync, true, false)) return;
    const int first_upper_ghost = (at_hi && sync.wait_hi) ? depth + R : nplanes;
    for (int k0 = 0;; k0 += STAGES) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        if (k0 + s >= nplanes) return;
        if (k0 + s == first_upper_ghost && !wait_for_neighbours(sync, false, true)) return;
        ring.stage[s].execute_dma_tile(&in_map, x0, y0, z0 - R + k0 + s, smem + s * PLANE_BYTES);
      }
    }
  } else {
    /* Only those CTAs run the instantiation with the second stores behind its loop (one body for
     * all measured 1 % slower without peers). */
    if (at_lo || at_hi) compute_side<true>(ring, smem, out, peer, sync, nx, ny, x0, y0, z0, depth, k);
    else compute_side<false>(ring, smem, out, peer, sync, nx, ny, x0, y0, z0, depth, k);
  }
}
#endif

}  // namespace stencil25

#endif
