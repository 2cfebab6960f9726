/*
 * stencil25.cuh -- radius-4, 25-point finite-difference step on an fp32 grid,
 *   out = c0*u + sum_{r=1..4} c_r*(u[x-r]+u[x+r]+u[y-r]+u[y+r]+u[z-r]+u[z+r]),
 * zero outside the grid, as a z-marching kernel fed by CudaDMA objects.
 *
 * One CTA owns a 32 x 16 xy tile and a run of z planes. Its DMA warp streams
 * the tile plus its radius-4 halo (40 x 24 floats), plane after plane, into a
 * ring of nine shared-memory buffers; 64 compute threads each own a 4 (x) by
 * 2 (y) patch of the tile, keep nine z planes of that patch in registers and
 * read the x/y neighbours of the current plane from shared memory with
 * 16-byte loads. Ring slot and register slot of a plane are both (plane mod 9),
 * so the loop is unrolled nine times and every index is static.
 *
 * The buffering scheme is the reference's warp-specialised stencil example
 * (src/examples/stencil/warp_specialized_manual_buffer.h:46-112) with nine
 * buffers instead of two; the arithmetic replaces its in-plane average
 * (src/examples/stencil/stencil_math.h:28-86) by the 25-point operator.
 *
 * The same body serves two loaders:
 *   - tensor-map loader (cudadma.h only): CudaDMAHalo::execute_dma_tile, one
 *     TMA box per plane from the unpadded grid, zero fill outside it;
 *   - portable loader (any CudaDMA header): CudaDMAStrided row copies of the
 *     40 x 24 window from a grid padded by four zero cells on every side,
 *     the way the reference's stencil example loads its tiles
 *     (src/examples/stencil/warp_specialized_single_buffer.h:35-58).
 */
#ifndef CUDADMA_B200_STENCIL25_CUH
#define CUDADMA_B200_STENCIL25_CUH

namespace stencil25 {

constexpr int R = 4;
constexpr int TILE_X = 32, TILE_Y = 16;
constexpr int WIN_X = TILE_X + 2 * R, WIN_Y = TILE_Y + 2 * R; /* 40 x 24 */
constexpr int PLANE_BYTES = WIN_X * WIN_Y * 4;                /* 3840 */
constexpr int SLOTS = 2 * R + 1;                              /* 9 */
constexpr int COMPUTE_THREADS = 64, DMA_THREADS = 32;
constexpr int SMEM_BYTES = SLOTS * PLANE_BYTES;

struct Coeffs { float c[5]; };

/* One output plane for this thread's 4 x 2 patch.
 * cur: the current plane's window in shared memory; q: register queue, q[s]
 * is the patch on the plane living in slot s; sc: slot of the current plane. */
template <int SC>
__device__ __forceinline__ void compute_patch(const float *__restrict__ cur, const float (&q)[SLOTS][2][4],
                                              const int tx, const int ty, const Coeffs &k, float (&res)[2][4]) {
  const float *row0 = cur + (2 * ty + R) * WIN_X + 4 * tx; /* column x-4 of own row 0 */
  float a[2][12];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float4 l = *reinterpret_cast<const float4 *>(row0 + j * WIN_X);
    const float4 r = *reinterpret_cast<const float4 *>(row0 + j * WIN_X + 8);
    a[j][0] = l.x; a[j][1] = l.y; a[j][2] = l.z; a[j][3] = l.w;
    a[j][4] = q[SC][j][0]; a[j][5] = q[SC][j][1]; a[j][6] = q[SC][j][2]; a[j][7] = q[SC][j][3];
    a[j][8] = r.x; a[j][9] = r.y; a[j][10] = r.z; a[j][11] = r.w;
  }
  /* yn[d]: window rows above the patch (d = 0..3 <-> row y0-4..y0-1) and below (d = 4..7 <-> y1+1..y1+4) */
  float yn[8][4];
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    const float4 u = *reinterpret_cast<const float4 *>(row0 + (d - 4) * WIN_X + 4);
    const float4 v = *reinterpret_cast<const float4 *>(row0 + (d + 2) * WIN_X + 4);
    yn[d][0] = u.x; yn[d][1] = u.y; yn[d][2] = u.z; yn[d][3] = u.w;
    yn[d + 4][0] = v.x; yn[d + 4][1] = v.y; yn[d + 4][2] = v.z; yn[d + 4][3] = v.w;
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float acc = k.c[0] * a[j][4 + i];
#pragma unroll
      for (int r = 1; r <= R; ++r) {
        /* rows y-r and y+r: own rows come from the queue, the rest from yn */
        float up, dn;
        if (j == 0) {
          up = yn[4 - r][i];
          dn = (r == 1) ? q[SC][1][i] : yn[4 + r - 2][i];
        } else {
          up = (r == 1) ? q[SC][0][i] : yn[4 - (r - 1)][i];
          dn = yn[3 + r][i];
        }
        const float s = ((a[j][4 + i - r] + a[j][4 + i + r]) + (up + dn)) +
                        (q[(SC + SLOTS - r) % SLOTS][j][i] + q[(SC + r) % SLOTS][j][i]);
        acc = fmaf(k.c[r], s, acc);
      }
      res[j][i] = acc;
    }
  }
}

/* Compute side of the CTA. RING exposes stage[s] with the CudaDMA sync calls.
 * Planes are numbered k = 0 .. nplanes-1 relative to (first output plane - 4);
 * output plane k-4 is produced at step k once planes k-8 .. k are in. */
template <typename RING>
__device__ __forceinline__ void compute_side(RING &ring, const unsigned char *smem, float *__restrict__ out,
                                             const long long out_pitch_y, const long long out_pitch_z,
                                             const int x_limit, const int y_limit, const int nplanes,
                                             const Coeffs &k) {
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  float q[SLOTS][2][4];
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) ring.stage[s].start_async_dma();
  const bool store_ok = (4 * tx < x_limit);
  float *o = out + (long long)(2 * ty) * out_pitch_y + 4 * tx;
  for (int k0 = 0; k0 < nplanes; k0 += SLOTS) {
#pragma unroll
    for (int kk = 0; kk < SLOTS; ++kk) {
      const int kp = k0 + kk;
      if (kp >= nplanes) break;
      ring.stage[kk].wait_for_dma_finish();
      const float *pl = reinterpret_cast<const float *>(smem + kk * PLANE_BYTES) + (2 * ty + R) * WIN_X + 4 * tx + 4;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float4 c = *reinterpret_cast<const float4 *>(pl + j * WIN_X);
        q[kk][j][0] = c.x; q[kk][j][1] = c.y; q[kk][j][2] = c.z; q[kk][j][3] = c.w;
      }
      if (kp < R) ring.stage[kk].start_async_dma(); /* lead-in planes are never a current plane */
      if (kp >= 2 * R) {
        const int sc = (kk + SLOTS - R) % SLOTS;
        float res[2][4];
        /* sc is a compile-time constant after unrolling; dispatch keeps the queue indices static */
        switch (sc) {
          case 0: compute_patch<0>(reinterpret_cast<const float *>(smem + 0 * PLANE_BYTES), q, tx, ty, k, res); break;
          case 1: compute_patch<1>(reinterpret_cast<const float *>(smem + 1 * PLANE_BYTES), q, tx, ty, k, res); break;
          case 2: compute_patch<2>(reinterpret_cast<const float *>(smem + 2 * PLANE_BYTES), q, tx, ty, k, res); break;
          case 3: compute_patch<3>(reinterpret_cast<const float *>(smem + 3 * PLANE_BYTES), q, tx, ty, k, res); break;
          case 4: compute_patch<4>(reinterpret_cast<const float *>(smem + 4 * PLANE_BYTES), q, tx, ty, k, res); break;
          case 5: compute_patch<5>(reinterpret_cast<const float *>(smem + 5 * PLANE_BYTES), q, tx, ty, k, res); break;
          case 6: compute_patch<6>(reinterpret_cast<const float *>(smem + 6 * PLANE_BYTES), q, tx, ty, k, res); break;
          case 7: compute_patch<7>(reinterpret_cast<const float *>(smem + 7 * PLANE_BYTES), q, tx, ty, k, res); break;
          default: compute_patch<8>(reinterpret_cast<const float *>(smem + 8 * PLANE_BYTES), q, tx, ty, k, res); break;
        }
        float *oz = o + (long long)(kp - 2 * R) * out_pitch_z;
        if (store_ok) {
          if (2 * ty < y_limit) *reinterpret_cast<float4 *>(oz) = make_float4(res[0][0], res[0][1], res[0][2], res[0][3]);
          if (2 * ty + 1 < y_limit)
            *reinterpret_cast<float4 *>(oz + out_pitch_y) = make_float4(res[1][0], res[1][1], res[1][2], res[1][3]);
        }
        ring.stage[sc].start_async_dma();
      }
    }
  }
}

#ifdef CUDADMA_B200_CUDADMA_H
/* Tensor-map loader. in_map: 3-D map over the nx x ny x nz input (x fastest),
 * box 40 x 24 x 1. Output planes [z_begin, z_end) are produced, blockIdx.z
 * taking z_chunk of them; input planes outside [0, nz) read as zero. */
__global__ void __launch_bounds__(COMPUTE_THREADS + DMA_THREADS)
tensor_kernel(const __grid_constant__ CUtensorMap in_map, float *__restrict__ out, const int nx, const int ny,
              const int z_begin, const int z_end, const int z_chunk, const Coeffs k) {
  extern __shared__ __align__(128) unsigned char smem[];
  typedef CudaDMAHalo<float, R, true, 16> Halo;
  cudadma_b200::kernels::Ring<Halo, SLOTS> ring(DMA_THREADS, COMPUTE_THREADS, COMPUTE_THREADS, TILE_X, TILE_Y, nx);
  const int x0 = blockIdx.x * TILE_X, y0 = blockIdx.y * TILE_Y;
  const int z0 = z_begin + blockIdx.z * z_chunk;
  const int depth = (z_end - z0 < z_chunk) ? (z_end - z0) : z_chunk;
  const int nplanes = depth + 2 * R;
  if (ring.stage[0].owns_this_thread()) {
    for (int k0 = 0;; k0 += SLOTS) {
#pragma unroll
      for (int kk = 0; kk < SLOTS; ++kk) {
        if (k0 + kk >= nplanes) return;
        ring.stage[kk].execute_dma_tile(&in_map, x0, y0, z0 - R + k0 + kk, smem + kk * PLANE_BYTES);
      }
    }
  } else {
    const long long py = nx, pz = (long long)nx * ny;
    compute_side(ring, smem, out + (long long)z0 * pz + (long long)y0 * py + x0, py, pz, nx - x0, ny - y0, nplanes, k);
  }
}
#endif

}  // namespace stencil25

#endif
