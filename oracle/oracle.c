/*
 * oracle.c -- CPU restatement of the CudaDMA transfer semantics and of the
 * benchmark workloads. TEST INFRASTRUCTURE ONLY: it is the checker for the
 * GPU library and the timed CPU baseline, never part of the product path.
 *
 * Every function states the reference code it follows (paths inside the
 * CudaDMA project). The reference ships no golden vectors: its tests
 * recompute the expected output from the input with the host loops restated
 * here, so those loops are the parity definition. Pinning:
 *   - copy, strided, gather, halo ring: pinned by the reference's own
 *     self-checking tests (same loops) and, on a GPU, by running the
 *     reference classes compiled for sm_100a on the same inputs;
 *   - scatter: PARITY UNPINNED by any reference test (its only scatter check
 *     is dead code); the rule comes from the header alone;
 *   - 25-point stencil: PARITY UNPINNED (the reference has no such kernel);
 *     defined by the benchmark text: radius 4, coefficients c0..c4,
 *     zero outside the domain, ping-pong time steps.
 *
 * Build: see oracle/Makefile (gcc -O3 -ffp-contract=off -fopenmp -shared -fPIC; contraction is
 * off so that the guarded and the vectorised path of the fp32 step round alike).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define CLONES __attribute__((target_clones("default", "avx2", "avx512f")))

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- seeded synthetic inputs (stateless: element i depends on seed + i) ---- */

static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
uint64_t oracle_splitmix64(uint64_t x) { return splitmix64(x); }

/* uniform in [lo, hi): u = top 24 bits * 2^-24 */
void oracle_fill_uniform(float *out, size_t n, uint64_t seed, float lo, float hi) {
  const float scale = hi - lo;
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++) {
    const float u = (float)(splitmix64(seed + i) >> 40) * (1.0f / 16777216.0f);
    out[i] = lo + scale * u;
  }
}
void oracle_fill_index(int32_t *out, size_t n, uint64_t seed, uint32_t modulo) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++) out[i] = (int32_t)(splitmix64(seed + i) % modulo);
}
/* Fisher-Yates permutation of 0..n-1 driven by splitmix64(seed + i) */
void oracle_permutation(int32_t *p, size_t n, uint64_t seed) {
  for (size_t i = 0; i < n; i++) p[i] = (int32_t)i;
  for (size_t i = n; i-- > 1;) {
    const size_t j = (size_t)(splitmix64(seed + i) % (i + 1));
    const int32_t t = p[i]; p[i] = p[j]; p[j] = t;
  }
}

/* ---- transfer semantics of the classes ---- */

/* CudaDMASequential: out[j] == in[j] for the element's bytes
 * (src/tests/test_sequential/cudaDMA_test_sequential_v2.cu:500-512). */
void oracle_sequential(void *dst, const void *src, size_t bytes) { memcpy(dst, src, bytes); }

/* CudaDMAStrided: row i of elmt_bytes goes from src + i*src_stride to
 * dst + i*dst_stride (src/tests/test_strided/cudaDMA_test_strided_v2.cu:659-676). */
void oracle_strided(void *dst, const void *src, size_t elmt_bytes, size_t num_elmts, size_t src_stride,
                    size_t dst_stride) {
  for (size_t i = 0; i < num_elmts; i++)
    memcpy((char *)dst + i * dst_stride, (const char *)src + i * src_stride, elmt_bytes);
}

/* CudaDMAIndirect gather: row i comes from src + index[i]*elmt_bytes and lands
 * at dst + i*pitch, pitch = max(alternate_stride, elmt_bytes)
 * (src/tests/test_indirect/cudaDMA_test_indirect_v2.cu:661-692;
 *  include/cudaDMAv2.h:9406, :13618-13619). */
void oracle_gather(void *dst, const void *src, const int32_t *index, size_t num_elmts, size_t elmt_bytes,
                   size_t alternate_stride) {
  const size_t pitch = alternate_stride > elmt_bytes ? alternate_stride : elmt_bytes;
  for (size_t i = 0; i < num_elmts; i++)
    memcpy((char *)dst + i * pitch, (const char *)src + (size_t)index[i] * elmt_bytes, elmt_bytes);
}
/* CudaDMAIndirect scatter: row i comes from src + i*pitch and lands at
 * dst + index[i]*elmt_bytes (include/cudaDMAv2.h:14021-14025). */
void oracle_scatter(void *dst, const void *src, const int32_t *index, size_t num_elmts, size_t elmt_bytes,
                    size_t alternate_stride) {
  const size_t pitch = alternate_stride > elmt_bytes ? alternate_stride : elmt_bytes;
  for (size_t i = 0; i < num_elmts; i++)
    memcpy((char *)dst + (size_t)index[i] * elmt_bytes, (const char *)src + i * pitch, elmt_bytes);
}

/* cudaDMAHalo: copies only the ring of a dimx x dimy tile -- radius rows above
 * and below (with the corner columns when corners != 0) and radius-wide side
 * panels -- from an array of row pitch `pitch` elements into a tile of row
 * pitch dimx + 2*radius elements; src and dst point at the first element of
 * the padded region (row 0, column 0), as check_halo sees them
 * (src/tests/test_halo/cudaDMA_test_halo.cu:91-164). Everything else in dst
 * is left untouched. */
void oracle_halo_ring(void *dst, const void *src, int dimx, int dimy, int pitch, int radius, int corners,
                      size_t elmt_bytes) {
  const size_t dp = (size_t)(dimx + 2 * radius);
  const size_t lead = corners ? 0 : (size_t)radius;
  const size_t row_elems = (size_t)dimx + (corners ? 2 * (size_t)radius : 0);
  for (int i = 0; i < radius; i++) {
    memcpy((char *)dst + ((size_t)i * dp + lead) * elmt_bytes,
           (const char *)src + ((size_t)i * pitch + lead) * elmt_bytes, row_elems * elmt_bytes);
    const size_t r = (size_t)(radius + dimy + i);
    memcpy((char *)dst + (r * dp + lead) * elmt_bytes, (const char *)src + (r * pitch + lead) * elmt_bytes,
           row_elems * elmt_bytes);
  }
  for (int i = 0; i < dimy; i++) {
    const size_t r = (size_t)(radius + i);
    memcpy((char *)dst + (r * dp) * elmt_bytes, (const char *)src + (r * pitch) * elmt_bytes,
           (size_t)radius * elmt_bytes);
    memcpy((char *)dst + (r * dp + radius + dimx) * elmt_bytes,
           (const char *)src + (r * pitch + radius + dimx) * elmt_bytes, (size_t)radius * elmt_bytes);
  }
}

/* ---- benchmark workloads (also the timed CPU baselines) ---- */

/* C1: chunked copy, the loop structure of src/perf/sequential/perf_sequential.cu:79-114
 * with the write-back the benchmark adds. */
void oracle_chunked_copy(void *dst, const void *src, size_t bytes, size_t chunk_bytes) {
  const size_t nchunks = (bytes + chunk_bytes - 1) / chunk_bytes;
#pragma omp parallel for schedule(static)
  for (size_t c = 0; c < nchunks; c++) {
    const size_t off = c * chunk_bytes;
    const size_t len = (bytes - off < chunk_bytes) ? (bytes - off) : chunk_bytes;
    memcpy((char *)dst + off, (const char *)src + off, len);
  }
}

/* C2: every tile_rows x tile_cols tile of a rows x cols fp32 matrix is pulled
 * with the strided rule above and written back transposed:
 * out[c * rows + r] = in[r * cols + c]. */
CLONES void oracle_tile_transpose(float *dst, const float *src, size_t rows, size_t cols, size_t tile_rows,
                                  size_t tile_cols) {
  const size_t tr = (rows + tile_rows - 1) / tile_rows, tc = (cols + tile_cols - 1) / tile_cols;
#pragma omp parallel for collapse(2) schedule(static)
  for (size_t ti = 0; ti < tr; ti++)
    for (size_t tj = 0; tj < tc; tj++) {
      const size_t r1 = (ti + 1) * tile_rows < rows ? (ti + 1) * tile_rows : rows;
      const size_t c1 = (tj + 1) * tile_cols < cols ? (tj + 1) * tile_cols : cols;
      for (size_t c = tj * tile_cols; c < c1; c++)
        for (size_t r = ti * tile_rows; r < r1; r++) dst[c * rows + r] = src[r * cols + c];
    }
}

/* C3: out[scatter_idx[i]] = table[gather_idx[i]] for records of record_bytes:
 * the gather rule followed by the scatter rule above, buffer by buffer. */
void oracle_gather_scatter(void *out, const void *table, const int32_t *gather_idx, const int32_t *scatter_idx,
                           size_t n, size_t record_bytes) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++)
    memcpy((char *)out + (size_t)scatter_idx[i] * record_bytes,
           (const char *)table + (size_t)gather_idx[i] * record_bytes, record_bytes);
}

/* C4/C5: one time step of the radius-4 25-point stencil,
 *   out = c0*u + sum_{r=1..4} c_r * (u[x-r] + u[x+r] + u[y-r] + u[y+r] + u[z-r] + u[z+r]),
 * reads outside the nx x ny x nz grid give 0. Double precision: the parity
 * reference. x is the fastest axis, z the slowest. */
void oracle_stencil25_step_f64(double *out, const double *in, int nx, int ny, int nz, const double c[5]) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int z = 0; z < nz; z++)
    for (int y = 0; y < ny; y++)
      for (int x = 0; x < nx; x++) {
        const size_t i = ((size_t)z * ny + y) * nx + x;
        double acc = c[0] * in[i];
        for (int r = 1; r <= 4; r++) {
          double s = 0.0;
          if (x - r >= 0) s += in[i - r];
          if (x + r < nx) s += in[i + r];
          if (y - r >= 0) s += in[i - (size_t)r * nx];
          if (y + r < ny) s += in[i + (size_t)r * nx];
          if (z - r >= 0) s += in[i - (size_t)r * nx * ny];
          if (z + r < nz) s += in[i + (size_t)r * nx * ny];
          acc += c[r] * s;
        }
        out[i] = acc;
      }
}

/* `steps` ping-pong steps in double from an fp32 field; result rounded to fp32
 * only at the end. Returns 0, or -1 if memory could not be had. */
int oracle_stencil25_f64(float *out, const float *in, int nx, int ny, int nz, const float coeff[5], int steps) {
  const size_t n = (size_t)nx * ny * nz;
  double *a = (double *)malloc(n * sizeof(double)), *b = (double *)malloc(n * sizeof(double));
  if (!a || !b) { free(a); free(b); return -1; }
  double c[5];
  for (int i = 0; i < 5; i++) c[i] = (double)coeff[i];
  for (size_t i = 0; i < n; i++) a[i] = (double)in[i];
  for (int s = 0; s < steps; s++) {
    oracle_stencil25_step_f64(b, a, nx, ny, nz, c);
    double *t = a; a = b; b = t;
  }
  for (size_t i = 0; i < n; i++) out[i] = (float)a[i];
  free(a); free(b);
  return 0;
}

/* The same step in fp32, threaded and vectorised: the timed CPU baseline.
 * Interior rows take a branch-free path; rows or columns near a face take the
 * guarded one. */
CLONES void oracle_stencil25_step_f32(float *out, const float *in, int nx, int ny, int nz, const float c[5]) {
  const ptrdiff_t sx = 1, sy = (ptrdiff_t)nx, sz = (ptrdiff_t)nx * ny;
#pragma omp parallel for collapse(2) schedule(static)
  for (int z = 0; z < nz; z++)
    for (int y = 0; y < ny; y++) {
      const size_t row = ((size_t)z * ny + y) * nx;
      const int inner = (z >= 4 && z < nz - 4 && y >= 4 && y < ny - 4);
      for (int x = 0; x < nx; x++) {
        const size_t i = row + x;
        if (inner && x >= 4 && x < nx - 4) continue;
        float acc = c[0] * in[i];
        for (int r = 1; r <= 4; r++) {
          float s = 0.0f;
          if (x - r >= 0) s += in[i - r * sx];
          if (x + r < nx) s += in[i + r * sx];
          if (y - r >= 0) s += in[i - r * sy];
          if (y + r < ny) s += in[i + r * sy];
          if (z - r >= 0) s += in[i - r * sz];
          if (z + r < nz) s += in[i + r * sz];
          acc += c[r] * s;
        }
        out[i] = acc;
      }
      if (inner) {
        const float *p = in + row;
        float *q = out + row;
#pragma omp simd
        for (int x = 4; x < nx - 4; x++) {
          float acc = c[0] * p[x];
          acc += c[1] * (p[x - 1] + p[x + 1] + p[x - sy] + p[x + sy] + p[x - sz] + p[x + sz]);
          acc += c[2] * (p[x - 2] + p[x + 2] + p[x - 2 * sy] + p[x + 2 * sy] + p[x - 2 * sz] + p[x + 2 * sz]);
          acc += c[3] * (p[x - 3] + p[x + 3] + p[x - 3 * sy] + p[x + 3 * sy] + p[x - 3 * sz] + p[x + 3 * sz]);
          acc += c[4] * (p[x - 4] + p[x + 4] + p[x - 4 * sy] + p[x + 4 * sy] + p[x - 4 * sz] + p[x + 4 * sz]);
          q[x] = acc;
        }
      }
    }
}
