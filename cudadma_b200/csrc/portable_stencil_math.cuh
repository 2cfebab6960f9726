/*
 * portable_stencil_math.cuh -- tile shape, coefficients and per-point arithmetic of the
 * radius-4 25-point stencil kernels that are written against the CudaDMA object API as the
 * reference offers it (portable_kernels.cuh, and the halo-ring form in oracle/ref_halo_stencil.cu).
 * No CudaDMA class is named here, so the file builds next to either generation of the headers.
 */
#ifndef CUDADMA_B200_PORTABLE_STENCIL_MATH_CUH
#define CUDADMA_B200_PORTABLE_STENCIL_MATH_CUH

namespace portable {

constexpr int PS_TX = 32, PS_TY = 16, PS_R = 4, PS_WX = PS_TX + 2 * PS_R, PS_WY = PS_TY + 2 * PS_R;
constexpr int PS_COMPUTE = PS_TX * PS_TY, PS_DMA = 64;
struct PCoeffs { float c[5]; };

__device__ __forceinline__ float stencil_point(const float *__restrict__ w, const float cur, const float (&b)[4],
                                               const float (&f)[4], const PCoeffs &k) {
  /* w points at this thread's cell inside the 40 x 24 window */
  float acc = k.c[0] * cur;
#pragma unroll
  for (int r = 1; r <= PS_R; ++r) {
    const float s = ((w[-r] + w[r]) + (w[-r * PS_WX] + w[r * PS_WX])) + (b[r - 1] + f[r - 1]);
    acc = fmaf(k.c[r], s, acc);
  }
  return acc;
}

/* z-marching register queue of a thread: four planes behind, the current one, four ahead */
__device__ __forceinline__ void advance_queue(float (&b)[4], float &cur, float (&f)[4], const float next) {
  b[3] = b[2]; b[2] = b[1]; b[1] = b[0]; b[0] = cur;
  cur = f[0]; f[0] = f[1]; f[1] = f[2]; f[2] = f[3]; f[3] = next;
}

}  // namespace portable

#endif
