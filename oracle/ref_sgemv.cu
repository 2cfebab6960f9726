/*
 * ref_sgemv.cu -- host driver for the reference's sgemv example (src/examples/sgemv/sgemv_dma.cu of
 * the CudaDMA project: seven kernels written against v1 cudaDMASequential / cudaDMAStrided, one per
 * selector macro, :142-620), compiled from the source where it lies; nothing of it is copied here.
 * TEST INFRASTRUCTURE. Six of the seven are built: the BOTH_DOUBLE variant does not compile against
 * the reference's own header either ("blockIdx.x**COMPUTE_THREADS_PER_CTA", :468 and :479).
 *
 * The example file holds one variant per compilation (its macros pick kernel, CTA shape and buffer
 * sizes), so it is read six times, each time inside a namespace of its own (ref_sgemv_variant.inc,
 * which also launches the variant the way the example's main() does and undefines its macros again).
 * Built twice by oracle/Makefile: against the reference's v1 header (-> _ref/libsgemv_ref.so), and
 * with -DEXAMPLES_OURS against this repository's header (-> _ref/libsgemv_ours.so), for which the
 * reference's "#pragma once" header is parked in a namespace so that the example's relative include
 * of it becomes a no-op and its class names resolve to this repository's.
 */
#include <cstdio>
#include <cstdlib>
#include <cassert>
#include <cmath>
#include "cuda.h"
#include "cuda_runtime.h"

#ifdef EXAMPLES_OURS
#include "cudadma.h"
namespace reference_header_parked {
#include "include/cudaDMA.h" /* found through -I<reference checkout> */
}
#else
#include "include/cudaDMA.h"
#endif

#define main cudadma_reference_sgemv_main

namespace sgemv_vec_single {
#define VEC_SINGLE
#include "ref_sgemv_variant.inc"
#undef VEC_SINGLE
}
namespace sgemv_vec_double {
#define VEC_DOUBLE
#include "ref_sgemv_variant.inc"
#undef VEC_DOUBLE
}
namespace sgemv_vec_manual {
#define VEC_MANUAL
#include "ref_sgemv_variant.inc"
#undef VEC_MANUAL
}
namespace sgemv_both_single {
#define BOTH_SINGLE
#include "ref_sgemv_variant.inc"
#undef BOTH_SINGLE
}
namespace sgemv_both_manual {
#define BOTH_MANUAL
#include "ref_sgemv_variant.inc"
#undef BOTH_MANUAL
}
namespace sgemv_mat_single {
#define MAT_SINGLE
#include "ref_sgemv_variant.inc"
#undef MAT_SINGLE
}
#undef main

extern "C" {

int sgemv_num_variants(void) { return 6; }

/* variant 0 vec_single, 1 vec_double, 2 vec_manual, 3 both_single, 4 both_manual, 5 mat_single.
 * h_y == NULL: only *n is filled in. Returns 0 or a cudaError_t. */
int sgemv_run(int variant, float *h_y, int *n, float *ms_per_launch) {
  const int nreps = 20;
  int e;
  switch (variant) {
    case 0: e = sgemv_vec_single::run(h_y, n, ms_per_launch, nreps); break;
    case 1: e = sgemv_vec_double::run(h_y, n, ms_per_launch, nreps); break;
    case 2: e = sgemv_vec_manual::run(h_y, n, ms_per_launch, nreps); break;
    case 3: e = sgemv_both_single::run(h_y, n, ms_per_launch, nreps); break;
    case 4: e = sgemv_both_manual::run(h_y, n, ms_per_launch, nreps); break;
    case 5: e = sgemv_mat_single::run(h_y, n, ms_per_launch, nreps); break;
    default: return (int)cudaErrorInvalidValue;
  }
#ifdef EXAMPLES_OURS
  if (e == 0 && h_y) {
    unsigned int w = 0;
    cudaError_t s = cudadma_b200::read_status(&w, 0);
    if (s != cudaSuccess) return (int)s;
    if (w) return (int)cudaErrorLaunchTimeout; /* a bounded wait inside a kernel gave up */
  }
#endif
  return e;
}

} /* extern "C" */
