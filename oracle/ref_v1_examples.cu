/*
 * ref_v1_examples.cu -- compile check: the reference's v1-API example kernels
 * (src/examples/saxpy/saxpy_cudaDMA_kernel.cu, src/examples/saxpy_strided/saxpy_cudaDMA_kernel.cu of
 * the CudaDMA project), read unmodified from the checkout, built against this repository's header
 * through its v1 spellings (cudaDMASequential / cudaDMAStrided without BYTES_PER_THREAD).
 * TEST INFRASTRUCTURE; object files only, nothing is run. As in ref_examples.cu, the reference's
 * "#pragma once" header is read first inside a namespace so that the examples' relative include
 * of it becomes a no-op and their class names resolve to this repository's.
 * -DV1_EXAMPLE_STRIDED selects the strided example (the two files reuse kernel names).
 */
#include <cstdio>

#include "cudadma.h"
namespace reference_header_parked {
#include "include/cudaDMA.h" /* found through -I<reference checkout> */
}
#ifdef V1_EXAMPLE_STRIDED
#include "src/examples/saxpy_strided/saxpy_cudaDMA_kernel.cu"
#else
#include "src/examples/saxpy/saxpy_cudaDMA_kernel.cu"
#endif
