/* Drop-in name: kernels that include "cudaDMAv2.h" (reference: include/cudaDMAv2.h)
 * get the sm_100a implementation by putting this directory on the include path. */
#include "cudadma.h"
