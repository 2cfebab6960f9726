/* Drop-in name for kernels that include "cudaDMA.h" (the reference's v1 header, include/cudaDMA.h):
 * cudadma.h carries the v1 spellings cudaDMASequential / cudaDMAStrided / cudaDMAIndirect /
 * cudaDMAHalo / cudaDMACustom next to the v2 classes. */
#include "cudadma.h"
