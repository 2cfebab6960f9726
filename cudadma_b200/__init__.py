"""cudadma_b200 -- CudaDMA's object API on Blackwell (sm_100a).

The device library is header-only (include/cudadma/cudadma.h); this package
holds the kernels built on it, their C ABI (libcudadma_b200.so) and the thin
host layer over that ABI.
"""
from .capi import (CudaDMAError, Slab, MultiStencil, clock_probe, fill_index, fill_uniform, make_tensor_map_2d, make_tensor_map_3d, IMPL_NATIVE, IMPL_PORTABLE, LIB_PATH, STENCIL_COEFFS, SYMBOLS, device_status,
                   gather_scatter, gather_scatter_host, gather_scatter_tma, launch_count, lib, release_workspace, seq_copy, seq_copy_host,
                   stencil25_run, stencil25_run_host, stencil25_step, stencil25_step_noalloc, stencil25_step_padded, strided_transpose, strided_transpose_host,
                   version)

__all__ = [
    "CudaDMAError", "Slab", "MultiStencil", "clock_probe", "fill_index", "fill_uniform", "make_tensor_map_2d", "make_tensor_map_3d", "IMPL_NATIVE", "IMPL_PORTABLE", "LIB_PATH", "STENCIL_COEFFS", "SYMBOLS", "device_status",
    "gather_scatter", "gather_scatter_host", "gather_scatter_tma", "launch_count", "lib", "release_workspace", "seq_copy", "seq_copy_host",
    "stencil25_run", "stencil25_run_host", "stencil25_step", "stencil25_step_noalloc", "stencil25_step_padded", "strided_transpose", "strided_transpose_host", "version",
]
