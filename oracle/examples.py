"""The reference's own example and benchmark kernels, built unmodified against the reference
headers and against this repository's header (oracle/ref_examples.cu, oracle/ref_v1_examples.cu,
oracle/ref_perf_sequential.cu; `make -C oracle ref`), run side by side.
TEST INFRASTRUCTURE: tests/ compares the two builds' results, bench.py reports their times. The
libraries exist only where the reference checkout was present at build time.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
R = 4
STENCIL_NAMES = ["warp_specialized_single_buffer", "warp_specialized_double_buffer", "warp_specialized_manual_buffer",
                 "non_warp_specialized_single_buffer", "non_warp_specialized_double_buffer"]
PERFSEQ_NAMES = ["non_specialized", "single_buffer", "double_buffer", "manual_buffer"]
# src/examples/sgemv/sgemv_dma.cu without its BOTH_DOUBLE variant, which does not compile (:468, :479)
SGEMV_NAMES = ["vec_single", "vec_double", "vec_manual", "both_single", "both_manual", "mat_single"]
# the reference's default problem and tile (src/examples/stencil/params_directed.h:17-24)
STENCIL_DEFAULT_DIMS = (960, 160, 200)
TILE_X, TILE_Y = 32, 4


def _path(name):
    return os.path.join(_HERE, "_ref", name)


def available(*names):
    return all(os.path.exists(_path(n)) for n in names)


def run_stencil(which, kid, src, dims):
    """which: "ours" or "ref". src: padded float32 array [z + 8, y + 8, x + 8, 2]. Returns (dst, ms per launch)."""
    lib = ctypes.CDLL(_path("libexamples_%s.so" % which))
    fn = getattr(lib, "examples_%s_run" % which)
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.POINTER(ctypes.c_float)]
    dst = np.zeros_like(src)
    ms = ctypes.c_float(0)
    err = fn(kid, src.ctypes.data, dst.ctypes.data, dims[0], dims[1], dims[2], ctypes.byref(ms))
    if err != 0:
        raise RuntimeError("stencil example %d (%s header): cudaError %d" % (kid, which, err))
    return dst, ms.value


def stencil_bandwidth_gbs(dims, ms):
    """TOTAL bandwidth as the reference's driver prints it (src/examples/stencil/cudaDMA_stencil2D.cu:220-228):
    per CTA and z step one (TILE_Y + 2R) x (TILE_X + 2R) float2 window read and one TILE_Y x TILE_X tile written."""
    ctas = (dims[0] // TILE_X) * (dims[1] // TILE_Y)
    read = ctas * dims[2] * (TILE_Y + 2 * R) * (TILE_X + 2 * R) * 8
    written = ctas * dims[2] * TILE_Y * TILE_X * 8
    return (read + written) / ms * 1e-6


def run_saxpy(example, which, kernel_id, x, y, a):
    """example: "sequential" or "strided"; which: "ours", "ref", or "ours_ro" (this repository's header with
    -DCUDADMA_SOURCES_READ_ONLY, sequential only). Returns (a * x + y as computed on the device, ms per launch)."""
    name = "libv1saxpy_%s%s.so" % ("strided_" if example == "strided" else "", which)
    lib = ctypes.CDLL(_path(name))
    lib.v1saxpy_elements.restype = ctypes.c_longlong
    lib.v1saxpy_run.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                ctypes.POINTER(ctypes.c_float)]
    if lib.v1saxpy_elements() != x.size:
        raise ValueError("the example wants %d elements" % lib.v1saxpy_elements())
    out = y.copy()
    ms = ctypes.c_float(0)
    err = lib.v1saxpy_run(kernel_id, out.ctypes.data, x.ctypes.data, a, ctypes.byref(ms))
    if err != 0:
        raise RuntimeError("saxpy example (%s, %s header): cudaError %d" % (example, which, err))
    return out, ms.value


def saxpy_elements(example):
    lib = ctypes.CDLL(_path("libv1saxpy_%sours.so" % ("strided_" if example == "strided" else "")))
    lib.v1saxpy_elements.restype = ctypes.c_longlong
    return int(lib.v1saxpy_elements())


def run_perf_sequential(which, kernel_id):
    """The reference's throughput benchmark kernel `kernel_id` (PERFSEQ_NAMES); returns (GB/s, ms per launch)
    by its own formula (src/perf/sequential/perf_sequential.cu:355-360)."""
    lib = ctypes.CDLL(_path("libperfseq_%s.so" % which))
    lib.perfseq_run.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    gbs, ms = ctypes.c_double(0), ctypes.c_double(0)
    err = lib.perfseq_run(kernel_id, ctypes.byref(gbs), ctypes.byref(ms))
    if err != 0:
        raise RuntimeError("perf_sequential kernel %d (%s header): cudaError %d" % (kernel_id, which, err))
    return gbs.value, ms.value


def run_sgemv(which, variant):
    """The reference's sgemv example kernel `variant` (SGEMV_NAMES) on its own problem (896 x 896, alpha = 2,
    src/examples/sgemv/sgemv_dma.cu:72-73, 774-858). Returns (y, ms per launch)."""
    lib = ctypes.CDLL(_path("libsgemv_%s.so" % which))
    lib.sgemv_run.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_float)]
    n = ctypes.c_int(0)
    lib.sgemv_run(variant, None, ctypes.byref(n), None)
    y = np.zeros(n.value, dtype=np.float32)
    ms = ctypes.c_float(0)
    err = lib.sgemv_run(variant, y.ctypes.data, ctypes.byref(n), ctypes.byref(ms))
    if err != 0:
        raise RuntimeError("sgemv example %s (%s header): cudaError %d" % (SGEMV_NAMES[variant], which, err))
    return y, ms.value


def sgemv_expected(n):
    """What the example's own verify() computes (:756-772): every term is a small integer, so fp32 sums are exact."""
    i = np.arange(n, dtype=np.int64)
    a = (i[None, :] * i[:, None]) % 11          # a[j, i] = (i * j) % 11
    x = i % 11
    return (2 * (a * x[:, None]).sum(axis=0)).astype(np.float32)
