"""ctypes binding of oracle/_ref/libcudadma_ref.so: the benchmark workloads run
through the REFERENCE CudaDMA classes compiled for sm_100a (oracle/ref_bench.cu).
TEST INFRASTRUCTURE: a device-side parity oracle for tests/ and the reference
arm of bench.py; the product package never imports it. The library exists only
where the reference checkout was present when oracle/Makefile's `ref` target ran.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libcudadma_ref.so")
_lib = None


def available():
    return os.path.exists(LIB_PATH)


HALO_STENCIL_PATH = os.path.join(_HERE, "_ref", "libhalo_stencil_ref.so")
BPTS = (64, 128, 192)   # BYTES_PER_THREAD budgets the reference arm tries (the reference's register staging bound)
_halo = None


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise ImportError("%s is missing (built by `make -C oracle ref` from the reference checkout)" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        vp, c = ctypes.c_void_p, ctypes
        l.cudadma_ref_seq_copy.argtypes = [vp, vp, c.c_size_t, c.c_int, vp]
        l.cudadma_ref_strided_transpose.argtypes = [vp, vp, c.c_int, c.c_int, c.c_int, vp]
        l.cudadma_ref_gather_scatter.argtypes = [vp, vp, vp, vp, c.c_size_t, c.c_int, vp]
        if hasattr(l, "cudadma_ref_stencil25_step_padded"):
            l.cudadma_ref_stencil25_step_padded.argtypes = [vp, vp, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                                            c.POINTER(c.c_float), c.c_int, c.c_int, vp]
        _lib = l
    return _lib


def halo_stencil_available():
    return os.path.exists(HALO_STENCIL_PATH)


def halo_lib(path=None):
    """The stencil whose tile comes in through v1 cudaDMAHalo (ring) + cudaDMAStrided (interior),
    oracle/ref_halo_stencil.cu built against the reference's v1 header (or, with `path`, another build of it)."""
    global _halo
    if path is not None or _halo is None:
        l = ctypes.CDLL(path or HALO_STENCIL_PATH)
        vp, c = ctypes.c_void_p, ctypes
        l.halo_stencil25_step_padded.argtypes = [vp, vp, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.POINTER(c.c_float),
                                                 c.c_int, vp]
        if path is not None:
            return l
        _halo = l
    return _halo


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _check(name, err):
    if err != 0:
        raise RuntimeError("%s: cudaError %d" % (name, err))


def seq_copy(dst, src, nbytes, bpt=64):
    _check("cudadma_ref_seq_copy", lib().cudadma_ref_seq_copy(dst.data_ptr(), src.data_ptr(), nbytes, bpt, _stream()))


def strided_transpose(dst, src, rows, cols, bpt=64):
    _check("cudadma_ref_strided_transpose",
           lib().cudadma_ref_strided_transpose(dst.data_ptr(), src.data_ptr(), rows, cols, bpt, _stream()))


def gather_scatter(out, table, gather_idx, scatter_idx, n, bpt=64):
    _check("cudadma_ref_gather_scatter",
           lib().cudadma_ref_gather_scatter(out.data_ptr(), table.data_ptr(), gather_idx.data_ptr(),
                                            scatter_idx.data_ptr(), n, bpt, _stream()))


def stencil25_step_padded(out, inp, nx, ny, nz, z_begin, z_end, coeff, z_chunk=0, bpt=64):
    c = (ctypes.c_float * 5)(*[float(v) for v in coeff])
    _check("cudadma_ref_stencil25_step_padded",
           lib().cudadma_ref_stencil25_step_padded(out.data_ptr(), inp.data_ptr(), nx, ny, nz, z_begin, z_end, c,
                                                   z_chunk, bpt, _stream()))


def halo_stencil25_step_padded(out, inp, nx, ny, nz, z_begin, z_end, coeff, z_chunk=0, lib_handle=None):
    c = (ctypes.c_float * 5)(*[float(v) for v in coeff])
    l = lib_handle or halo_lib()
    _check("halo_stencil25_step_padded",
           l.halo_stencil25_step_padded(out.data_ptr(), inp.data_ptr(), nx, ny, nz, z_begin, z_end, c, z_chunk, _stream()))
