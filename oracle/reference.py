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


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise ImportError("%s is missing (built by `make -C oracle ref` from the reference checkout)" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        vp, c = ctypes.c_void_p, ctypes
        l.cudadma_ref_seq_copy.argtypes = [vp, vp, c.c_size_t, vp]
        l.cudadma_ref_strided_transpose.argtypes = [vp, vp, c.c_int, c.c_int, vp]
        l.cudadma_ref_gather_scatter.argtypes = [vp, vp, vp, vp, c.c_size_t, vp]
        if hasattr(l, "cudadma_ref_stencil25_step_padded"):
            l.cudadma_ref_stencil25_step_padded.argtypes = [vp, vp, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                                            c.POINTER(c.c_float), c.c_int, vp]
        _lib = l
    return _lib


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _check(name, err):
    if err != 0:
        raise RuntimeError("%s: cudaError %d" % (name, err))


def seq_copy(dst, src, nbytes):
    _check("cudadma_ref_seq_copy", lib().cudadma_ref_seq_copy(dst.data_ptr(), src.data_ptr(), nbytes, _stream()))


def strided_transpose(dst, src, rows, cols):
    _check("cudadma_ref_strided_transpose",
           lib().cudadma_ref_strided_transpose(dst.data_ptr(), src.data_ptr(), rows, cols, _stream()))


def gather_scatter(out, table, gather_idx, scatter_idx, n):
    _check("cudadma_ref_gather_scatter",
           lib().cudadma_ref_gather_scatter(out.data_ptr(), table.data_ptr(), gather_idx.data_ptr(),
                                            scatter_idx.data_ptr(), n, _stream()))


def stencil25_step_padded(out, inp, nx, ny, nz, z_begin, z_end, coeff, z_chunk=0):
    c = (ctypes.c_float * 5)(*[float(v) for v in coeff])
    _check("cudadma_ref_stencil25_step_padded",
           lib().cudadma_ref_stencil25_step_padded(out.data_ptr(), inp.data_ptr(), nx, ny, nz, z_begin, z_end, c,
                                                   z_chunk, _stream()))
