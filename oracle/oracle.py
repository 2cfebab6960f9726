"""ctypes binding of oracle/liboracle.so -- TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
import this module; the product package never does.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: run `make -C oracle`" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        c = ctypes
        vp, sz, i32, f32, u64 = c.c_void_p, c.c_size_t, c.c_int, c.c_float, c.c_uint64
        sigs = {
            "oracle_num_threads": (i32, []),
            "oracle_splitmix64": (u64, [u64]),
            "oracle_fill_uniform": (None, [vp, sz, u64, f32, f32]),
            "oracle_fill_index": (None, [vp, sz, u64, c.c_uint32]),
            "oracle_permutation": (None, [vp, sz, u64]),
            "oracle_sequential": (None, [vp, vp, sz]),
            "oracle_strided": (None, [vp, vp, sz, sz, sz, sz]),
            "oracle_gather": (None, [vp, vp, vp, sz, sz, sz]),
            "oracle_scatter": (None, [vp, vp, vp, sz, sz, sz]),
            "oracle_halo_ring": (None, [vp, vp, i32, i32, i32, i32, i32, sz]),
            "oracle_chunked_copy": (None, [vp, vp, sz, sz]),
            "oracle_tile_transpose": (None, [vp, vp, sz, sz, sz, sz]),
            "oracle_gather_scatter": (None, [vp, vp, vp, vp, sz, sz]),
            "oracle_stencil25_f64": (i32, [vp, vp, i32, i32, i32, vp, i32]),
            "oracle_stencil25_step_f32": (None, [vp, vp, i32, i32, i32, vp]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def _p(a):
    return a.ctypes.data


def num_threads():
    return lib().oracle_num_threads()


def fill_uniform(n, seed, lo, hi):
    out = np.empty(n, dtype=np.float32)
    lib().oracle_fill_uniform(_p(out), n, seed, lo, hi)
    return out


def fill_index(n, seed, modulo):
    out = np.empty(n, dtype=np.int32)
    lib().oracle_fill_index(_p(out), n, seed, modulo)
    return out


def permutation(n, seed):
    out = np.empty(n, dtype=np.int32)
    lib().oracle_permutation(_p(out), n, seed)
    return out


def sequential(src_bytes):
    src = np.ascontiguousarray(src_bytes).view(np.uint8)
    dst = np.zeros_like(src)
    lib().oracle_sequential(_p(dst), _p(src), src.size)
    return dst


def strided(dst, src, elmt_bytes, num_elmts, src_stride, dst_stride):
    """dst, src: uint8 arrays; rows are copied in place into dst."""
    lib().oracle_strided(_p(dst), _p(src), elmt_bytes, num_elmts, src_stride, dst_stride)
    return dst


def gather(dst, src, index, elmt_bytes, alternate_stride=0):
    index = np.ascontiguousarray(index, dtype=np.int32)
    lib().oracle_gather(_p(dst), _p(src), _p(index), index.size, elmt_bytes, alternate_stride)
    return dst


def scatter(dst, src, index, elmt_bytes, alternate_stride=0):
    index = np.ascontiguousarray(index, dtype=np.int32)
    lib().oracle_scatter(_p(dst), _p(src), _p(index), index.size, elmt_bytes, alternate_stride)
    return dst


def halo_ring(dst, src, dimx, dimy, pitch, radius, corners, elmt_bytes):
    lib().oracle_halo_ring(_p(dst), _p(src), dimx, dimy, pitch, radius, int(bool(corners)), elmt_bytes)
    return dst


def chunked_copy(src, chunk_bytes=16384):
    src = np.ascontiguousarray(src)
    dst = np.empty_like(src)
    lib().oracle_chunked_copy(_p(dst), _p(src), src.nbytes, chunk_bytes)
    return dst


def tile_transpose(src, tile_rows=128, tile_cols=64, out=None):
    src = np.ascontiguousarray(src, dtype=np.float32)
    rows, cols = src.shape
    if out is None:
        out = np.empty((cols, rows), dtype=np.float32)
    lib().oracle_tile_transpose(_p(out), _p(src), rows, cols, tile_rows, tile_cols)
    return out


def gather_scatter(out, table, gather_idx, scatter_idx, record_bytes=32):
    gather_idx = np.ascontiguousarray(gather_idx, dtype=np.int32)
    scatter_idx = np.ascontiguousarray(scatter_idx, dtype=np.int32)
    lib().oracle_gather_scatter(_p(out), _p(table), _p(gather_idx), _p(scatter_idx), gather_idx.size, record_bytes)
    return out


def stencil25_f64(field, coeff, steps):
    """field: float32 array [nz, ny, nx]; returns the float32 rounding of `steps` double-precision steps."""
    field = np.ascontiguousarray(field, dtype=np.float32)
    nz, ny, nx = field.shape
    out = np.empty_like(field)
    c = np.asarray(coeff, dtype=np.float32)
    if lib().oracle_stencil25_f64(_p(out), _p(field), nx, ny, nz, _p(c), steps) != 0:
        raise MemoryError("oracle_stencil25_f64")
    return out


def stencil25_step_f32(field, coeff, out=None):
    field = np.ascontiguousarray(field, dtype=np.float32)
    nz, ny, nx = field.shape
    if out is None:
        out = np.empty_like(field)
    c = np.asarray(coeff, dtype=np.float32)
    lib().oracle_stencil25_step_f32(_p(out), _p(field), nx, ny, nz, _p(c))
    return out
