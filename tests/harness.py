"""ctypes access to the single-CTA API test kernels (tests/csrc/api_harness.cu).

`ours()` is the harness built against this repository's header. `reference_v2()`
and `reference_v1()` are the same source built against the reference headers
(oracle/_ref, present only when the reference checkout was there at build time).
"""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
c = ctypes
FP = c.POINTER(c.c_float)
IP = c.POINTER(c.c_int)


class Harness:
    def __init__(self, path, prefix):
        self.lib = ctypes.CDLL(path)
        self.prefix = prefix
        self.families = getattr(self.lib, prefix + "families")()
        if self.families & 1:
            self._seq = getattr(self.lib, prefix + "sequential")
            self._seq.argtypes = [c.c_int] * 8 + [c.c_void_p, c.c_void_p, c.c_int]
            self._str = getattr(self.lib, prefix + "strided")
            self._str.argtypes = [c.c_int] * 11 + [c.c_void_p, c.c_int, c.c_void_p, c.c_int]
            self._ind = getattr(self.lib, prefix + "indirect")
            self._ind.argtypes = [c.c_int] * 11 + [c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_int]
        if self.families & 2:
            self._halo = getattr(self.lib, prefix + "halo")
            self._halo.argtypes = [c.c_int] * 9 + [c.c_void_p, c.c_void_p]

    def sequential(self, ws, level, two_phase, qualified, alignment, offset, nbytes, ndma, h_in):
        h_in = np.ascontiguousarray(h_in, dtype=np.float32)
        out = np.zeros_like(h_in)
        r = self._seq(ws, level, two_phase, qualified, alignment, offset, nbytes, ndma, h_in.ctypes.data,
                      out.ctypes.data, h_in.size)
        return r, out

    def strided(self, ws, level, two_phase, qualified, alignment, offset, nbytes, rows, sstride, dstride, ndma, h_in,
                buffer_floats):
        h_in = np.ascontiguousarray(h_in, dtype=np.float32)
        out = np.zeros(buffer_floats, dtype=np.float32)
        r = self._str(ws, level, two_phase, qualified, alignment, offset, nbytes, rows, sstride, dstride, ndma,
                      h_in.ctypes.data, h_in.size, out.ctypes.data, buffer_floats)
        return r, out

    def indirect(self, gather, ws, level, two_phase, qualified, alignment, offset, nbytes, rows, alt, ndma, index,
                 h_in, out_floats, buffer_floats):
        h_in = np.ascontiguousarray(h_in, dtype=np.float32)
        index = np.ascontiguousarray(index, dtype=np.int32)
        out = np.zeros(out_floats, dtype=np.float32)
        r = self._ind(gather, ws, level, two_phase, qualified, alignment, offset, nbytes, rows, alt, ndma,
                      index.ctypes.data, h_in.ctypes.data, h_in.size, out.ctypes.data, out_floats, buffer_floats)
        return r, out

    def halo(self, elmt_floats, radius, corners, alignment, offset, dimx, dimy, pitch, ndma, h_in):
        h_in = np.ascontiguousarray(h_in, dtype=np.float32)
        out = np.zeros(((dimx + 2 * radius) * (dimy + 2 * radius) + offset) * elmt_floats, dtype=np.float32)
        r = self._halo(elmt_floats, radius, corners, alignment, offset, dimx, dimy, pitch, ndma, h_in.ctypes.data,
                       out.ctypes.data)
        return r, out


_cache = {}


def _load(key, rel, prefix):
    if key not in _cache:
        path = os.path.join(ROOT, rel)
        _cache[key] = Harness(path, prefix) if os.path.exists(path) else None
    return _cache[key]


def ours():
    h = _load("ours", "tests/csrc/libcudadma_apitest.so", "apitest_")
    if h is None:
        raise ImportError("tests/csrc/libcudadma_apitest.so is missing: run __graft_entry__.build()")
    return h


def reference_v2():
    return _load("ref2", "oracle/_ref/libapitest_ref.so", "refapi_")


def reference_v1():
    return _load("ref1", "oracle/_ref/libapitest_ref_halo.so", "refapi_")
