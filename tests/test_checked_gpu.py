"""The -DCUDADMA_CHECKED build of the header (tests/csrc/checked_probe.cu): a transfer with a run of
bytes outside the ranges the caller named is not issued, the first such run is recorded, the
handshake still completes and the kernel ends normally. The allocation behind the named range
is larger than the range, so no case here can reach unmapped memory."""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "tests", "csrc", "libcudadma_checked_probe.so")
pytestmark = pytest.mark.gpu
ALLOC, WINDOW = 8192, 4096  # floats


def probe(offset, count, rows=1, stride=0):
    lib = ctypes.CDLL(LIB)
    lib.checked_probe_run.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint),
                                      ctypes.POINTER(ctypes.c_uint), ctypes.POINTER(ctypes.c_longlong),
                                      ctypes.POINTER(ctypes.c_ulonglong)]
    src = oracle.fill_uniform(ALLOC, 0xCC, 1.0, 2.0)
    out = np.zeros(count, dtype=np.float32)
    status, kind, off, nbytes = ctypes.c_uint(0), ctypes.c_uint(0), ctypes.c_longlong(0), ctypes.c_ulonglong(0)
    err = lib.checked_probe_run(src.ctypes.data, ALLOC, WINDOW, offset, count, rows, stride, out.ctypes.data,
                                ctypes.byref(status), ctypes.byref(kind), ctypes.byref(off), ctypes.byref(nbytes))
    assert err == 0, "cudaError %d" % err
    return src, out, status.value, kind.value, off.value, nbytes.value


@pytest.mark.parametrize("offset,count,rows,stride", [(0, 1024, 1, 0), (3072, 1024, 1, 0), (5, 333, 1, 0),
                                                      (0, 1024, 4, 1024), (64, 512, 8, 500)])
def test_transfers_inside_the_named_range_run_as_usual(offset, count, rows, stride):
    src, out, status, kind, _, _ = probe(offset, count, rows, stride)
    assert status == 0 and kind == 0
    per = count // rows
    want = np.concatenate([src[offset + r * stride: offset + r * stride + per] for r in range(rows)]) if rows > 1 \
        else src[offset:offset + count]
    assert np.array_equal(out, want)


@pytest.mark.parametrize("offset,count,rows,stride,bad_off,bad_bytes",
                         [(3073, 1024, 1, 0, 3073 * 4, 4096),       # one float past the end of the range
                          (4096, 256, 1, 0, 4096 * 4, 1024),        # wholly outside
                          (0, 1024, 4, 1300, 3900 * 4, 1024)])      # the last of four runs sticks out
def test_a_run_outside_the_named_range_is_refused_and_recorded(offset, count, rows, stride, bad_off, bad_bytes):
    _, out, status, kind, off, nbytes = probe(offset, count, rows, stride)
    assert status == 0x8000B001 and kind == 1          # refused on the source side
    assert off == bad_off and nbytes == bad_bytes      # the first run that did not fit
    assert np.all(out == -1.0)                         # nothing was moved: the buffer kept its fill
