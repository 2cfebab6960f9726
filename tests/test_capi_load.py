"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

import cudadma_b200 as cd

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cudadma_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cudadma_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 15
    raw = ctypes.CDLL(cd.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), "library does not export %s" % n
    bound = {s[0] for s in cd.SYMBOLS}
    assert set(names) == bound, "python binding and header disagree: %s" % (set(names) ^ bound)


def test_version_and_strings():
    assert cd.version() >= 100
    lib = cd.lib()
    assert lib.cudadma_status_string(0) == b"ok"
    assert b"argument" in lib.cudadma_status_string(-1)
    assert b"wait" in lib.cudadma_status_string(1)


def test_argument_errors_need_no_device():
    lib = cd.lib()
    assert lib.cudadma_seq_copy(None, None, 64, 16384, 0, None) == -1
    assert lib.cudadma_seq_copy(16, 32, 6, 16384, 0, None) == -1          # size not a multiple of 4
    assert lib.cudadma_seq_copy(16, 32, 64, 100, 0, None) == -1           # chunk not a multiple of 16
    assert lib.cudadma_strided_transpose(16, 32, 100, 64, 0, None) == -1  # rows not a multiple of 128
    assert lib.cudadma_gather_scatter(16, 32, 48, 64, 100, 32, 0, None) == -1
    assert lib.cudadma_gather_scatter(16, 32, 48, 64, 128, 24, 0, None) == -1
    c = (ctypes.c_float * 5)(*cd.STENCIL_COEFFS)
    assert lib.cudadma_stencil25_step(16, 16, 32, 16, 8, 0, 8, c, 0, 0, None) == -1   # in == out
    assert lib.cudadma_stencil25_step(16, 32, 30, 16, 8, 0, 8, c, 0, 0, None) == -1   # nx not a multiple of 4
    assert lib.cudadma_stencil25_step(16, 32, 32, 16, 8, 4, 9, c, 0, 0, None) == -1   # plane range outside the grid
    assert lib.cudadma_stencil25_run_host(None, None, 32, 16, 8, c, 1, 0) == -1


def test_header_library_is_self_contained():
    """The device header compiles on its own for sm_100a (no GPU needed for nvcc)."""
    import shutil
    import subprocess
    import tempfile
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        import pytest
        pytest.skip("no nvcc")
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cu")
        open(src, "w").write('#include "cudaDMAv2.h"\n__global__ void k(float* a){ extern __shared__ float b[];'
                             ' CudaDMASequential<true,16,64,1024,32> d(1,32,32);'
                             ' if (d.owns_this_thread()) d.execute_dma(a,b); else { d.start_async_dma(); d.wait_for_dma_finish(); a[threadIdx.x]=b[threadIdx.x]; } }\n')
        subprocess.check_call([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-c", "-o",
                               os.path.join(d, "t.o"), "-I" + os.path.join(ROOT, "include", "cudadma"), src])
