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
        # the v1 spellings, used the way the reference's saxpy example uses them
        # (src/examples/saxpy/saxpy_cudaDMA_kernel.cu:276-279, src/examples/saxpy_strided/saxpy_cudaDMA_kernel.cu:54-57)
        src1 = os.path.join(d, "v1.cu")
        open(src1, "w").write('#include "cudaDMA.h"\n__global__ void k(float* x, float* y, const int* idx){ extern __shared__ float b[];'
                              ' cudaDMASequential<true,16,4096,64> d0(1,128,128);'
                              ' cudaDMAStrided<true,16,256,64,16> d1(2,128,128+64,1024);'
                              ' cudaDMAIndirect<true,true,16,32,64,32> d2(3,128,128+128);'
                              ' cudaDMAHalo<float,4,false,16> d3(4,32,128,128+192,32,16,512);'
                              ' cudaDMACustom d4(5,32,128,128+224);'
                              ' if (d0.owns_this_thread()) d0.execute_dma(x,b);'
                              ' else if (d1.owns_this_thread()) d1.execute_dma(y,b+1024);'
                              ' else if (d2.owns_this_thread()) d2.execute_dma(idx,x,b+2048);'
                              ' else if (d3.owns_this_thread()) d3.execute_dma(x+4*512+4,b+4096+4*40+4);'
                              ' else if (d4.owns_this_thread()) { d4.wait_for_dma_start(); d4.finish_async_dma(); }'
                              ' else { d0.start_async_dma(); d1.start_async_dma(); d2.start_async_dma(); d3.start_async_dma(); d4.start_async_dma();'
                              ' d0.wait_for_dma_finish(); d1.wait_for_dma_finish(); d2.wait_for_dma_finish(); d3.wait_for_dma_finish();'
                              ' d4.wait_for_dma_finish(); y[threadIdx.x]=b[threadIdx.x]; } }\n')
        subprocess.check_call([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-c", "-o",
                               os.path.join(d, "v1.o"), "-I" + os.path.join(ROOT, "include", "cudadma"), src1])
        subprocess.check_call([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-c", "-o",
                               os.path.join(d, "t.o"), "-I" + os.path.join(ROOT, "include", "cudadma"), src])
