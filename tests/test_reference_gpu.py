"""Device-side parity with the REFERENCE CudaDMA classes compiled for sm_100a
(oracle/_ref/libcudadma_ref.so, built from the reference checkout where it is
present): the same portable kernel source runs against the reference headers
and against this repository's header on the same seeded inputs, and the two
device results must agree bit for bit -- for the stencil too, since the
arithmetic is the same source. Skipped where the reference build is absent."""
import numpy as np
import pytest
import torch

import cudadma_b200 as cd
from oracle import oracle
from oracle import reference as ref

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref.available(), reason="reference build not present")]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_sequential_matches_reference_build():
    n = 16384 * 123
    src = dev(oracle.fill_uniform(n // 4, 0xC1, -1.0, 1.0))
    a, b, c = (torch.zeros_like(src) for _ in range(3))
    ref.seq_copy(a, src, n)
    cd.seq_copy(b, src, n, 16384, "portable")
    cd.seq_copy(c, src, n, 16384, "native")
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    assert torch.equal(a.view(torch.int32), c.view(torch.int32))
    assert torch.equal(a.view(torch.int32), src.view(torch.int32))


def test_strided_matches_reference_build():
    rows, cols = 1024, 1536
    src = dev(oracle.fill_uniform(rows * cols, 0xC2, -1.0, 1.0))
    a, b, c = (torch.zeros_like(src) for _ in range(3))
    ref.strided_transpose(a, src, rows, cols)
    cd.strided_transpose(b, src, rows, cols, "portable")
    cd.strided_transpose(c, src, rows, cols, "native")
    assert torch.equal(a, b) and torch.equal(a, c)
    assert torch.equal(a.view(cols, rows), src.view(rows, cols).t())


def test_gather_scatter_matches_reference_build():
    n, records = 128 * 777, 1 << 18
    table = dev(oracle.fill_uniform(records * 8, 0xC3, -1.0, 1.0))
    g = dev(oracle.fill_index(n, 0xC3A, records))
    s = dev(oracle.permutation(n, 0xC3B))
    a, b, c = (torch.zeros(n * 8, dtype=torch.float32, device="cuda") for _ in range(3))
    ref.gather_scatter(a, table, g, s, n)
    cd.gather_scatter(b, table, g, s, n, 32, "portable")
    cd.gather_scatter(c, table, g, s, n, 32, "native")
    exp = oracle.gather_scatter(np.zeros(n * 8, dtype=np.float32), table.cpu().numpy(), g.cpu().numpy(),
                                s.cpu().numpy())
    assert np.array_equal(b.cpu().numpy().view(np.uint32), exp.view(np.uint32))
    assert torch.equal(b, c)
    if not torch.equal(a, b):
        # The reference's warp-specialised execute_dma loads its source before it waits for the compute
        # threads' start signal (start_xfer_async precedes wait_for_dma_start, include/cudaDMAv2.h:1461-1475).
        # That is harmless for a gather from global memory, but the scatter object then reads the shared
        # buffer before the gather that fills it has been handed over. No reference test runs a scatter.
        pytest.xfail("reference scatter reads its shared-memory source before the handshake")


def test_stencil_matches_reference_build():
    if not hasattr(ref.lib(), "cudadma_ref_stencil25_step_padded"):
        pytest.skip("reference build has no stencil kernel")
    nx, ny, nz = 128, 64, 40
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
    pad = torch.zeros((nz + 8, ny + 8, nx + 8), dtype=torch.float32, device="cuda")
    pad[4:-4, 4:-4, 4:-4] = dev(field)
    a, b = torch.zeros_like(pad), torch.zeros_like(pad)
    ref.stencil25_step_padded(a, pad, nx, ny, nz, 0, nz, cd.STENCIL_COEFFS)
    cd.stencil25_step_padded(b, pad, nx, ny, nz, 0, nz)
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    exp = oracle.stencil25_f64(field, cd.STENCIL_COEFFS, 1)
    got = a[4:-4, 4:-4, 4:-4].cpu().numpy()
    assert np.abs(got - exp).max() / np.abs(exp).max() <= 1e-5


@pytest.mark.parametrize("bpt", ref.BPTS)
def test_every_staging_budget_of_the_reference_arm_gives_the_same_bits(bpt):
    """The reference arm of the benchmark tries BYTES_PER_THREAD = 64, 128 and 192 and keeps the fastest:
    each must be the same copy, transpose and stencil."""
    n = 16384 * 40
    src = dev(oracle.fill_uniform(n // 4, 0xC1, -1.0, 1.0))
    a = torch.zeros_like(src)
    ref.seq_copy(a, src, n, bpt)
    assert torch.equal(a.view(torch.int32), src.view(torch.int32))
    rows, cols = 256, 192
    m = dev(oracle.fill_uniform(rows * cols, 0xC2, -1.0, 1.0))
    t = torch.zeros_like(m)
    ref.strided_transpose(t, m, rows, cols, bpt)
    assert torch.equal(t.view(cols, rows), m.view(rows, cols).t())
    nx, ny, nz = 64, 32, 20
    pad = torch.zeros((nz + 8, ny + 8, nx + 8), dtype=torch.float32, device="cuda")
    pad[4:-4, 4:-4, 4:-4] = dev(oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)).view(nz, ny, nx)
    x, y = torch.zeros_like(pad), torch.zeros_like(pad)
    ref.stencil25_step_padded(x, pad, nx, ny, nz, 0, nz, cd.STENCIL_COEFFS, 0, bpt)
    cd.stencil25_step_padded(y, pad, nx, ny, nz, 0, nz)
    assert torch.equal(x.view(torch.int32), y.view(torch.int32))


def test_halo_ring_stencil_matches_on_both_headers():
    """oracle/ref_halo_stencil.cu: ring by v1 cudaDMAHalo, interior by cudaDMAStrided. Built against the
    reference's v1 header and against this repository's header it gives the same bits, and those are the
    bits of the window-loading stencil (same arithmetic source)."""
    import os
    ours_path = os.path.join(os.path.dirname(ref.HALO_STENCIL_PATH), "libhalo_stencil_ours.so")
    if not (ref.halo_stencil_available() and os.path.exists(ours_path)):
        pytest.skip("halo stencil libraries not built")
    ours = ref.halo_lib(ours_path)
    for nx, ny, nz, zb, ze in ((64, 32, 20, 0, 20), (128, 64, 41, 3, 38), (32, 16, 9, 0, 9)):
        pad = torch.zeros((nz + 8, ny + 8, nx + 8), dtype=torch.float32, device="cuda")
        pad[4:-4, 4:-4, 4:-4] = dev(oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)).view(nz, ny, nx)
        a, b, c = (torch.zeros_like(pad) for _ in range(3))
        ref.halo_stencil25_step_padded(a, pad, nx, ny, nz, zb, ze, cd.STENCIL_COEFFS)
        ref.halo_stencil25_step_padded(b, pad, nx, ny, nz, zb, ze, cd.STENCIL_COEFFS, lib_handle=ours)
        cd.stencil25_step_padded(c, pad, nx, ny, nz, zb, ze)
        torch.cuda.synchronize()
        assert torch.equal(b.view(torch.int32), c.view(torch.int32)), "this header: ring + interior against whole windows"
        assert torch.equal(a.view(torch.int32), c.view(torch.int32)), "reference header"
    w = __import__("ctypes").c_uint(0)
    assert ours.halo_stencil_status(__import__("ctypes").byref(w)) == 0 and w.value == 0
