"""Parity of the four single-GPU workloads, called through the C ABI, with the
CPU oracle: bit-exact for copy, transpose and gather/scatter; within 1e-5
(max |gpu - ref| / max |ref|) of the double-precision oracle for the stencil.
Small cases are compared element by element; the full benchmark sizes are
checked through properties that do not need the oracle to walk them twice.
"""
import numpy as np
import pytest
import torch

import cudadma_b200 as cd
from oracle import oracle

pytestmark = pytest.mark.gpu
IMPLS = ("native", "portable")
STENCIL_TOL = 1e-5  # L-infinity relative, the tolerance the benchmark states


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def status_clean():
    assert cd.device_status() == 0


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("nbytes,chunk", [(16384, 16384), (16384 * 37, 16384), (16384 * 300 + 4096 + 8, 16384),
                                          (4, 16384), (1 << 20, 4096), (100000, 1008)])
def test_seq_copy_small(impl, nbytes, chunk):
    src = oracle.fill_uniform(nbytes // 4, 0xC1, -1.0, 1.0)
    d_src = dev(src)
    d_dst = torch.zeros(nbytes // 4 + 64, dtype=torch.float32, device="cuda")
    cd.seq_copy(d_dst, d_src, nbytes, chunk, impl)
    status_clean()
    out = d_dst.cpu().numpy()
    exp = oracle.chunked_copy(src, chunk)
    assert np.array_equal(out[:nbytes // 4].view(np.uint32), exp.view(np.uint32))
    assert not out[nbytes // 4:].any(), "wrote past the end"


def test_seq_copy_rejects_bad_arguments():
    t = torch.zeros(1024, dtype=torch.float32, device="cuda")
    for args in ((t, t, 6, 16384), (t, t, 64, 100), (t, t, 64, 32768)):
        with pytest.raises(cd.CudaDMAError) as e:
            cd.seq_copy(*args)
        assert e.value.status == -1
    # misaligned pointer, null pointer, overlapping stencil buffers
    assert cd.lib().cudadma_seq_copy(t.data_ptr() + 4, t.data_ptr(), 64, 16384, 0, None) == -1
    assert cd.lib().cudadma_seq_copy(None, t.data_ptr(), 64, 16384, 0, None) == -1
    with pytest.raises(cd.CudaDMAError):
        cd.stencil25_step(t, t, 16, 8, 8)
    with pytest.raises(cd.CudaDMAError):
        cd.gather_scatter(t, t, t, t, 100, 32)


@pytest.mark.parametrize("impl", IMPLS)
def test_seq_copy_full_size(impl):
    """64 MiB, 16 KiB chunks: the benchmark's configuration, compared on the device with the source."""
    n = 1 << 24
    d_src = dev(oracle.fill_uniform(n, 0xC1, -1.0, 1.0))
    d_dst = torch.zeros_like(d_src)
    cd.seq_copy(d_dst, d_src, n * 4, 16384, impl)
    status_clean()
    assert torch.equal(d_dst.view(torch.int32), d_src.view(torch.int32))


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("rows,cols", [(128, 64), (256, 192), (1024, 2048), (128 * 7, 64 * 37)])
def test_transpose_small(impl, rows, cols):
    src = oracle.fill_uniform(rows * cols, 0xC2, -1.0, 1.0).reshape(rows, cols)
    d_src = dev(src)
    d_dst = torch.zeros(cols * rows + 64, dtype=torch.float32, device="cuda")
    cd.strided_transpose(d_dst, d_src, rows, cols, impl)
    status_clean()
    out = d_dst.cpu().numpy()
    exp = oracle.tile_transpose(src)
    assert np.array_equal(out[:rows * cols].view(np.uint32), exp.ravel().view(np.uint32))
    assert not out[rows * cols:].any()


@pytest.mark.parametrize("impl", IMPLS)
def test_transpose_full_size_is_an_involution(impl):
    """16384 x 16384: transposing twice gives the input back, and one transpose matches torch's."""
    n = 16384
    d_src = torch.empty(n * n, dtype=torch.float32, device="cuda")
    # seeded fill made on the device in pieces to keep host memory small
    piece = 1 << 26
    for i in range(0, n * n, piece):
        d_src[i:i + piece] = dev(oracle.fill_uniform(piece, 0xC2 + i, -1.0, 1.0))
    d_t = torch.empty_like(d_src)
    cd.strided_transpose(d_t, d_src, n, n, impl)
    status_clean()
    assert torch.equal(d_t.view(n, n), d_src.view(n, n).t())
    d_back = torch.empty_like(d_src)
    cd.strided_transpose(d_back, d_t, n, n, impl)
    assert torch.equal(d_back, d_src)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("n,table_records", [(128, 1000), (128 * 5, 128 * 5), (128 * 333, 1 << 16), (1 << 16, 1 << 20)])
def test_gather_scatter_small(impl, n, table_records):
    table = oracle.fill_uniform(table_records * 8, 0xC3, -1.0, 1.0)
    gidx = oracle.fill_index(n, 0xC3A, table_records)
    sidx = oracle.permutation(n, 0xC3B)
    d_out = torch.zeros(n * 8 + 64, dtype=torch.float32, device="cuda")
    cd.gather_scatter(d_out, dev(table), dev(gidx), dev(sidx), n, 32, impl)
    status_clean()
    out = d_out.cpu().numpy()
    exp = oracle.gather_scatter(np.zeros(n * 8, dtype=np.float32), table, gidx, sidx, 32)
    assert np.array_equal(out[:n * 8].view(np.uint32), exp.view(np.uint32))
    assert not out[n * 8:].any()


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("record_bytes", [16, 64, 128])
@pytest.mark.parametrize("n,table_records", [(128, 77), (128 * 41, 1 << 14), (1 << 15, 1 << 18)])
def test_gather_scatter_record_sizes(impl, record_bytes, n, table_records):
    """Records of 16, 64 and 128 bytes go through the same pipeline (the benchmark's size is 32)."""
    w = record_bytes // 4
    table = oracle.fill_uniform(table_records * w, 0xC30 + record_bytes, -1.0, 1.0)
    gidx = oracle.fill_index(n, 0xC3A, table_records)
    sidx = oracle.permutation(n, 0xC3B)
    d_out = torch.zeros(n * w + 64, dtype=torch.float32, device="cuda")
    cd.gather_scatter(d_out, dev(table), dev(gidx), dev(sidx), n, record_bytes, impl)
    status_clean()
    out = d_out.cpu().numpy()
    exp = oracle.gather_scatter(np.zeros(n * w, dtype=np.float32), table, gidx, sidx, record_bytes)
    assert np.array_equal(out[:n * w].view(np.uint32), exp.view(np.uint32))
    assert not out[n * w:].any()


@pytest.mark.parametrize("mode", [1, 2, 3])
@pytest.mark.parametrize("n,table_records", [(128, 1000), (128 * 333, 1 << 16), (1 << 16, 1 << 20)])
def test_gather_scatter_tma_rows(n, table_records, mode):
    """The TMA forms (row gathers, row scatters, both) give the same bytes."""
    table = oracle.fill_uniform(table_records * 8, 0xC3, -1.0, 1.0)
    gidx = oracle.fill_index(n, 0xC3A, table_records)
    sidx = oracle.permutation(n, 0xC3B)
    d_out = torch.zeros(n * 8 + 64, dtype=torch.float32, device="cuda")
    cd.gather_scatter_tma(d_out, n, dev(table), table_records, dev(gidx), dev(sidx), n, 32, mode)
    status_clean()
    out = d_out.cpu().numpy()
    exp = oracle.gather_scatter(np.zeros(n * 8, dtype=np.float32), table, gidx, sidx, 32)
    assert np.array_equal(out[:n * 8].view(np.uint32), exp.view(np.uint32))
    assert not out[n * 8:].any()


@pytest.mark.parametrize("impl", IMPLS)
def test_gather_scatter_full_size(impl):
    """2^24-record table, 2^22 indices: every output slot holds the record its index names
    (checked on the device through the inverse permutation)."""
    n, records = 1 << 22, 1 << 24
    d_table = torch.empty(records * 8, dtype=torch.float32, device="cuda")
    piece = 1 << 25
    for i in range(0, records * 8, piece):
        d_table[i:i + piece] = dev(oracle.fill_uniform(piece, 0xC3 + i, -1.0, 1.0))
    d_g = dev(oracle.fill_index(n, 0xC3A, records))
    d_s = dev(oracle.permutation(n, 0xC3B))
    d_out = torch.zeros(n * 8, dtype=torch.float32, device="cuda")
    cd.gather_scatter(d_out, d_table, d_g, d_s, n, 32, impl)
    status_clean()
    exp = torch.empty(n, 8, dtype=torch.float32, device="cuda")
    exp[d_s.long()] = d_table.view(records, 8)[d_g.long()]
    assert torch.equal(d_out.view(n, 8).view(torch.int32), exp.view(torch.int32))


def rel_err(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / np.abs(b).max())


@pytest.mark.parametrize("nx,ny,nz,steps", [(32, 16, 8, 1), (64, 48, 40, 3), (96, 80, 33, 2), (36, 20, 19, 2),
                                            (128, 64, 72, 10)])
def test_stencil_small(nx, ny, nz, steps):
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
    a = dev(field)
    b = torch.zeros_like(a)
    res = cd.stencil25_run(a, b, nx, ny, nz, steps)
    status_clean()
    exp = oracle.stencil25_f64(field, cd.STENCIL_COEFFS, steps)
    assert rel_err(res.cpu().numpy(), exp) <= STENCIL_TOL


@pytest.mark.parametrize("nx,ny,nz,steps", [(32, 16, 8, 1), (64, 48, 40, 3), (128, 64, 33, 4)])
def test_stencil_portable(nx, ny, nz, steps):
    """The reference-API kernel (padded arrays, CudaDMAStrided window loads) through the same entry point."""
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
    a = dev(field)
    b = torch.zeros_like(a)
    res = cd.stencil25_run(a, b, nx, ny, nz, steps, impl="portable")
    status_clean()
    exp = oracle.stencil25_f64(field, cd.STENCIL_COEFFS, steps)
    assert rel_err(res.cpu().numpy(), exp) <= STENCIL_TOL
    # and one step on a plane range, through the padded entry point
    pad = torch.zeros((nz + 8, ny + 8, nx + 8), dtype=torch.float32, device="cuda")
    pad[4:-4, 4:-4, 4:-4] = dev(field)
    out = torch.zeros_like(pad)
    cd.stencil25_step_padded(out, pad, nx, ny, nz, 1, nz - 1)
    status_clean()
    one = oracle.stencil25_f64(field, cd.STENCIL_COEFFS, 1)
    got = out[4:-4, 4:-4, 4:-4].cpu().numpy()
    assert rel_err(got[1:nz - 1], one[1:nz - 1]) <= STENCIL_TOL
    assert not got[0].any() and not got[nz - 1].any()
    assert not out[:4].any() and not out[:, :4].any() and not out[:, :, :4].any(), "wrote into the border"


def test_stencil_plane_ranges_compose():
    """Computing [0, k) and [k, nz) separately equals one full step bit for bit (what the sharded driver relies on)."""
    nx, ny, nz = 64, 32, 50
    a = dev(oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0))
    full = torch.zeros_like(a)
    cd.stencil25_step(full, a, nx, ny, nz)
    parts = torch.zeros_like(a)
    cd.stencil25_step(parts, a, nx, ny, nz, 0, 4)
    cd.stencil25_step(parts, a, nx, ny, nz, 4, 46, z_chunk=7)
    cd.stencil25_step(parts, a, nx, ny, nz, 46, 50)
    status_clean()
    assert torch.equal(full.view(torch.int32), parts.view(torch.int32))


def test_slab_interface_without_neighbours_is_the_plain_stencil():
    """The slab calls of the sharded driver on a rank with no neighbour on either side: same field, bit for bit,
    as the plain ping-pong run (the two-rank forms of it are in tests/test_sharded_gpu.py)."""
    nx, ny, nz, steps = 96, 48, 21, 4
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)
    slab = cd.Slab(nx, ny, nz, False, False)
    try:
        assert len(slab.export()) == cd.lib().cudadma_slab_handle_bytes()
        cur = slab.tensor(0).view(nz + 8, ny, nx)
        assert not cur.any()
        cur[4:4 + nz] = dev(field).view(nz, ny, nx)
        for _ in range(steps):
            slab.step()
        got = slab.tensor(0).view(nz + 8, ny, nx)
        a = dev(field)
        want = cd.stencil25_run(a, torch.zeros_like(a), nx, ny, nz, steps).view(nz, ny, nx)
        status_clean()
        assert torch.equal(got[4:4 + nz].view(torch.int32), want.view(torch.int32))
        assert not got[:4].any() and not got[4 + nz:].any(), "ghost planes of a rank without neighbours stay zero"
    finally:
        slab.destroy()
    with pytest.raises(cd.CudaDMAError):
        cd.Slab(nx, ny, 4, True, False)  # a rank with a neighbour needs at least eight planes


def test_stencil_full_size_linearity_and_sample():
    """512^3, 10 steps. The operator is linear: stepping 2u equals twice stepping u exactly (scaling by two is exact
    in fp32), and a slab of the one-step result is compared with the double-precision oracle."""
    n = 512
    field = oracle.fill_uniform(n * n * n, 0xC4, 0.0, 1.0)
    a = dev(field)
    b = torch.zeros_like(a)
    a2 = a * 2.0
    b2 = torch.zeros_like(a)
    r1 = cd.stencil25_run(a, b, n, n, n, 10)
    r2 = cd.stencil25_run(a2, b2, n, n, n, 10)
    status_clean()
    assert torch.equal((r1 * 2.0).view(torch.int32), r2.view(torch.int32))
    del a2, b2, r2
    # one step on a 24-plane slab at the top of the grid against the oracle (out-of-grid planes read as zero)
    slab = field.reshape(n, n, n)[:28]
    exp = oracle.stencil25_f64(np.ascontiguousarray(slab), cd.STENCIL_COEFFS, 1)[:24]
    a = dev(field)
    cd.stencil25_step(b, a, n, n, n, 0, 24)
    got = b.view(n, n, n)[:24].cpu().numpy()
    assert rel_err(got, exp) <= STENCIL_TOL


def test_stencil_full_job_against_the_double_precision_oracle():
    """The benchmark's single-GPU stencil job whole: 512^3, 10 steps, every point of the final field
    against the double-precision host reference (max |gpu - ref| / max |ref| <= 1e-5)."""
    n, steps = 512, 10
    field = oracle.fill_uniform(n * n * n, 0xC4, 0.0, 1.0)
    a = cd.fill_uniform(torch.empty(n * n * n, dtype=torch.float32, device="cuda"), 0xC4, 0.0, 1.0)
    assert torch.equal(a.view(torch.int32), dev(field).view(torch.int32)), "device and host generators agree"
    b = torch.zeros_like(a)
    got = cd.stencil25_run(a, b, n, n, n, steps).cpu().numpy().reshape(n, n, n)
    status_clean()
    exp = oracle.stencil25_f64(field.reshape(n, n, n), cd.STENCIL_COEFFS, steps)
    assert rel_err(got, exp) <= STENCIL_TOL


def test_host_buffer_forms_match_device_forms():
    n = 16384 * 9
    src = oracle.fill_uniform(n // 4, 0xC1, -1.0, 1.0)
    out = np.zeros_like(src)
    cd.seq_copy_host(out, src, n)
    assert np.array_equal(out.view(np.uint32), src.view(np.uint32))
    m = oracle.fill_uniform(256 * 128, 0xC2, -1.0, 1.0).reshape(256, 128)
    t = np.zeros((128, 256), dtype=np.float32)
    cd.strided_transpose_host(t, m, 256, 128)
    assert np.array_equal(t, m.T)
    table = oracle.fill_uniform(4096 * 8, 0xC3, -1.0, 1.0)
    g = oracle.fill_index(1280, 0xC3A, 4096)
    s = oracle.permutation(1280, 0xC3B)
    o = np.zeros(1280 * 8, dtype=np.float32)
    cd.gather_scatter_host(o, 1280, table, 4096, g, s, 1280)
    assert np.array_equal(o, oracle.gather_scatter(np.zeros_like(o), table, g, s))
    f = oracle.fill_uniform(64 * 32 * 20, 0xC4, 0.0, 1.0).reshape(20, 32, 64)
    r = np.zeros_like(f)
    cd.stencil25_run_host(r, f, 64, 32, 20, 3)
    assert rel_err(r, oracle.stencil25_f64(f, cd.STENCIL_COEFFS, 3)) <= STENCIL_TOL
    cd.release_workspace()


@pytest.mark.parametrize("nx,ny,nz,steps,chunk", [(64, 48, 120, 3, 16), (36, 20, 50, 2, 7), (32, 16, 40, 4, 1),
                                                  (64, 32, 30, 5, 64), (128, 64, 200, 6, 24), (32, 16, 9, 1, 4)])
def test_stencil_host_run_overlapped_is_the_plain_run(nx, ny, nz, steps, chunk):
    """Upload, steps and download overlapped in pieces of `chunk` planes: the same bits as the plain
    upload / run / download sequence, from pinned and from pageable host memory, and in place."""
    f = oracle.fill_uniform(nx * ny * nz, 0xC4 + nz, 0.0, 1.0)
    d_a, d_b = dev(f), torch.zeros(nx * ny * nz, dtype=torch.float32, device="cuda")
    cd.stencil25_run(d_a, d_b, nx, ny, nz, steps)
    exp = (d_b if steps & 1 else d_a).cpu().numpy()
    got = np.full_like(f, np.nan)
    cd.stencil25_run_host(got, f, nx, ny, nz, steps, chunk_planes=chunk)
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))
    h_in = torch.from_numpy(f).pin_memory()
    h_out = torch.full((nx * ny * nz,), float("nan")).pin_memory()
    cd.stencil25_run_host(h_out, h_in, nx, ny, nz, steps, chunk_planes=chunk)
    assert np.array_equal(h_out.numpy().view(np.uint32), exp.view(np.uint32))
    cd.stencil25_run_host(h_in, h_in, nx, ny, nz, steps, chunk_planes=chunk)
    assert np.array_equal(h_in.numpy().view(np.uint32), exp.view(np.uint32))
    status_clean()
    assert rel_err(exp.reshape(nz, ny, nx), oracle.stencil25_f64(f.reshape(nz, ny, nx), cd.STENCIL_COEFFS, steps)) <= STENCIL_TOL


def test_stencil_host_run_library_pieces_on_the_512_cube():
    """The benchmark's single-GPU stencil (512^3, 10 steps) from and to pinned host memory with the
    library's own piece size: the overlapped form is taken (four pieces of 128 planes) and gives
    the bits of the device-resident run."""
    nx = ny = nz = 512
    steps = 10
    h_in = torch.empty(nx * ny * nz, dtype=torch.float32).pin_memory()
    h_in.copy_(torch.from_numpy(oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)))
    h_out = torch.full((nx * ny * nz,), float("nan")).pin_memory()
    cd.stencil25_run_host(h_out, h_in, nx, ny, nz, steps)
    d_a, d_b = h_in.cuda(), torch.zeros(nx * ny * nz, dtype=torch.float32, device="cuda")
    cd.stencil25_run(d_a, d_b, nx, ny, nz, steps)
    want = d_b if steps & 1 else d_a
    assert torch.equal(h_out.cuda().view(torch.int32), want.view(torch.int32))
    status_clean()
    cd.release_workspace()
