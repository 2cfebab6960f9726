"""The sharded stencil's slab step on ONE GPU: several slabs of one process share the device and
its stream (cudadma_stencil25_multi_* with a repeated device entry), so every step runs after the
steps it waits for and nothing ever blocks. The N-slab field must equal the one-slab field bit
for bit. Also here: what happens when a neighbour never arrives (a wait with a short limit on a
flag that nothing sets), the tensor-map helpers, and the device-side input generators against
the oracle's. The two-GPU forms are in tests/test_sharded_gpu.py."""
import ctypes

import numpy as np
import pytest
import torch

import cudadma_b200 as cd
from oracle import oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def one_gpu_field(field, nx, ny, nz, steps):
    a = dev(field)
    b = torch.zeros_like(a)
    return cd.stencil25_run(a, b, nx, ny, nz, steps).cpu().numpy()


# nz / slabs >= 96 takes the form with two 32-plane boundary runs dispatched first; below that, equal runs
@pytest.mark.parametrize("slabs,nx,ny,nz,steps", [(2, 64, 32, 16, 3), (3, 96, 48, 61, 4), (2, 128, 64, 200, 5),
                                                  (4, 64, 64, 400, 3), (8, 32, 32, 64, 6), (2, 36, 20, 230, 2)])
@pytest.mark.parametrize("signal_mode", ["trailing", "trailing-ascending", "fused"])
def test_slabs_of_one_process_equal_the_single_field(slabs, nx, ny, nz, steps, signal_mode):
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)
    want = one_gpu_field(field, nx, ny, nz, steps)
    m = cd.MultiStencil(slabs, nx, ny, nz, devices=[0] * slabs, signal_mode=signal_mode)
    try:
        assert m.planes(0)[0] == 0 and m.planes(slabs - 1)[1] == nz
        m.load(field)
        m.run(steps)
        got = np.full_like(field, np.nan)
        m.store(got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        # the object goes on from where it stands, and a reload starts over
        m.run(1)
        m.store(got)
        assert np.array_equal(got.view(np.uint32), one_gpu_field(field, nx, ny, nz, steps + 1).view(np.uint32))
        m.load(field)
        m.run(steps)
        m.store(got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    finally:
        m.destroy()
    assert cd.device_status() == 0
    exp = oracle.stencil25_f64(field.reshape(nz, ny, nx), cd.STENCIL_COEFFS, steps)
    assert np.abs(want.reshape(nz, ny, nx) - exp).max() / np.abs(exp).max() <= 1e-5


def test_multi_rejects_bad_arguments():
    h = ctypes.c_void_p()
    lib = cd.lib()
    assert lib.cudadma_stencil25_multi_create(ctypes.byref(h), 0, None, 64, 32, 64) == -1
    assert lib.cudadma_stencil25_multi_create(ctypes.byref(h), 4, None, 64, 32, 31) == -1   # fewer than 8 planes per slab
    assert lib.cudadma_stencil25_multi_create(ctypes.byref(h), 1, None, 30, 32, 31) == -1   # nx % 4
    assert lib.cudadma_stencil25_multi_run(None, None, 1) == -1
    assert lib.cudadma_stencil25_multi_destroy(None) == 0


@pytest.mark.parametrize("signal_mode", ["trailing", "trailing-ascending", "fused"])
@pytest.mark.parametrize("nx,ny,nzl", [(64, 32, 24), (512, 512, 100), (256, 256, 300)])
def test_a_neighbour_that_never_arrives_ends_the_step_with_a_status(nx, ny, nzl, signal_mode):
    """Two slabs joined in one process; only the lower one ever steps. Its second step needs the
    upper one to have finished a step, which never happens: the boundary CTAs' wait (limit set
    to a few milliseconds here) runs out, nothing is stored into the upper slab's ghost planes,
    the step count is not published, the status call reports it, later steps are refused, and the
    GPU goes on working. The larger case has 512 boundary CTAs in two 32-plane runs; their DMA
    warps leave without loading anything and their compute threads run through their planes with
    every wait giving up at once. The deepest case has three runs of planes per tile, so that in the
    descending order the run that waits comes last."""
    field = oracle.fill_uniform(nx * ny * nzl, 0xC4, 0.0, 1.0)
    lower, upper = cd.Slab(nx, ny, nzl, False, True), cd.Slab(nx, ny, nzl, True, False)
    try:
        lower.connect_local(None, upper)
        upper.connect_local(lower, None)
        lower.set_signal_mode(signal_mode)
        upper.set_signal_mode(signal_mode)
        lower.set_wait_limit(4_000_000)   # about two milliseconds of SM clocks
        lower.tensor(0).view(nzl + 8, ny, nx)[4:4 + nzl] = dev(field).view(nzl, ny, nx)
        lower.step()                       # step 0 waits for nothing: it pushes and publishes
        assert lower.status() == cd.capi.OK
        up_flags_after_first = [upper.tensor(w).clone() for w in (0, 1)]
        assert up_flags_after_first[1].view(nzl + 8, ny, nx)[:4].any(), "the first step's planes arrived in the ghost planes"
        lower.step()                       # needs the upper slab to have finished one step
        assert lower.status() == cd.capi.ERR_TIMEOUT
        word = cd.device_status()
        assert word & 0x80000000 and (word & 0xF000) == 0xE000 and (word & 1) == 1, hex(word)
        for w in (0, 1):                   # nothing of the failed step reached the neighbour
            assert torch.equal(upper.tensor(w), up_flags_after_first[w])
        assert cd.lib().cudadma_slab_step(lower._h, (ctypes.c_float * 5)(*cd.STENCIL_COEFFS), None) == cd.capi.ERR_TIMEOUT
        # the context is intact: the plain stencil still runs and is right
        got = one_gpu_field(field, nx, ny, nzl, 2)
        exp = oracle.stencil25_f64(field.reshape(nzl, ny, nx), cd.STENCIL_COEFFS, 2)
        assert np.abs(got.reshape(nzl, ny, nx) - exp).max() / np.abs(exp).max() <= 1e-5
        assert cd.device_status() == 0
    finally:
        lower.destroy()
        upper.destroy()


def test_device_generators_equal_the_oracle_generators():
    n = (1 << 20) + 37
    for seed, lo, hi in ((0xC1, -1.0, 1.0), (0xC4, 0.0, 1.0)):
        got = cd.fill_uniform(torch.empty(n, dtype=torch.float32, device="cuda"), seed, lo, hi).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), oracle.fill_uniform(n, seed, lo, hi).view(np.uint32))
    # a piece of a field equals the same range of the whole
    piece = cd.fill_uniform(torch.empty(1000, dtype=torch.float32, device="cuda"), 0xC4, 0.0, 1.0, first_index=12345)
    assert np.array_equal(piece.cpu().numpy(), oracle.fill_uniform(n, 0xC4, 0.0, 1.0)[12345:13345])
    idx = cd.fill_index(torch.empty(n, dtype=torch.int32, device="cuda"), 0xC3A, 1 << 24).cpu().numpy()
    assert np.array_equal(idx, oracle.fill_index(n, 0xC3A, 1 << 24))
    probe = torch.zeros(2, dtype=torch.int64, device="cuda")
    cd.clock_probe(probe, 200_000)
    cycles, ns = probe.cpu().tolist()
    assert ns >= 200_000 and 100.0 < cycles / ns * 1e3 < 3000.0   # an SM clock in MHz


def test_tensor_map_helpers():
    a = torch.zeros(256 * 128, dtype=torch.float32, device="cuda")
    m2 = cd.make_tensor_map_2d(a, 128, 256, 128 * 4, 32, 128, True)
    m3 = cd.make_tensor_map_3d(a, 64, 32, 16, 64 * 4, 64 * 32 * 4, 40, 24, 1)
    assert len(m2) == 128 and len(m3) == 128 and m2 != m3 and any(m2) and any(m3)
    bad = [(a, 128, 256, 128 * 4 + 4, 32, 128, False),    # pitch not a multiple of 16
           (a, 128, 256, 128 * 4, 33, 128, False),        # box width not a multiple of 16 bytes
           (a, 128, 256, 128 * 4, 64, 128, True),         # 128-byte swizzle with a 256-byte box row
           (a, 128, 256, 64 * 4, 32, 128, False),         # pitch shorter than a row
           (a.data_ptr() + 4, 128, 256, 128 * 4, 32, 128, False)]
    for args in bad:
        with pytest.raises(cd.CudaDMAError) as e:
            cd.make_tensor_map_2d(*args)
        assert e.value.status == -1
    with pytest.raises(cd.CudaDMAError):
        cd.make_tensor_map_3d(a, 64, 32, 16, 64 * 4, 64 * 16 * 4, 40, 24, 1)   # plane pitch shorter than a plane
