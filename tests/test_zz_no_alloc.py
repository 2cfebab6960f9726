"""The stencil entry point that allocates nothing, for solvers that cannot call cudaMalloc from
their time-step loop (all device memory already belongs to their framework's pool, or the
device-wide stall of an allocation would break the overlap of their streams).

It must give exactly what the existing portable entry point gives, call after call: every call
reuses one scratch array built into the library, so the second call here uses a different,
smaller grid and would see the first call's leftovers if the zero border were not re-made.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest
import torch

import cudadma_b200 as cd
from oracle import oracle

pytestmark = pytest.mark.gpu


def one_step_both_ways(nx, ny, nz, seed):
    field = oracle.fill_uniform(nx * ny * nz, seed, 0.0, 1.0)
    inp = torch.from_numpy(field).cuda()
    want = torch.zeros_like(inp)
    cd.stencil25_step(want, inp, nx, ny, nz, impl="portable")   # the existing entry point
    got = torch.full_like(inp, float("nan"))
    cd.stencil25_step_noalloc(got, inp, nx, ny, nz)             # the one under test
    torch.cuda.synchronize()
    assert cd.device_status() == 0
    return field.reshape(nz, ny, nx), want.cpu().numpy(), got.cpu().numpy()


def test_matches_the_portable_entry_point_on_two_calls_in_a_row():
    for nx, ny, nz, seed in ((128, 64, 24, 0xC4), (64, 48, 40, 0xC5)):
        field, want, got = one_step_both_ways(nx, ny, nz, seed)
        # same kernel, same arithmetic: no rounding difference is allowed between the two entry points
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        # and both are the stencil: within the tolerance the other stencil tests use
        exp = oracle.stencil25_f64(field, cd.STENCIL_COEFFS, 1).ravel()
        assert np.abs(got.astype(np.float64) - exp).max() / np.abs(exp).max() <= 1e-5


def test_allocates_no_device_memory_and_honours_its_exact_limit():
    """What the entry point is for: once the library is loaded on the GPU, calls leave the
    device's free memory exactly as it was, on small grids and on the largest grid it takes.
    All tensors are made first, the library's own workspace (which the comparison arm above
    grew) is released, and then free memory is read around the calls."""
    shapes = ((64, 48, 40), (128, 112, 120), (32, 16, 8))     # 128 x 112 x 120 pads to 2 088 960 of 2^21 cells
    ins = [cd.fill_uniform(torch.empty(nx * ny * nz, dtype=torch.float32, device="cuda"), 0xC6 + i, 0.0, 1.0)
           for i, (nx, ny, nz) in enumerate(shapes)]
    outs = [torch.zeros_like(t) for t in ins]
    wants = [torch.zeros_like(t) for t in ins]
    for (nx, ny, nz), i, w in zip(shapes, ins, wants):
        cd.stencil25_step(w, i, nx, ny, nz, impl="portable")
    cd.stencil25_step_noalloc(outs[0], ins[0], *shapes[0])      # warm-up: the one-time address lookup
    torch.cuda.synchronize()
    cd.release_workspace()
    free_before = torch.cuda.mem_get_info()[0]
    launches_before = cd.launch_count()
    for _ in range(3):
        for (nx, ny, nz), i, o in zip(shapes, ins, outs):
            cd.stencil25_step_noalloc(o, i, nx, ny, nz)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "a call allocated or freed device memory"
    assert cd.launch_count() - launches_before == 3 * len(shapes), "one kernel per call"
    assert cd.device_status() == 0
    for o, w in zip(outs, wants):
        assert torch.equal(o.view(torch.int32), w.view(torch.int32))
    # one plane more than the largest grid is refused
    with pytest.raises(cd.CudaDMAError) as e:
        cd.stencil25_step_noalloc(outs[1], ins[1], 128, 112, 121)
    assert e.value.status == -5


def test_rejects_grids_beyond_its_scratch_and_bad_arguments():
    big = torch.zeros(16, dtype=torch.float32, device="cuda")  # never touched: the call must refuse first
    with pytest.raises(cd.CudaDMAError) as e:
        cd.stencil25_step_noalloc(big, big[4:], 512, 512, 64)
    assert e.value.status == -5
    assert b"scratch" in cd.lib().cudadma_status_string(-5)
    with pytest.raises(cd.CudaDMAError) as e:
        cd.stencil25_step_noalloc(big, big[4:], 30, 16, 8)   # nx not a multiple of 32
    assert e.value.status == -1
