"""Host logic of the z-sharded stencil on CPU ranks (gloo, world size 2 and 3):
slab bounds, ghost-plane exchange and the boundary/interior split. The step
function is the CPU oracle here (test infrastructure); the product's step
function is the CUDA kernel and is covered by the GPU tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cudadma_b200 import sharded
from oracle import oracle

COEFF = (-2.847, 1.6, -0.2, 0.0254, -0.00179)


def test_slab_bounds_cover_the_grid():
    for nz in (8, 9, 33, 2048):
        for world in (1, 2, 3, 8):
            b = [sharded.slab_bounds(nz, world, r) for r in range(world)]
            assert b[0][0] == 0 and b[-1][1] == nz
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            assert max(h - l for l, h in b) - min(h - l for l, h in b) <= 1


def test_refuses_to_run_without_cuda_or_step_function():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(RuntimeError):
        sharded.ShardedStencil(32, 16, 16)


def oracle_step(out, inp, nx, ny, nz_total, z_begin, z_end, coeff):
    """Planes [z_begin, z_end) of one fp32 step on the local array (ghosts included as data)."""
    full = oracle.stencil25_step_f32(inp.numpy().reshape(nz_total, ny, nx), coeff)
    out.view(nz_total, ny, nx)[z_begin:z_end] = torch.from_numpy(full[z_begin:z_end])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, nx, ny, nz, steps, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
        st = sharded.ShardedStencil(nx, ny, nz, COEFF, device="cpu", step_fn=oracle_step)
        st.load(torch.from_numpy(field[st.z_lo:st.z_hi].copy()))
        got = st.run(steps).numpy().copy()
        q.put((rank, st.z_lo, st.z_hi, got))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,nz", [(2, 24), (3, 29), (2, 9)])
def test_sharded_equals_single_rank_bit_for_bit(world, nz):
    nx, ny, steps = 16, 12, 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, nx, ny, nz, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    parts = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
    cur = field
    for _ in range(steps):
        cur = oracle.stencil25_step_f32(cur, COEFF)
    for rank, lo, hi, got in parts:
        assert np.array_equal(got.view(np.uint32), cur[lo:hi].view(np.uint32)), "rank %d differs" % rank
