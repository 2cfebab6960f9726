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


def test_weighted_slab_bounds():
    """Slabs in proportion to the ranks' speeds: they cover the grid, respect the minimum depth,
    follow the weights, and equal weights give (nearly) the even cut."""
    for nz, w, least in ((2048, [1.0, 0.9, 1.1, 1.0, 0.95, 1.05, 1.0, 1.0], 8), (64, [5.0, 1.0, 1.0], 8),
                         (24, [1.0, 100.0, 1.0], 8), (33, [1.0, 1.0], 1)):
        b = [sharded.slab_bounds(nz, len(w), r, w, least) for r in range(len(w))]
        assert b[0][0] == 0 and b[-1][1] == nz
        assert all(b[i][1] == b[i + 1][0] for i in range(len(w) - 1))
        assert all(h - l >= least for l, h in b)
    b = [sharded.slab_bounds(2048, 4, r, [1.0, 2.0, 1.0, 4.0], 8) for r in range(4)]
    assert [h - l for l, h in b] == [256, 512, 256, 1024]
    even = [sharded.slab_bounds(2048, 8, r) for r in range(8)]
    assert [sharded.slab_bounds(2048, 8, r, [3.0] * 8, 8) for r in range(8)] == even
    with pytest.raises(ValueError):
        sharded.slab_bounds(16, 4, 0, [1.0] * 4, 8)
    with pytest.raises(ValueError):
        sharded.slab_bounds(64, 2, 0, [1.0, 0.0], 8)


def test_binding_near_a_gpu_is_harmless_without_one():
    """Without NVML or a device the helper leaves the process as it was and says so."""
    before = os.sched_getaffinity(0)
    cores = sharded.bind_host_thread_near_gpu(0)
    after = os.sched_getaffinity(0)
    if cores is None:
        assert after == before
    else:
        assert cores and set(cores) == set(after) and set(after) <= set(before)
        os.sched_setaffinity(0, before)


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


def _worker(rank, world, port, nx, ny, nz, steps, q, weights=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
        st = sharded.ShardedStencil(nx, ny, nz, COEFF, device="cpu", step_fn=oracle_step, weights=weights)
        st.load(torch.from_numpy(field[st.z_lo:st.z_hi].copy()))
        got = st.run(steps).numpy().copy()
        q.put((rank, st.z_lo, st.z_hi, got))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,nz,weights", [(2, 24, None), (3, 29, None), (2, 9, None), (3, 40, (1.0, 2.0, 1.5))])
def test_sharded_equals_single_rank_bit_for_bit(world, nz, weights):
    nx, ny, steps = 16, 12, 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, nx, ny, nz, steps, q, weights)) for r in range(world)]
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


def _lost_neighbour_worker(rank, world, port, q, release):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nx, ny, nz = 16, 12, 24
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
    st = sharded.ShardedStencil(nx, ny, nz, COEFF, device="cpu", step_fn=oracle_step, exchange_timeout=2.0)
    st.load(torch.from_numpy(field[st.z_lo:st.z_hi].copy()))
    st.step()
    if rank == 1:
        # this rank stops taking part after the first step, without leaving the group
        q.put((rank, "idle"))
        release.wait(300)  # stays alive, and silent, until the other rank has given up on it
        os._exit(0)
    try:
        st.step()
        q.put((rank, "no error"))
    except sharded.ExchangeError as e:
        q.put((rank, "ExchangeError: %s" % e))
    q.close()
    q.join_thread()  # put() only hands the item to a feeder thread: let it reach the pipe before leaving
    os._exit(0)  # the group is not usable after a lost exchange; leave without its teardown


def test_lost_neighbour_is_reported_by_the_exchange_deadline():
    """A rank whose z-neighbour stops stepping gets ExchangeError from step() within the deadline
    instead of waiting for ever (the failure is made on the host: the other rank just idles)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    release = ctx.Event()
    procs = [ctx.Process(target=_lost_neighbour_worker, args=(r, 2, port, q, release)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=240) for _ in range(2))
    release.set()
    for p in procs:
        p.join(timeout=30)
    assert got[1] == "idle"
    assert got[0].startswith("ExchangeError: rank 0, step 2"), got[0]


def _checkpoint_worker(rank, world, port, tmpdir, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        nx, ny, nz = 16, 12, 26
        field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
        path = os.path.join(tmpdir, "slab%d.bin" % rank)
        a = sharded.ShardedStencil(nx, ny, nz, COEFF, device="cpu", step_fn=oracle_step)
        a.load(torch.from_numpy(field[a.z_lo:a.z_hi].copy()))
        a.run(2)
        a.save(path)
        straight = a.run(2).numpy().copy()
        b = sharded.ShardedStencil(nx, ny, nz, COEFF, device="cpu", step_fn=oracle_step)
        b.restore(path)
        resumed_at = b.steps_done
        resumed = b.run(2).numpy().copy()
        wrong = sharded.ShardedStencil(nx, ny, nz + 2, COEFF, device="cpu", step_fn=oracle_step)
        try:
            wrong.restore(path)
            refused = False
        except ValueError:
            refused = True
        q.put((rank, resumed_at, b.steps_done, bool(np.array_equal(straight.view(np.uint32), resumed.view(np.uint32))), refused))
    finally:
        dist.destroy_process_group()


def test_checkpoint_restart_continues_bit_for_bit(tmp_path):
    """save() after two steps, restore() into a new object, two more steps: the same bits as four
    steps straight through; a checkpoint of another grid is refused."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_checkpoint_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, resumed_at, steps_done, same, refused in got:
        assert resumed_at == 2 and steps_done == 4 and same and refused, (rank, resumed_at, steps_done, same, refused)


def _overlap_worker(rank, world, port, nz, steps, chunk, weights, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        nx, ny = 16, 12
        field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
        st = sharded.ShardedStencil(nx, ny, nz, COEFF, device="cpu", step_fn=oracle_step, weights=weights)
        h_in = torch.from_numpy(field[st.z_lo:st.z_hi].copy())
        plain = torch.full_like(h_in, float("nan"))
        st.run_host(plain, h_in, steps, overlap=False)
        over = torch.full_like(h_in, float("nan"))
        st.run_host(over, h_in, steps, overlap=True, chunk_planes=chunk)
        same = bool(np.array_equal(plain.numpy().view(np.uint32), over.numpy().view(np.uint32)))
        # the object holds the final field afterwards: one more step from it equals steps + 1 plain steps
        more = st.run(1).numpy().copy()
        ref = sharded.ShardedStencil(nx, ny, nz, COEFF, device="cpu", step_fn=oracle_step, weights=weights)
        ref.load(h_in)
        want = ref.run(steps + 1).numpy()
        q.put((rank, same, bool(np.array_equal(more.view(np.uint32), want.view(np.uint32))), st.steps_done))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,nz,steps,chunk,weights", [(2, 40, 3, 4, None), (2, 33, 2, 1, None), (3, 61, 4, 5, None),
                                                          (3, 48, 5, 100, None), (4, 70, 3, 3, (1.0, 1.6, 0.8, 1.2)),
                                                          (2, 16, 1, 2, None)])
def test_overlapped_host_run_on_several_ranks_is_the_plain_run(world, nz, steps, chunk, weights):
    """Upload, steps and download overlapped on N ranks (even ranks walk up, odd ranks down, boundary
    planes exchanged per step where two walks begin or end): the same bits as upload / run / download,
    for pieces from one plane to more than a slab, equal and unequal slabs."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_overlap_worker, args=(r, world, port, nz, steps, chunk, weights, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, same, continues, steps_done in got:
        assert same, "rank %d: overlapped run differs from the plain run" % rank
        assert continues and steps_done == steps + 1, "rank %d: state after the overlapped run" % rank
