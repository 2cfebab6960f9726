"""The z-sharded stencil on real GPUs: N ranks (NCCL halo exchange) reproduce the one-GPU field
bit for bit. Needs at least two CUDA devices; skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, nx, ny, nz, steps, exchange, q, weights=None, p2p_signal=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cudadma_b200.sharded import ShardedStencil
        from oracle import oracle
        field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
        if exchange.startswith("p2p-"):    # "p2p-fused", "p2p-trailing-ascending"
            exchange, p2p_signal = "p2p", exchange[4:]
        st = ShardedStencil(nx, ny, nz, exchange=exchange, weights=weights, p2p_signal=p2p_signal)
        st.load(torch.from_numpy(field[st.z_lo:st.z_hi].copy()).cuda())
        got = st.run(steps).cpu().numpy().copy()
        torch.cuda.synchronize()
        import cudadma_b200 as cd
        assert cd.device_status() == 0, "a bounded wait gave up on rank %d" % rank
        dist.barrier()  # nobody unmaps a neighbour's memory while the other side still steps
        q.put((rank, st.z_lo, st.z_hi, got))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("nz,steps,exchange,weights",
                         [(40, 3, "nccl", None), (19, 2, "nccl", None), (40, 5, "p2p", None), (17, 2, "p2p", None),
                          (48, 4, "p2p", (1.0, 1.7)), (48, 3, "nccl", (2.1, 1.0)), (230, 4, "p2p", None),
                          (40, 5, "p2p-fused", None), (230, 4, "p2p-fused", None), (48, 4, "p2p-fused", (1.0, 1.7)),
                          (230, 4, "p2p-trailing-ascending", None), (600, 3, "p2p", None)])
def test_two_gpus_equal_one_gpu(nz, steps, exchange, weights):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import cudadma_b200 as cd
    from oracle import oracle
    nx, ny, world = 128, 64, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, nx, ny, nz, steps, exchange, q, weights)) for r in range(world)]
    for p in procs:
        p.start()
    parts = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)
    a = torch.from_numpy(field).cuda()
    b = torch.zeros_like(a)
    one = cd.stencil25_run(a, b, nx, ny, nz, steps).cpu().numpy().reshape(nz, ny, nx)
    for rank, lo, hi, got in parts:
        assert np.array_equal(got.view(np.uint32), one[lo:hi].view(np.uint32)), "rank %d differs" % rank
    exp = oracle.stencil25_f64(field.reshape(nz, ny, nx), cd.STENCIL_COEFFS, steps)
    assert np.abs(one - exp).max() / np.abs(exp).max() <= 1e-5


def _host_worker(rank, world, port, nx, ny, nz, steps, exchange, chunk, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cudadma_b200.sharded import ShardedStencil
        from oracle import oracle
        import cudadma_b200 as cd
        field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0).reshape(nz, ny, nx)
        st = ShardedStencil(nx, ny, nz, exchange=exchange)
        h_in = torch.from_numpy(field[st.z_lo:st.z_hi].copy()).pin_memory()
        plain = torch.full_like(h_in, float("nan")).pin_memory()
        over = torch.full_like(h_in, float("nan")).pin_memory()
        st.run_host(plain, h_in, steps, overlap=False)
        st.run_host(over, h_in, steps, overlap=True, chunk_planes=chunk)
        more = st.run(1).cpu().numpy().copy()   # the object goes on from the final field
        torch.cuda.synchronize()
        assert cd.device_status() == 0, "a bounded wait gave up on rank %d" % rank
        dist.barrier()
        q.put((rank, st.z_lo, st.z_hi, plain.numpy().copy(), over.numpy().copy(), more))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("nz,steps,exchange,chunk", [(96, 4, "nccl", 8), (64, 3, "p2p", 5), (40, 2, "p2p", 64)])
def test_two_gpus_overlapped_host_run_is_the_plain_run(nz, steps, exchange, chunk):
    """run_host with upload, steps and download overlapped on two GPUs: the same bits as the plain
    sequence and as one GPU, and the object continues correctly from the final field."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import cudadma_b200 as cd
    from oracle import oracle
    nx, ny, world = 128, 64, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_host_worker, args=(r, world, port, nx, ny, nz, steps, exchange, chunk, q)) for r in range(world)]
    for p in procs:
        p.start()
    parts = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)
    a = torch.from_numpy(field).cuda()
    b = torch.zeros_like(a)
    one = cd.stencil25_run(a, b, nx, ny, nz, steps).cpu().numpy().reshape(nz, ny, nx).copy()
    a = torch.from_numpy(field).cuda()
    b = torch.zeros_like(a)
    one_more = cd.stencil25_run(a, b, nx, ny, nz, steps + 1).cpu().numpy().reshape(nz, ny, nx)
    for rank, lo, hi, plain, over, more in parts:
        assert np.array_equal(plain.view(np.uint32), one[lo:hi].view(np.uint32)), "rank %d: plain host run" % rank
        assert np.array_equal(over.view(np.uint32), one[lo:hi].view(np.uint32)), "rank %d: overlapped host run" % rank
        assert np.array_equal(more.view(np.uint32), one_more[lo:hi].view(np.uint32)), "rank %d: next step" % rank


@pytest.mark.parametrize("nz,steps", [(40, 4), (230, 3)])
def test_two_gpus_driven_from_one_process(nz, steps):
    """cudadma_stencil25_multi_*: one process, one slab and one stream per GPU, neighbours joined by
    peer access. The library keeps what it knows per device, so the second GPU of the process works
    like the first; the field equals the one-GPU field bit for bit."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import cudadma_b200 as cd
    from oracle import oracle
    nx, ny = 128, 64
    field = oracle.fill_uniform(nx * ny * nz, 0xC4, 0.0, 1.0)
    m = cd.MultiStencil(2, nx, ny, nz)
    try:
        m.load(field)
        m.run(steps)
        got = np.full_like(field, np.nan)
        m.store(got)
    finally:
        m.destroy()
    a = torch.from_numpy(field).cuda()
    one = cd.stencil25_run(a, torch.zeros_like(a), nx, ny, nz, steps).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), one.view(np.uint32))
    # every other entry point on the second device of the same process
    with torch.cuda.device(1):
        a1 = torch.from_numpy(field).cuda()
        one1 = cd.stencil25_run(a1, torch.zeros_like(a1), nx, ny, nz, steps).cpu().numpy()
        src = torch.from_numpy(oracle.fill_uniform(16384 * 5 // 4, 0xC1, -1.0, 1.0)).cuda()
        dst = torch.zeros_like(src)
        cd.seq_copy(dst, src)
        g = torch.from_numpy(oracle.fill_index(1280, 0xC3A, 4096)).cuda()
        p = torch.from_numpy(oracle.permutation(1280, 0xC3B)).cuda()
        table = torch.from_numpy(oracle.fill_uniform(4096 * 8, 0xC3, -1.0, 1.0)).cuda()
        out = torch.zeros(1280 * 8, device="cuda")
        cd.gather_scatter(out, table, g, p, 1280)
        torch.cuda.synchronize()
        assert cd.device_status() == 0
        assert torch.equal(dst, src)
        assert torch.equal(out.view(1280, 8)[p.long()], table.view(4096, 8)[g.long()])
    assert np.array_equal(one1.view(np.uint32), one.view(np.uint32))
