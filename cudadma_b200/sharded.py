"""z-sharded 25-point stencil: one process per GPU, radius-wide halo planes
exchanged between z-neighbours every step and overlapped with the interior.

The reference has no multi-GPU code (every program of it uses device 0,
src/examples/stencil/cudaDMA_stencil2D.cu:62); this is the driver the sharded
benchmark configuration needs. Layout per rank: planes [z_lo, z_hi) of the
global nx x ny x nz grid plus four ghost planes on either side, z slowest, so
the four boundary planes of a side are one contiguous block. Ghost planes
beyond the ends of the global grid stay zero, which is the stencil's
out-of-grid rule.

One step, exchange = "nccl":
  1. the first and last four owned planes are computed first;
  2. they are sent to the z-neighbours' ghost planes (torch.distributed
     send/recv: NCCL over NVLink on GPUs) on a side stream;
  3. the remaining interior planes are computed meanwhile on the main stream;
  4. the main stream joins the exchange, buffers swap.
One step, exchange = "p2p" (CUDA devices only): the kernel's CTAs at a shared
boundary wait (bounded) for the neighbour's step count, all owned planes are
computed, the first and last four stored a second time, into the neighbours'
ghost planes over NVLink (the arrays are shared between the processes with
CUDA IPC), and this rank's step count is published by a one-thread launch
behind the kernel (or, p2p_signal="fused", by the kernel's last boundary CTA
while the interior is still running); see cudadma_slab_step in
include/cudadma_b200.h. No collective library on the step.
Every plane is computed by the same kernel with the same arithmetic whatever
the sharding, so an N-rank run reproduces the 1-rank field bit for bit.

Around the step: slabs cut in proportion to the ranks' speeds (weights), a
host-side deadline on the exchange (exchange_timeout), checkpoint / restart of a
rank's slab (save / restore), and run_host, the whole job from and to host
memory with upload, steps and download overlapped.
"""
import datetime

import torch
import torch.distributed as dist

from . import capi

R = 4


class ExchangeError(RuntimeError):
    """A halo exchange did not complete: a z-neighbour is gone or too late."""


def slab_bounds(nz, world, rank, weights=None, min_planes=1):
    """Planes [lo, hi) of rank `rank`. Without weights: as even as possible, earlier ranks take the
    remainder. With weights (one positive number per rank, e.g. each GPU's measured stencil rate):
    slab sizes in proportion to them, every slab at least min_planes deep. All ranks must pass
    the same weights; the cut is a pure function of its arguments."""
    if weights is None:
        base, rem = divmod(nz, world)
        lo = rank * base + min(rank, rem)
        return lo, lo + base + (1 if rank < rem else 0)
    w = [float(x) for x in weights]
    if len(w) != world or min(w) <= 0.0:
        raise ValueError("weights: one positive number per rank")
    if nz < world * min_planes:
        raise ValueError("nz=%d is too shallow for %d slabs of at least %d planes" % (nz, world, min_planes))
    total, acc, cuts = sum(w), 0.0, [0]
    for r in range(world):
        acc += w[r]
        cut = nz if r == world - 1 else int(round(nz * acc / total))
        # keep min_planes for this slab and for each of the slabs still to come
        cut = max(cut, cuts[-1] + min_planes)
        cut = min(cut, nz - (world - 1 - r) * min_planes)
        cuts.append(cut)
    return cuts[rank], cuts[rank + 1]


def bind_host_thread_near_gpu(device_index):
    """Restricts the calling process to the CPU cores next to GPU `device_index` (the set NVML
    reports for it), so that host buffers allocated and touched afterwards land in that GPU's
    NUMA node and its PCIe copies do not cross the socket interconnect. Only this process's own
    scheduling mask changes; nothing of the GPU is set. Returns the core list, or None where NVML
    or the affinity call is not available (the process then stays as it was)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = None
        try:  # by PCI address: the CUDA index need not be NVML's when CUDA_VISIBLE_DEVICES is set
            p = torch.cuda.get_device_properties(int(device_index))
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(
                ("%08x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)).encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(int(device_index))
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cores = [64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1]
        allowed = sorted(set(cores) & set(os.sched_getaffinity(0)))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:
        return None


def _cuda_step(out, inp, nx, ny, nz_total, z_begin, z_end, coeff):
    capi.stencil25_step(out, inp, nx, ny, nz_total, z_begin, z_end, coeff)


class ShardedStencil:
    """step_fn(out, inp, nx, ny, nz_total, z_begin, z_end, coeff) computes output planes
    [z_begin, z_end) of a local array of nz_total planes; the default is the CUDA kernel
    through the C ABI (there is no CPU path in the product; tests of the host logic on
    CPU ranks pass their own step function)."""

    def __init__(self, nx, ny, nz, coeff=None, device=None, group=None, step_fn=None, pad_xy=0, exchange="nccl",
                 weights=None, exchange_timeout=None, p2p_signal=None):
        """pad_xy: zero cells kept around every plane in x and y (0 for the tensor-map kernel, which
        needs no border; 4 for kernels that read a padded array). The step function sees the padded
        planes: nx + 2 * pad_xy by ny + 2 * pad_xy.
        weights: relative speed of every rank (same list on all ranks); slabs are cut in proportion,
        so that ranks which step in lockstep finish a step together even when their GPUs do not run
        equally fast (power-capped parts differ by several per cent). None = equal slabs.
        p2p_signal: who publishes a rank's step count in the "p2p" exchange: "trailing" (a one-thread
        launch behind the step's kernel, runs of planes dispatched from the top down),
        "trailing-ascending" (the same, from the bottom up) or "fused" (the step is one launch; its
        last boundary CTA publishes); None = the library's default. The same on every rank.
        exchange_timeout: seconds a rank waits on the host for its neighbours' planes before step()
        raises ExchangeError (ranks on CPU). On CUDA devices nothing waits on the host during a
        step: a lost neighbour ends the "nccl" exchange through the process group's own timeout,
        and the "p2p" exchange through the bounded wait inside cudadma_slab_step's kernel (about two
        seconds): that rank then stops pushing planes and publishing its step count, so its
        neighbours' waits run out in turn, and check_status() -- which run() and run_host() call --
        raises ExchangeError on every rank."""
        self.nx, self.ny, self.nz = nx, ny, nz
        self.pad = pad_xy
        self.coeff = tuple(capi.STENCIL_COEFFS if coeff is None else coeff)
        self.group = group
        self.exchange_timeout = exchange_timeout
        self.distributed = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.z_lo, self.z_hi = slab_bounds(nz, self.world, self.rank, weights, 2 * R if self.world > 1 else 1)
        self.nzl = self.z_hi - self.z_lo
        if self.world > 1 and self.nzl < R:
            raise ValueError("every rank needs at least %d planes (nz=%d over %d ranks)" % (R, nz, self.world))
        if step_fn is None:
            if not torch.cuda.is_available():
                raise RuntimeError("the sharded stencil runs on CUDA devices only; no CPU fallback exists")
            step_fn = _cuda_step
            device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.step_fn = step_fn
        self.device = torch.device("cpu") if device is None else torch.device(device)
        self.on_cuda = self.device.type == "cuda"
        self.px, self.py = nx + 2 * pad_xy, ny + 2 * pad_xy
        plane = self.px * self.py
        self.plane = plane
        if exchange not in ("nccl", "p2p"):
            raise ValueError("exchange is 'nccl' or 'p2p'")
        self.slab = None
        if exchange == "p2p" and self.world > 1:
            if not self.on_cuda or step_fn is not _cuda_step or pad_xy != 0:
                raise ValueError("the peer-to-peer exchange belongs to the CUDA kernel of this library")
            self.slab = capi.Slab(nx, ny, self.nzl, self.rank > 0, self.rank < self.world - 1)
            if p2p_signal is not None:
                self.slab.set_signal_mode(p2p_signal)
            blobs = [None] * self.world
            dist.all_gather_object(blobs, self.slab.export(), group=group)
            self.slab.connect(blobs[self.rank - 1] if self.rank > 0 else None,
                              blobs[self.rank + 1] if self.rank < self.world - 1 else None)
            self.cur, self.nxt = self.slab.tensor(0), self.slab.tensor(1)
        else:
            self.cur = torch.zeros((self.nzl + 2 * R) * plane, dtype=torch.float32, device=self.device)
            self.nxt = torch.zeros_like(self.cur)
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.on_cuda and self.world > 1 else None
        self.steps_done = 0
        self._copy_streams = None

    # -- data in and out ---------------------------------------------------
    def owned(self, buf=None):
        """View [nzl, ny, nx] of the owned cells (no ghost planes, no border) of the current field."""
        buf = self.cur if buf is None else buf
        v = buf.view(self.nzl + 2 * R, self.py, self.px)
        return v[R:R + self.nzl, self.pad:self.pad + self.ny, self.pad:self.pad + self.nx]

    def load(self, slab):
        """slab: this rank's planes [z_lo, z_hi) as a flat or [nzl, ny, nx] float32 tensor (any device)."""
        self.cur.zero_()
        self.nxt.zero_()
        self.owned().copy_(slab.reshape(self.nzl, self.ny, self.nx), non_blocking=True)
        self.steps_done = 0
        if self.world > 1:
            self._exchange(self.cur, wait=True)

    def store(self, out):
        out.reshape(self.nzl, self.ny, self.nx).copy_(self.owned(), non_blocking=True)

    # -- halo exchange -----------------------------------------------------
    def _planes(self, buf, first, count):
        return buf[first * self.plane:(first + count) * self.plane]

    def _exchange_ops(self, buf):
        ops = []
        up, down = self.rank + 1, self.rank - 1
        if down >= 0:
            ops.append(dist.P2POp(dist.isend, self._planes(buf, R, R), down, self.group))
            ops.append(dist.P2POp(dist.irecv, self._planes(buf, 0, R), down, self.group))
        if up < self.world:
            ops.append(dist.P2POp(dist.isend, self._planes(buf, self.nzl, R), up, self.group))
            ops.append(dist.P2POp(dist.irecv, self._planes(buf, R + self.nzl, R), up, self.group))
        return ops

    def _wait(self, works):
        if self.on_cuda or self.exchange_timeout is None:
            for w in works:
                w.wait()  # on CUDA: the current stream waits for the exchange, the host does not block
            return
        limit = datetime.timedelta(seconds=float(self.exchange_timeout))
        for w in works:
            try:
                done = w.wait(limit)
            except RuntimeError as e:
                raise ExchangeError("rank %d, step %d: %s" % (self.rank, self.steps_done + 1, e)) from e
            if done is False:
                raise ExchangeError("rank %d, step %d: no planes from a neighbour within %.1f s"
                                    % (self.rank, self.steps_done + 1, float(self.exchange_timeout)))

    def _exchange(self, buf, wait):
        ops = self._exchange_ops(buf)
        works = dist.batch_isend_irecv(ops) if ops else []
        if wait:
            self._wait(works)
        return works

    # -- time stepping -----------------------------------------------------
    def step(self):
        nx, ny, nzt = self.nx, self.ny, self.nzl + 2 * R
        cur, nxt = self.cur, self.nxt
        first, last = R, R + self.nzl  # owned planes are [first, last) of the local array
        if self.world == 1:
            self.step_fn(nxt, cur, nx, ny, nzt, first, last, self.coeff)
        elif self.slab is not None:
            self.slab.step(self.coeff)
        else:
            lo_end = min(first + R, last)
            hi_begin = max(last - R, lo_end)
            self.step_fn(nxt, cur, nx, ny, nzt, first, lo_end, self.coeff)
            if hi_begin < last:
                self.step_fn(nxt, cur, nx, ny, nzt, hi_begin, last, self.coeff)
            if self.on_cuda:
                main = torch.cuda.current_stream(self.device)
                self.comm_stream.wait_stream(main)
                with torch.cuda.stream(self.comm_stream):
                    works = self._exchange(nxt, wait=False)
            else:
                works = self._exchange(nxt, wait=False)
            if lo_end < hi_begin:
                self.step_fn(nxt, cur, nx, ny, nzt, lo_end, hi_begin, self.coeff)
            self._wait(works)
            if self.on_cuda:
                torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        self.cur, self.nxt = nxt, cur
        self.steps_done += 1

    def run(self, steps):
        for _ in range(steps):
            self.step()
        if self.slab is not None:
            self.check_status()
        return self.owned()

    def check_status(self):
        """Waits for the steps issued so far and raises ExchangeError, on every rank alike, if a
        bounded wait inside any rank's kernels gave up (a neighbour gone or too far behind): the
        fields are not to be trusted then. step() itself never waits on the host, so a time loop
        calls this where it would look at its results anyway."""
        if not self.on_cuda:
            return
        with torch.cuda.device(self.device):
            bad = 0
            if self.slab is not None and self.slab.status() != capi.OK:
                bad = 1
            if capi.device_status() != 0:
                bad = 1
        if self.distributed and self.world > 1:
            t = torch.tensor([bad], dtype=torch.int32, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            bad = int(t.item())
        if bad:
            raise ExchangeError("rank %d: a wait for a neighbour's planes gave up on some rank by step %d"
                                % (self.rank, self.steps_done))

    # -- checkpoint / restart ----------------------------------------------
    _MAGIC = b"CDB200S1"

    def save(self, path):
        """Writes this rank's owned planes and the step count to `path` (one file per rank; raw
        little-endian: magic, nx, ny, nz, z_lo, z_hi, steps_done as int64, then the float32 planes).
        Ghost planes are not stored: restore() exchanges them again."""
        import numpy as np
        if self.on_cuda:
            torch.cuda.current_stream(self.device).synchronize()
        planes = self.owned().contiguous().cpu().numpy()
        head = np.array([self.nx, self.ny, self.nz, self.z_lo, self.z_hi, self.steps_done], dtype="<i8")
        with open(path, "wb") as f:
            f.write(self._MAGIC)
            f.write(head.tobytes())
            f.write(planes.astype("<f4", copy=False).tobytes())

    def restore(self, path):
        """Reads a file written by save() for the same grid and the same slab, refills the ghost
        planes from the neighbours (every rank must call it) and continues from the stored step."""
        import numpy as np
        with open(path, "rb") as f:
            if f.read(len(self._MAGIC)) != self._MAGIC:
                raise ValueError("%s is not a slab checkpoint" % path)
            head = np.frombuffer(f.read(6 * 8), dtype="<i8")
            if tuple(head[:5]) != (self.nx, self.ny, self.nz, self.z_lo, self.z_hi):
                raise ValueError("%s holds planes [%d, %d) of a %d x %d x %d grid, not this rank's slab"
                                 % (path, head[3], head[4], head[0], head[1], head[2]))
            planes = np.frombuffer(f.read(), dtype="<f4")
        if planes.size != self.nzl * self.ny * self.nx:
            raise ValueError("%s is truncated" % path)
        self.load(torch.from_numpy(planes.copy()))
        self.steps_done = int(head[5])

    def run_host(self, h_out, h_in, steps, overlap=None, chunk_planes=None):
        """The whole job from and to host memory (pinned tensors copy fastest): upload the slab,
        `steps` steps, download the slab. Returns when h_out holds the result.
        overlap: on several ranks, overlap the three phases (see _run_host_overlapped); None = where
        the slab is deep enough for it to pay (and the step function is this library's kernel).
        chunk_planes: planes per upload piece of the overlapped form (None = 128 MiB pieces).

        On a single GPU with this library's kernel the call is cudadma_stencil25_run_host, which
        overlaps the upload, the steps and the download in pieces (same bits); the field held by
        this object is then left as it was."""
        if self.world == 1 and self.on_cuda and self.step_fn is _cuda_step and self.pad == 0:
            with torch.cuda.device(self.device):
                capi.stencil25_run_host(h_out, h_in, self.nx, self.ny, self.nz, steps, self.coeff)
            return
        if self.world > 1 and overlap is None:
            overlap = self.step_fn is _cuda_step and self.nzl >= 4 * steps + 2 * self._chunk_planes(None)
        if self.world > 1 and overlap and steps > 0:
            self._run_host_overlapped(h_out, h_in, steps, self._chunk_planes(chunk_planes))
        else:
            self.load(h_in)
            self.run(steps)
            self.store(h_out)
        if self.on_cuda:
            torch.cuda.current_stream(self.device).synchronize()
            self.check_status()

    def _chunk_planes(self, chunk_planes):
        if chunk_planes:
            return int(chunk_planes)
        return max(8, min((128 << 20) // (self.plane * 4), self.nzl // 8))

    def _run_host_overlapped(self, h_out, h_in, steps, chunk):
        """Upload, steps and download of a slab overlapped, on several ranks.

        A rank walks its slab in one direction, even ranks upwards and odd ranks downwards, so that
        the two ranks at an interface either both begin there or both end there. Planes are uploaded
        in that order; after `done[0]` of them have arrived, step t can produce the first
        done[0] - 4t planes of the walk, and once the whole slab is up every step runs on to the far
        end. Planes of a z-neighbour are needed in two places only: at an interface where both walks
        begin, the first four planes of step t-1 are exchanged before either side starts step t
        (early in the run, one small exchange per step); at an interface where both walks end, the
        last four planes of step t-1 are exchanged once both sides have finished that step (at the
        very end). Two ping-pong arrays suffice for the same reason as on one GPU (step t only
        overwrites planes that step t-1 has finished reading). Every plane is computed by the same
        kernel on the same operands as in run(), so the result is the same, bit for bit."""
        nzl, nx, ny, nzt = self.nzl, self.nx, self.ny, self.nzl + 2 * R
        up = self.rank % 2 == 0                        # direction of the walk
        lower, upper = self.rank > 0, self.rank < self.world - 1
        start_peer = (self.rank - 1 if lower else None) if up else (self.rank + 1 if upper else None)
        end_peer = (self.rank + 1 if upper else None) if up else (self.rank - 1 if lower else None)
        self.cur.zero_()
        self.nxt.zero_()
        buf = [self.cur, self.nxt]
        h_in = h_in.reshape(nzl, ny, nx)
        h_out = h_out.reshape(nzl, ny, nx)

        def owned_range(s0, s1):
            """walk positions [s0, s1) as a range of owned planes [a, b)"""
            return (s0, s1) if up else (nzl - s1, nzl - s0)

        def planes(b, a0, a1):
            """owned planes [a0, a1) of array b, with the x/y border the step function may want"""
            return buf[b].view(nzt, self.py, self.px)[R + a0:R + a1]

        def inner(t):
            return t[:, self.pad:self.pad + ny, self.pad:self.pad + nx]

        def exchange(peer, b, at_start):
            """Swap four boundary planes of array b with `peer`: mine go into its ghost planes, its
            into mine. at_start: the interface is where this rank's walk begins."""
            low_side = (at_start and up) or (not at_start and not up)   # the interface is below this slab
            mine = self._planes(buf[b], R, R) if low_side else self._planes(buf[b], nzl, R)
            ghost = self._planes(buf[b], 0, R) if low_side else self._planes(buf[b], R + nzl, R)
            ops = [dist.P2POp(dist.isend, mine, peer, self.group), dist.P2POp(dist.irecv, ghost, peer, self.group)]
            self._wait(dist.batch_isend_irecv(ops))

        if self.on_cuda:
            main = torch.cuda.current_stream(self.device)
            if self._copy_streams is None:
                self._copy_streams = (torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device))
            s_up, s_down = self._copy_streams
            s_up.wait_stream(main)
            s_down.wait_stream(main)
        done = [0] * (steps + 1)   # done[t]: the first done[t] planes of the walk hold the field after t steps
        started = 0                # exchanges made at the interface where the walk begins (steps 0 .. started-1)
        ended = 0                  # the same for the interface where it ends
        down = 0                   # planes of the walk already on their way to the host
        while done[steps] < nzl:
            if done[0] < nzl:
                s0, s1 = done[0], min(nzl, done[0] + chunk)
                a0, a1 = owned_range(s0, s1)
                if self.on_cuda:
                    with torch.cuda.stream(s_up):
                        inner(planes(0, a0, a1)).copy_(h_in[a0:a1], non_blocking=True)
                    main.wait_stream(s_up)
                else:
                    inner(planes(0, a0, a1)).copy_(h_in[a0:a1])
                done[0] = s1
            for t in range(1, steps + 1):
                src, dst = (t - 1) % 2, t % 2
                if done[t] == 0 and start_peer is not None and started < t:
                    if done[t - 1] < R:
                        break
                    exchange(start_peer, src, True)
                    started = t
                if done[t - 1] == nzl:
                    if end_peer is not None and ended < t:
                        exchange(end_peer, src, False)
                        ended = t
                    reach = nzl
                else:
                    reach = done[t - 1] - R
                if reach <= done[t]:
                    break
                a0, a1 = owned_range(done[t], reach)
                self.step_fn(buf[dst], buf[src], nx, ny, nzt, R + a0, R + a1, self.coeff)
                done[t] = reach
            if done[steps] > down:
                a0, a1 = owned_range(down, done[steps])
                if self.on_cuda:
                    s_down.wait_stream(main)
                    with torch.cuda.stream(s_down):
                        h_out[a0:a1].copy_(inner(planes(steps % 2, a0, a1)), non_blocking=True)
                else:
                    h_out[a0:a1].copy_(inner(planes(steps % 2, a0, a1)))
                down = done[steps]
        if self.on_cuda:
            main.wait_stream(s_down)
        # leave the object holding the final field, as run() would
        if steps % 2:
            if self.slab is not None:
                self.cur.copy_(self.nxt)   # the library's arrays keep their roles
            else:
                self.cur, self.nxt = self.nxt, self.cur
        self._exchange(self.cur, wait=True)   # ghost planes of the final field, so that step() can go on from here
        self.steps_done = steps
