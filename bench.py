"""Benchmark of the hot path: the radius-4 25-point stencil fed by CudaDMA objects,
on the sharded configuration of the benchmark list (1024 x 1024 x 2048 fp32 grid,
z-split over the ranks, four-plane halos exchanged every step), plus, at one GPU,
the three data-movement patterns and the 512^3 stencil.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1). A
step is one time step over the whole grid. Rank 0 prints one JSON line.

--impl ours       this repository's kernels.
--impl reference  the same workloads through the REFERENCE CudaDMA classes compiled for
                  sm_100a (oracle/_ref, built from the reference checkout) where that
                  library is present, else the CPU restatement on the host cores.
Both lines carry `cpu_baseline`: the host loops of oracle/ on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

NX, NY, NZ = 1024, 1024, 2048          # the sharded stencil configuration
C4 = (512, 512, 512)                   # the single-GPU stencil configuration
BYTES_PER_POINT = 8                    # one fp32 read + one fp32 write per point and step
# DRAM bytes per point of stencil25::tensor_kernel: dram__bytes_read + dram__bytes_write of an ncu capture
# of the 512^3 case (1042.4 MB per launch; summary under profiles/), which grows in proportion to the points
STENCIL_DRAM_BYTES_PER_POINT = 1042.4e6 / 512 ** 3
L2_FLUSH_BYTES = 256 << 20
EXCHANGE = "p2p"                       # halo exchange of this repository's arm at N > 1 (--exchange)
P2P_SIGNAL = None                      # who publishes a rank's step count in that exchange (--p2p-signal; None: library default)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for l in self.lines:
            parts = [x.strip() for x in l.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


HOST_CORES = None  # the cores this rank was bound to (N > 1 only)


def setup_dist(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    global HOST_CORES
    if world > 1:
        # N ranks copy to and from N GPUs at once: keep each rank's threads and pinned buffers in its GPU's NUMA node
        from cudadma_b200.sharded import bind_host_thread_near_gpu
        HOST_CORES = bind_host_thread_near_gpu(local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner on stdout at the VERSION level; stdout carries the JSON line only
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != n_gpus and rank == 0:
        print("warning: --gpus %d but WORLD_SIZE=%d; using WORLD_SIZE" % (n_gpus, world), file=sys.stderr)
    return rank, world, local


def barrier():
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(x):
    if not dist.is_initialized():
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_ranks(x):
    """The value of every rank, in rank order, on every rank."""
    if not dist.is_initialized():
        return [x]
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    g = [torch.zeros_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(g, t)
    return [float(v.item()) for v in g]


def time_region(fn, reps):
    """Device time of `reps` calls of fn, in ms, bracketed by barrier + synchronize; max over ranks."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return max_over_ranks(e0.elapsed_time(e1))


def median_launch_ms(fn, reps, flush=None):
    """Median device time of single calls, each timed by its own event pair (L2 flushed before each if asked)."""
    ts = []
    for _ in range(reps):
        if flush is not None:
            flush.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def seeded_field(n, seed, lo=0.0, hi=1.0, first_index=0):
    """Element i = lo + (hi - lo) * u(seed + first_index + i), the stateless splitmix64 rule that
    oracle/oracle.c states for the benchmark inputs, made on the device (cudadma_fill_uniform)."""
    import cudadma_b200 as cd
    return cd.fill_uniform(torch.empty(n, device="cuda", dtype=torch.float32), seed, lo, hi, first_index)


class SmClockProbe:
    """The SM clock a workload really runs at: one-thread kernels on a second, high-priority
    stream spin for a millisecond each beside it and report cycles / nanoseconds."""

    def __init__(self, slots=64):
        self.buf = torch.zeros(2 * slots, dtype=torch.int64, device="cuda")
        self.stream = torch.cuda.Stream(priority=-1)
        self.used, self.slots = 0, slots

    def fire(self, spin_ns=1000000):
        import cudadma_b200 as cd
        if self.used < self.slots:
            cd.clock_probe(self.buf[2 * self.used:], spin_ns, self.stream)
            self.used += 1

    def mhz(self):
        torch.cuda.synchronize()
        h = self.buf.cpu().view(-1, 2)[:self.used]
        v = sorted(float(c) / float(ns) * 1e3 for c, ns in h.tolist() if ns > 0)
        return v


# ------------------------------------------------------------------ CPU baseline
def cpu_baseline_stencil():
    """The oracle's fp32 stencil step (oracle/oracle.c, all host threads) on a 1024 x 1024 x 64 slab."""
    import numpy as np
    from oracle import oracle
    nz = 64
    field = oracle.fill_uniform(NX * NY * nz, 0xC4, 0.0, 1.0).reshape(nz, NY, NX)
    out = np.empty_like(field)
    coeff = (-2.847, 1.6, -0.2, 0.0254, -0.00179)
    oracle.stencil25_step_f32(field, coeff, out)  # warm-up
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or time.perf_counter() - t0 < 5.0:
        oracle.stencil25_step_f32(field, coeff, out)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": NX * NY * nz * reps / dt / 1e9, "unit": "Gpts/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": "%d steps of the fp32 host loop on a %dx%dx%d slab of the grid" % (reps, NX, NY, nz)}


def cpu_baseline_patterns():
    import numpy as np
    from oracle import oracle
    out = {}

    def rate(fn, nbytes):
        fn()
        reps, t0 = 0, time.perf_counter()
        while reps < 2 or time.perf_counter() - t0 < 2.0:
            fn()
            reps += 1
        return nbytes * reps / (time.perf_counter() - t0) / 1e9

    src = oracle.fill_uniform(1 << 24, 0xC1, -1.0, 1.0)
    out["sequential_gbs"] = rate(lambda: oracle.chunked_copy(src), 2 * src.nbytes)
    m = oracle.fill_uniform(4096 * 4096, 0xC2, -1.0, 1.0).reshape(4096, 4096)
    t = np.empty((4096, 4096), dtype=np.float32)
    out["strided_gbs"] = rate(lambda: oracle.tile_transpose(m, out=t), 2 * m.nbytes)
    out["strided_sample"] = "4096x4096 of the 16384x16384 matrix"
    n, rec = 1 << 22, 1 << 24
    table = oracle.fill_uniform(rec * 8, 0xC3, -1.0, 1.0)
    g, s = oracle.fill_index(n, 0xC3A, rec), oracle.permutation(n, 0xC3B)
    o = np.zeros(n * 8, dtype=np.float32)
    out["indirect_gbs"] = rate(lambda: oracle.gather_scatter(o, table, g, s), n * 72)
    out["cores"] = oracle.num_threads()
    return out


# ------------------------------------------------------------------ single-GPU patterns
_EXPECTED = {}   # what the CPU oracle makes of the seeded inputs, computed once per process


def expected(name):
    """Inputs and expected outputs of the data-movement configurations from oracle/ (host side, the
    checker): the same seeds as the device-side generator, so the kernels' results can be compared
    bit for bit with what the reference's host check loops give."""
    import numpy as np
    from oracle import oracle
    if name not in _EXPECTED:
        if name == "sequential":
            src = oracle.fill_uniform(1 << 24, 0xC1, -1.0, 1.0)
            _EXPECTED[name] = oracle.chunked_copy(src)
        elif name == "strided":
            m = 16384
            src = oracle.fill_uniform(m * m, 0xC2, -1.0, 1.0).reshape(m, m)
            _EXPECTED[name] = oracle.tile_transpose(src)
        elif name == "indirect":
            n, rec = 1 << 22, 1 << 24
            table = oracle.fill_uniform(rec * 8, 0xC3, -1.0, 1.0)
            g, perm = oracle.fill_index(n, 0xC3A, rec), oracle.permutation(n, 0xC3B)
            _EXPECTED[name] = (oracle.gather_scatter(np.zeros(n * 8, dtype=np.float32), table, g, perm), perm)
    return _EXPECTED[name]


def same_bits(dev_tensor, host_array):
    import numpy as np
    got = dev_tensor.cpu().numpy().reshape(-1).view(np.uint32)
    return bool(np.array_equal(got, np.ascontiguousarray(host_array).reshape(-1).view(np.uint32)))


def pick_bpt(call, flush=None):
    """The reference's classes take BYTES_PER_THREAD, their register staging budget, as a template
    argument; the reference arm tries 64, 128 and 192 and keeps the fastest (median of 7 launches)."""
    from oracle import reference as ref
    times = {}
    for bpt in ref.BPTS:
        f = lambda: call(bpt)
        f()
        times[bpt], _ = median_launch_ms(f, 7, flush)
    best = min(times, key=times.get)
    return {"best": best, "ms": {str(k): round(v, 4) for k, v in times.items()}}


REFERENCE_STENCIL_FORMS = ("windows_bpt64", "windows_bpt128", "windows_bpt192", "halo_ring")


def reference_stencil_step(form):
    """step(out, in, nx, ny, nz, z_begin, z_end, coeff) on padded arrays through the reference's classes:
    whole windows by CudaDMAStrided (three staging budgets) or ring by v1 cudaDMAHalo + interior by cudaDMAStrided."""
    from oracle import reference as ref
    if form == "halo_ring":
        return lambda o, i, nx, ny, nz, zb, ze, c: ref.halo_stencil25_step_padded(o, i, nx, ny, nz, zb, ze, c)
    bpt = int(form.rsplit("bpt", 1)[1])
    return lambda o, i, nx, ny, nz, zb, ze, c: ref.stencil25_step_padded(o, i, nx, ny, nz, zb, ze, c, 0, bpt)


_REFERENCE_STENCIL = {}


def pick_reference_stencil(a, b, nx, ny, nz):
    """Times every form of the reference-class stencil on the given padded arrays and names the fastest."""
    import cudadma_b200 as cd
    from oracle import reference as ref
    times = {}
    for form in REFERENCE_STENCIL_FORMS:
        if form == "halo_ring" and not ref.halo_stencil_available():
            continue
        step = reference_stencil_step(form)

        def f():
            step(b, a, nx, ny, nz, 0, nz, cd.STENCIL_COEFFS)
        f()
        times[form], _ = median_launch_ms(f, 5)
    best = min(times, key=times.get)
    _REFERENCE_STENCIL["best"] = best
    return {"best": best, "ms_per_step": {k: round(v, 4) for k, v in times.items()}}


def run_patterns(kind, peak):
    """Device-timed GB/s of the three data-movement patterns and the 512^3 stencil.
    kind: "native", "portable" (this repository) or "reference" (oracle/_ref).
    Inputs are the seeded fields of the benchmark list; every output of a timed launch is compared
    bit for bit with the CPU oracle's."""
    import cudadma_b200 as cd
    if kind == "reference":
        from oracle import reference as ref
    flush = torch.zeros(L2_FLUSH_BYTES // 4, device="cuda")
    res = {}

    def entry(ms, best, nbytes, launches=1):
        gbs = nbytes / ms / 1e6
        return {"gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4), "ms": round(ms, 4),
                "best_gbs": round(nbytes / best / 1e6, 1), "algorithmic_bytes": nbytes, "launches_per_pass": launches}

    # sequential: 64 MiB, 16 KiB chunks
    n = 1 << 24
    src, dst = seeded_field(n, 0xC1, -1.0, 1.0), torch.zeros(n, device="cuda")
    bpt_seq = None
    if kind == "reference":
        bpt_seq = pick_bpt(lambda bpt: ref.seq_copy(dst, src, n * 4, bpt), flush)
        f = lambda: ref.seq_copy(dst, src, n * 4, bpt_seq["best"])
    else:
        f = lambda: cd.seq_copy(dst, src, n * 4, 16384, kind)
    for _ in range(3):
        f()
    ms, best = median_launch_ms(f, 30, flush)
    res["sequential_64MiB"] = entry(ms, best, 2 * n * 4)
    if bpt_seq:
        res["sequential_64MiB"]["bytes_per_thread"] = bpt_seq
    res["sequential_64MiB"]["parity"] = "pass" if same_bits(dst, expected("sequential")) else "FAIL"
    # what a plain device-to-device copy of the same 64 MiB takes in the same loop (same L2 flush, same event
    # pair): the job lasts under 30 us, most of which is the ramp of an idle GPU, whatever kernel runs
    ceil_dst = torch.empty_like(dst)
    g = lambda: ceil_dst.copy_(src)
    for _ in range(3):
        g()
    msc, bestc = median_launch_ms(g, 30, flush)
    res["sequential_64MiB"]["copy_ceiling_gbs"] = round(2 * n * 4 / msc / 1e6, 1)
    res["sequential_64MiB"]["copy_ceiling_note"] = "torch copy_ (cudaMemcpyAsync device-to-device) of the same array, same loop"
    del ceil_dst
    # The same 64 MiB job back to back over 12 different array pairs (1.5 GiB in all, so nothing is found
    # in L2 either): one event pair around 24 launches, which takes the event pair's own microseconds
    # (a tenth of such a short launch) out of the figure.
    pairs = [(seeded_field(n, 0xC10 + i, -1.0, 1.0), torch.empty(n, device="cuda")) for i in range(12)]
    cur_stream = torch.cuda.current_stream().cuda_stream  # looked up once: the launches must not wait for Python
    if kind == "reference":
        rot = lambda: [ref.seq_copy(d, s_, n * 4, bpt_seq["best"]) for _ in range(2) for s_, d in pairs]
    else:
        rot = lambda: [cd.seq_copy(d, s_, n * 4, 16384, kind, cur_stream) for _ in range(2) for s_, d in pairs]
    rot()
    msr, bestr = median_launch_ms(rot, 10)
    res["sequential_64MiB"]["rotating_gbs"] = round(2 * n * 4 * 2 * len(pairs) / msr / 1e6, 1)
    res["sequential_64MiB"]["rotating_frac_of_peak"] = round(2 * n * 4 * 2 * len(pairs) / msr / 1e6 / peak, 4)
    rotc = lambda: [d.copy_(s_) for _ in range(2) for s_, d in pairs]
    rotc()
    msrc, _ = median_launch_ms(rotc, 10)
    res["sequential_64MiB"]["rotating_copy_ceiling_gbs"] = round(2 * n * 4 * 2 * len(pairs) / msrc / 1e6, 1)
    del pairs
    # the same kernel on 1 GiB, where launch and tail effects no longer dominate
    nb = 1 << 28
    big_s, big_d = seeded_field(nb, 0xC1, -1.0, 1.0), torch.empty(nb, device="cuda")
    if kind == "reference":
        bpt_big = pick_bpt(lambda bpt: ref.seq_copy(big_d, big_s, nb * 4, bpt))
        f = lambda: ref.seq_copy(big_d, big_s, nb * 4, bpt_big["best"])
    else:
        f = lambda: cd.seq_copy(big_d, big_s, nb * 4, 16384, kind)
    for _ in range(3):
        f()
    ms, best = median_launch_ms(f, 10)
    res["sequential_1GiB"] = entry(ms, best, 2 * nb * 4)
    if kind == "reference":
        res["sequential_1GiB"]["bytes_per_thread"] = bpt_big
    ok = torch.equal(big_d.view(torch.int32), big_s.view(torch.int32))
    res["sequential_1GiB"]["parity"] = "pass" if ok else "FAIL"
    g = lambda: big_d.copy_(big_s)
    for _ in range(3):
        g()
    msc, _ = median_launch_ms(g, 10)
    res["sequential_1GiB"]["copy_ceiling_gbs"] = round(2 * nb * 4 / msc / 1e6, 1)
    del big_s, big_d, src, dst

    # strided: 16384 x 16384 transpose in 128 x 64 tiles (1 GiB in, 1 GiB out: larger than L2)
    m = 16384
    a, b = seeded_field(m * m, 0xC2, -1.0, 1.0), torch.zeros(m * m, device="cuda")
    if kind == "reference":
        bpt_tr = pick_bpt(lambda bpt: ref.strided_transpose(b, a, m, m, bpt))
        f = lambda: ref.strided_transpose(b, a, m, m, bpt_tr["best"])
    else:
        f = lambda: cd.strided_transpose(b, a, m, m, kind)
    for _ in range(3):
        f()
    ms, best = median_launch_ms(f, 10)
    res["strided_16384"] = entry(ms, best, 2 * m * m * 4)
    if kind == "reference":
        res["strided_16384"]["bytes_per_thread"] = bpt_tr
    res["strided_16384"]["parity"] = "pass" if same_bits(b, expected("strided")) else "FAIL"
    del a, b

    # indirect: 2^24 x 32 B table, 2^22 gathers, scattered through a permutation
    n, rec = 1 << 22, 1 << 24
    want, perm = expected("indirect")
    table = seeded_field(rec * 8, 0xC3, -1.0, 1.0)
    gi = cd.fill_index(torch.empty(n, dtype=torch.int32, device="cuda"), 0xC3A, rec)
    si = torch.from_numpy(perm).cuda()
    out = torch.zeros(n * 8, device="cuda")
    if kind == "reference":
        bpt_gs = pick_bpt(lambda bpt: ref.gather_scatter(out, table, gi, si, n, bpt), flush)
        f = lambda: ref.gather_scatter(out, table, gi, si, n, bpt_gs["best"])
    else:
        f = lambda: cd.gather_scatter(out, table, gi, si, n, 32, kind)
    for _ in range(3):
        f()
    ms, best = median_launch_ms(f, 20, flush)
    res["indirect_2e22x32B"] = entry(ms, best, n * 72)
    if kind == "reference":
        res["indirect_2e22x32B"]["bytes_per_thread"] = bpt_gs
    res["indirect_2e22x32B"]["payload_gbs"] = round(n * 64 / ms / 1e6, 1)
    res["indirect_2e22x32B"]["parity"] = "pass" if same_bits(out, want) else "FAIL"
    del out
    if kind != "reference":
        # The same 512 MiB table read as 2^22 records of 128 bytes: every record is one whole DRAM
        # line, so this is what random line fetches sustain; a 32-byte record costs such a line too.
        rec128 = rec // 4
        gi128 = gi % rec128
        out = torch.zeros(n * 32, device="cuda")
        f = lambda: cd.gather_scatter(out, table, gi128, si, n, 128, kind)
        for _ in range(3):
            f()
        ms, best = median_launch_ms(f, 10)
        res["indirect_2e22x128B"] = entry(ms, best, n * (2 * 128 + 8))
        head = 1 << 16
        exp = table.view(rec128, 32)[gi128.long()]
        res["indirect_2e22x128B"]["parity"] = "pass" if torch.equal(out.view(n, 32)[si[:head].long()], exp[:head]) else "FAIL"
        del out, exp, gi128
    del table

    # stencil 512^3, 10 steps
    nx, ny, nz = C4
    pts = nx * ny * nz
    if kind == "native":
        a, b = seeded_field(pts, 0xC4), torch.zeros(pts, device="cuda")
        f = lambda: cd.stencil25_run(a, b, nx, ny, nz, 10, None, kind)
    else:
        pad = (nx + 8) * (ny + 8) * (nz + 8)
        a, b = torch.zeros(pad, device="cuda"), torch.zeros(pad, device="cuda")
        a.view(nz + 8, ny + 8, nx + 8)[4:-4, 4:-4, 4:-4] = seeded_field(pts, 0xC4).view(nz, ny, nx)
        coeff = cd.STENCIL_COEFFS
        if kind == "reference":
            choice = pick_reference_stencil(a, b, nx, ny, nz)
            step = reference_stencil_step(choice["best"])
        else:
            step = cd.stencil25_step_padded

        def f():
            x, y = a, b
            for _ in range(10):
                step(y, x, nx, ny, nz, 0, nz, coeff)
                x, y = y, x
    f()
    ms, best = median_launch_ms(f, 5)
    res["stencil_512"] = entry(ms / 10, best / 10, pts * BYTES_PER_POINT)
    res["stencil_512"]["gpts"] = round(pts * 10 / ms / 1e6, 1)
    if kind == "reference":
        res["stencil_512"]["form"] = choice
    del a, b
    if kind != "reference":
        res["device_status"] = cd.device_status()
    return res


def run_examples():
    """The reference's own kernels on both headers (oracle/_ref, built from the reference checkout): its five
    stencil buffering examples on their default problem, its two saxpy example pairs and its throughput
    benchmark, each compiled unmodified against the reference header and against this repository's.
    `ratio` = reference-header time / this-header time (above 1: this header is faster)."""
    import numpy as np
    from oracle import examples as ex, oracle
    out = {}
    if ex.available("libexamples_ours.so", "libexamples_ref.so"):
        dims = ex.STENCIL_DEFAULT_DIMS
        shape = (dims[2] + 8, dims[1] + 8, dims[0] + 8, 2)
        src = oracle.fill_uniform(int(np.prod(shape)), 0xE0, -1.0, 1.0).reshape(shape)
        for kid, name in enumerate(ex.STENCIL_NAMES):
            t = {}
            for which in ("ours", "ref", "ours", "ref"):   # interleaved, best of two
                _, ms = ex.run_stencil(which, kid, src, dims)
                t[which] = min(ms, t.get(which, ms))
            out["stencil_" + name] = {"this_header_ms": round(t["ours"], 4), "reference_header_ms": round(t["ref"], 4),
                                      "ratio": round(t["ref"] / t["ours"], 3),
                                      "this_header_gbs": round(ex.stencil_bandwidth_gbs(dims, t["ours"]), 1),
                                      "reference_header_gbs": round(ex.stencil_bandwidth_gbs(dims, t["ref"]), 1)}
    for example in ("sequential", "strided"):
        tag = "strided_" if example == "strided" else ""
        if not ex.available("libv1saxpy_%sours.so" % tag, "libv1saxpy_%sref.so" % tag):
            continue
        n = ex.saxpy_elements(example)
        x, y = oracle.fill_uniform(n, 0x5A0, 0.0, 1.0), oracle.fill_uniform(n, 0x5B0, 0.0, 1.0)
        for kernel_id, kname in enumerate(("saxpy_cudaDMA", "saxpy_cudaDMA_doublebuffer")):
            t = {}
            for which in ("ours", "ref", "ours", "ref"):
                _, ms = ex.run_saxpy(example, which, kernel_id, x, y, 0.84018773)
                t[which] = min(ms, t.get(which, ms))
            out["%s_%s" % (kname, example)] = {"this_header_ms": round(t["ours"], 4), "reference_header_ms": round(t["ref"], 4),
                                                "ratio": round(t["ref"] / t["ours"], 3)}
            if example == "sequential" and ex.available("libv1saxpy_ours_ro.so"):
                # the same build with -DCUDADMA_SOURCES_READ_ONLY (read-only data path for the staged loads)
                ro = min(ex.run_saxpy(example, "ours_ro", kernel_id, x, y, 0.84018773)[1] for _ in range(2))
                out["%s_%s" % (kname, example)].update(this_header_read_only_sources_ms=round(ro, 4),
                                                       ratio_read_only_sources=round(t["ref"] / ro, 3))
    if ex.available("libperfseq_ours.so", "libperfseq_ref.so"):
        for kid, name in enumerate(ex.PERFSEQ_NAMES):
            g = {}
            for which in ("ours", "ref", "ours", "ref"):
                gbs, _ = ex.run_perf_sequential(which, kid)
                g[which] = max(gbs, g.get(which, gbs))
            out["perf_sequential_" + name] = {"this_header_gbs": round(g["ours"], 1), "reference_header_gbs": round(g["ref"], 1),
                                              "ratio": round(g["ours"] / g["ref"], 3)}
    if ex.available("libsgemv_ours.so", "libsgemv_ref.so"):
        for v, name in enumerate(ex.SGEMV_NAMES):
            t = {}
            for which in ("ours", "ref", "ours", "ref"):
                _, ms = ex.run_sgemv(which, v)
                t[which] = min(ms, t.get(which, ms))
            out["sgemv_" + name] = {"this_header_ms": round(t["ours"], 4), "reference_header_ms": round(t["ref"], 4),
                                    "ratio": round(t["ref"] / t["ours"], 3)}
    if not out:
        return {"unavailable": "oracle/_ref holds no example libraries (no reference checkout at build time)"}
    out["slowest_ratio"] = min(v["ratio"] for v in out.values())   # default builds only
    return out


def host_link_rate(h_in, h_out, world):
    """Every rank copies (up to) 1 GiB of its pinned input to the device and as much from the device to its pinned
    output, on two streams at once, all ranks together; returns the per-direction rates."""
    n = min(h_in.numel(), 1 << 28)
    d_up = torch.empty(n, dtype=torch.float32, device="cuda")
    d_down = torch.zeros(n, dtype=torch.float32, device="cuda")
    keep = h_out[:n].clone()   # the result of the end-to-end run is still needed
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(s_up):
        d_up.copy_(h_in[:n], non_blocking=True)
    with torch.cuda.stream(s_down):
        h_out[:n].copy_(d_down, non_blocking=True)
    torch.cuda.synchronize()
    mine = 4 * n / (time.perf_counter() - t0) / 1e9
    barrier()
    h_out[:n].copy_(keep)
    rates = all_ranks(mine)
    return {"gbs_per_direction_per_rank": [round(r, 1) for r in rates], "gbs_per_direction_sum": round(sum(rates), 1),
            "bytes_per_rank_and_direction": 4 * n,
            "note": "all ranks copy host->device and device->host at the same time, pinned memory, no kernels"}


# ------------------------------------------------------------------ the stencil job
def calibrate_rates(world):
    """Every rank times the stencil kernel alone on a 1024 x 1024 x 256 field of its own GPU, under
    sustained load, and all ranks share the rates (Gpts/s). Power-capped GPUs of one box differ by
    several per cent, and ranks that exchange planes every step run at the pace of the slowest:
    slabs cut in proportion to these rates let them finish a step together."""
    import cudadma_b200 as cd
    import torch.distributed as dist
    nz = 256
    a, b = seeded_field(NX * NY * nz, 0xCA), torch.empty(NX * NY * nz, device="cuda")
    t_end = time.perf_counter() + 0.5
    while time.perf_counter() < t_end:  # reach the power state of a long run first
        cd.stencil25_run(a, b, NX, NY, nz, 10)
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    cd.stencil25_run(a, b, NX, NY, nz, 40)
    e1.record()
    torch.cuda.synchronize()
    rate = NX * NY * nz * 40 / e0.elapsed_time(e1) / 1e6
    rates = [None] * world
    dist.all_gather_object(rates, round(rate, 1))
    return rates


def make_stencil(impl, nz_global, weights=None):
    """The sharded stencil driver with this arm's step function."""
    import cudadma_b200 as cd
    from cudadma_b200.sharded import ShardedStencil
    if impl == "ours":
        return ShardedStencil(NX, NY, nz_global, exchange=EXCHANGE, weights=weights, p2p_signal=P2P_SIGNAL)
    if "best" not in _REFERENCE_STENCIL:
        # which form of the reference-class stencil is fastest here: tried once, on a 1024 x 1024 x 64 padded slab
        pad = (NX + 8) * (NY + 8) * (64 + 8)
        pa, pb = torch.zeros(pad, device="cuda"), torch.zeros(pad, device="cuda")
        pa.view(72, NY + 8, NX + 8)[4:-4, 4:-4, 4:-4] = seeded_field(NX * NY * 64, 0xC4).view(64, NY, NX)
        _REFERENCE_STENCIL["choice"] = pick_reference_stencil(pa, pb, NX, NY, 64)
        del pa, pb
    ref_step = reference_stencil_step(_REFERENCE_STENCIL["best"])

    def step(out, inp, nx, ny, nz_total, zb, ze, coeff):
        # padded layout: the four ghost planes of a slab are the z border of the padded array
        ref_step(out, inp, nx, ny, nz_total - 8, zb - 4, ze - 4, coeff)
    return ShardedStencil(NX, NY, nz_global, step_fn=step, pad_xy=4, device=torch.device("cuda", torch.cuda.current_device()))


def slab_of_global_field(st):
    """This rank's planes of the one global seeded field (seed 0xC4, uniform [0, 1))."""
    return seeded_field(NX * NY * st.nzl, 0xC4, 0.0, 1.0, first_index=st.z_lo * NX * NY)


def sharded_parity(st, world, steps=3):
    """Correctness of the sharded step inside the measured run. The object is reloaded with its
    planes of the global seeded field and stepped `steps` times with halo exchange; every rank then
    recomputes its own planes ALONE, by plain single-GPU steps on the planes [z_lo - 4 steps,
    z_hi + 4 steps) of the same global field (cut at the grid's ends), where nothing depends on a
    neighbour: whatever the cut does wrong travels four planes per step and has not reached the
    owned planes. The two must agree bit for bit on every rank. On one GPU, where there is nothing to
    exchange, the first planes of the result are compared with the double-precision CPU oracle."""
    import cudadma_b200 as cd
    nz = st.nz
    torch.cuda.synchronize()
    barrier()  # no neighbour still pushes planes of the timed steps while this rank reloads its arrays
    st.load(slab_of_global_field(st))
    got = st.run(steps)
    lo, hi = max(0, st.z_lo - 4 * steps), min(nz, st.z_hi + 4 * steps)
    if world > 1:
        pts = NX * NY * (hi - lo)
        a = seeded_field(pts, 0xC4, 0.0, 1.0, first_index=lo * NX * NY)
        b = torch.zeros_like(a)
        alone = cd.stencil25_run(a, b, NX, NY, hi - lo, steps).view(hi - lo, NY, NX)[st.z_lo - lo:st.z_hi - lo]
        ok = bool(torch.equal(alone.view(torch.int32), got.contiguous().view(torch.int32)))
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        verdict = "pass" if int(t.item()) == 1 else "FAIL"
        del a, b, alone
        return {"parity": verdict, "how": "%d steps with halo exchange on every rank against the same planes stepped alone on "
                                          "that rank from the global seeded field: bit-identical on all %d ranks" % (steps, world)
                if verdict == "pass" else "a rank's sharded planes differ from its planes stepped alone"}
    import numpy as np
    from oracle import oracle
    planes = 24
    field = oracle.fill_uniform(NX * NY * (planes + 4 * steps), 0xC4, 0.0, 1.0).reshape(planes + 4 * steps, NY, NX)
    exp = oracle.stencil25_f64(field, cd.STENCIL_COEFFS, steps)[:planes]
    res = got[:planes].cpu().numpy()
    err = float(np.abs(res.astype(np.float64) - exp).max() / np.abs(exp).max())
    return {"parity": "pass" if err <= 1e-5 else "FAIL", "rel_err": err,
            "how": "%d steps of the whole grid from the global seeded field; the first %d planes against the double-precision "
                   "CPU oracle (max |gpu - ref| / max |ref| <= 1e-5)" % (steps, planes)}


def copy_rate_now(seconds):
    """GB/s of a plain device copy (torch copy_ of 1 GiB, read + write bytes) sustained for about
    `seconds`, right now: the copy bandwidth of the GPU in the power state the measured region left it in."""
    n = 1 << 28
    a, b = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    a.zero_()
    b.copy_(a)
    torch.cuda.synchronize()
    reps = max(4, int(seconds * 6.0e12 / (8.0 * n)))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        b.copy_(a)
    e1.record()
    torch.cuda.synchronize()
    return 8.0 * n * reps / e0.elapsed_time(e1) / 1e6


def run_stencil_job(impl, args, rank, world, local, peak, peak_kind):
    import cudadma_b200 as cd
    rates = None
    if impl == "ours" and world > 1 and args.balance:
        rates = calibrate_rates(world)
    st = make_stencil(impl, NZ, rates)
    planes = [st.nzl]
    if world > 1:
        planes = [None] * world
        dist.all_gather_object(planes, st.nzl)
    slab_pts = NX * NY * st.nzl
    field = slab_of_global_field(st)
    st.load(field)
    for _ in range(max(args.warmup, 3)):
        st.step()
    # The warm-up steps have moved the field on; put the seeded field back, so that the timed steps are the job's
    # own steps 1..K (under the GPU's power cap the kernel's speed depends on the values it works on: a field of
    # zeros or NaNs steps up to a quarter faster than one of ordinary numbers)
    st.load(field)
    del field
    probe = SmClockProbe()
    with ClockSampler(local) as clocks:
        probe.fire()
        ms = time_region(st.step, args.steps)
        copy_gbs = copy_rate_now(ms / 1e3)
        if ms < 400.0:  # give the sampler a few periods: repeat the same region, untimed for the record
            reps = int(400.0 / max(ms, 1e-3))
            for i in range(reps):
                if i % 4 == 0:
                    probe.fire()
                for _ in range(args.steps):
                    st.step()
            torch.cuda.synchronize()
    pts = NX * NY * NZ
    value = pts * args.steps / ms / 1e6  # Gpts/s, whole job
    per_step_ms = ms / args.steps
    status = cd.device_status() if impl == "ours" else 0
    sm_mhz = probe.mhz()
    parity = sharded_parity(st, world) if impl == "ours" else None

    # the same job with this repository's kernel but the exchange the reference arm has to use (NCCL send/recv of the
    # boundary planes): against the reference arm's figure it isolates the kernel, against `value` the exchange
    nccl_form = None
    if impl == "ours" and world > 1 and EXCHANGE == "p2p":
        from cudadma_b200.sharded import ShardedStencil
        del st
        torch.cuda.empty_cache()
        stn = ShardedStencil(NX, NY, NZ, exchange="nccl", weights=rates)
        stn.load(slab_of_global_field(stn))
        for _ in range(3):
            stn.step()
        msn = time_region(stn.step, args.steps)
        nccl_form = {"value": round(NX * NY * NZ * args.steps / msn / 1e6, 2), "unit": "Gpts/s",
                     "ms_per_step": round(msn / args.steps, 4),
                     "note": "boundary planes first, torch.distributed send/recv on a side stream, interior meanwhile"}
        del stn
        torch.cuda.empty_cache()
        st = make_stencil(impl, NZ, rates)

    # weak-scaling companion: 256 planes per GPU (the 8-GPU point is the configuration above)
    weak = None
    if not args.no_weak:
        del st
        torch.cuda.empty_cache()
        stw = make_stencil(impl, 256 * world, rates)
        stw.load(seeded_field(NX * NY * stw.nzl, 0xC4, 0.0, 1.0, first_index=stw.z_lo * NX * NY))
        for _ in range(3):
            stw.step()
        msw = time_region(stw.step, args.steps)
        weak = {"grid": [NX, NY, 256 * world], "value": round(NX * NY * 256 * world * args.steps / msw / 1e6, 2),
                "unit": "Gpts/s", "ms_per_step": round(msw / args.steps, 4)}
        # the same object a while later, when the GPUs have settled at their power cap (the figure
        # above is the first 20 steps after a pause)
        for _ in range(30):
            for _ in range(args.steps):
                stw.step()
        msw2 = time_region(stw.step, args.steps)
        weak["settled_ms_per_step"] = round(msw2 / args.steps, 4)
        del stw
        torch.cuda.empty_cache()
        st = make_stencil(impl, NZ, rates)

    # end to end: pinned host slab -> device, K steps with halo exchange, device -> pinned host slab
    h_in = torch.empty(slab_pts, dtype=torch.float32).pin_memory()
    h_out = torch.empty(slab_pts, dtype=torch.float32).pin_memory()
    h_in.copy_(slab_of_global_field(st))
    st.run_host(h_out, h_in, 1)  # warm-up (also faults the pinned pages in)
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    st.run_host(h_out, h_in, args.steps)
    torch.cuda.synchronize()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e = {"value": round(pts * args.steps / e2e_s / 1e9, 3), "unit": "Gpts/s",
           "h2d_bytes_per_step": slab_pts * 4 // args.steps, "d2h_bytes_per_step": slab_pts * 4 // args.steps,
           "note": ("whole job through ShardedStencil.run_host, which on one GPU is the C-ABI call "
                    "cudadma_stencil25_run_host: pinned host field up in 128 MiB pieces, %d steps trailing the "
                    "upload, finished planes down, all overlapped; bytes divided by the steps" % args.steps)
                   if (world == 1 and impl == "ours") else
                   ("whole job through ShardedStencil.run_host, overlapped form: every rank uploads its pinned slab "
                    "in pieces while its %d steps trail the upload and finished planes go back; even ranks walk "
                    "their slab upwards, odd ranks downwards, boundary planes exchanged per step where two walks "
                    "begin or end; bytes are per rank, divided by the steps" % args.steps)
                   if impl == "ours" else
                   ("whole job through ShardedStencil.run_host: the slab is uploaded once, stepped %d times and "
                    "downloaded once; bytes are per rank, divided by the steps" % args.steps),
           "seconds": round(e2e_s, 4)}
    # what the box's host links carry when every rank copies both ways at once (plain cudaMemcpyAsync of the same
    # pinned slabs, no kernels): the bound of any end-to-end figure on this box
    e2e["host_link"] = host_link_rate(h_in, h_out, world)
    if world == 1 and impl == "ours":
        # the overlapped host run against the plain device run on the same input, all 2^31 points
        st.load(h_in)
        want = st.run(args.steps).reshape(-1)
        same, piece = True, 1 << 28
        for i in range(0, slab_pts, piece):
            same = same and torch.equal(want[i:i + piece].view(torch.int32),
                                        h_out[i:i + piece].to("cuda", non_blocking=True).view(torch.int32))
        e2e["parity"] = "pass (bit-identical to the device-resident run)" if same else "FAIL"
    del h_in, h_out

    clock_rec = clocks.summary()
    if sm_mhz:
        clock_rec["sm_mhz_in_kernel"] = {"first": round(probe_first(probe), 0), "median": round(sm_mhz[len(sm_mhz) // 2], 0),
                                         "min": round(sm_mhz[0], 0),
                                         "how": "one-thread probe kernels beside the steps: SM cycles / nanoseconds; `first` ran "
                                                "inside the timed region, the others during the repeats of it"}
    achieved = BYTES_PER_POINT * pts / world / per_step_ms / 1e6
    line = {
        "metric": "stencil Gpts/s (radius-4 25-point fp32, %dx%dx%d z-sharded over N GPUs)" % (NX, NY, NZ),
        "value": round(value, 2), "unit": "Gpts/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(per_step_ms, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "sharded 25-point stencil, grid %dx%dx%d, 64x16 tiles + radius-4 halo, "
                               "4-plane halo exchange per step" % (NX, NY, NZ),
                   "planes_per_gpu": planes if rates else NZ // world,
                   "slab_balance": ({"rates_gpts": rates, "note": "slabs cut in proportion to each GPU's stencil rate, "
                                     "measured alone on a 256-plane field just before"} if rates else "equal slabs"),
                   "exchange": ("none" if world == 1 else "torch.distributed send/recv (NCCL)" if (impl != "ours" or EXCHANGE == "nccl")
                                else "boundary CTAs wait for the neighbours' step count and store their planes into the neighbours' "
                                     "ghost planes over NVLink (CUDA IPC); the step count is published by " +
                                     ("the kernel's last boundary CTA (one launch per step)" if P2P_SIGNAL == "fused"
                                      else "a one-thread launch behind the kernel")),
                   "l2": "inputs larger than L2 (%.1f GiB per array per GPU)" % (slab_pts * 4 / 2**30),
                   "synthetic_for": "uniform[0,1) field, element i = u(splitmix64(0xC4 + i)), the same global field at every N"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1),
                     "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4),
                     "traffic": int(STENCIL_DRAM_BYTES_PER_POINT * pts / world) if impl == "ours" else None,
                     "peak_kind": "of " + peak_kind,
                     "kernel": "stencil25::tensor_kernel" if impl == "ours" else "portable::stencil_kernel",
                     "algorithmic_bytes_per_launch": BYTES_PER_POINT * pts // world,
                     "copy_gbs_right_after": round(copy_gbs, 1),
                     "frac_of_copy_right_after": round(achieved / copy_gbs, 4),
                     "copy_note": "a plain device copy (torch copy_, 1 GiB, read + write bytes) run for as long as the timed "
                                  "region, directly after it, on rank 0's GPU: the copy bandwidth in the same power state"},
        "e2e": e2e, "clocks": clock_rec, "device_status": status,
    }
    if parity is not None:
        line["parity"] = parity["parity"]
        line["parity_detail"] = parity
    if weak is not None:
        line["weak"] = weak
    if nccl_form is not None:
        line["nccl_exchange"] = nccl_form
    return line, st


def probe_first(probe):
    h = probe.buf.cpu().view(-1, 2)[0].tolist()
    return float(h[0]) / float(h[1]) * 1e3 if h[1] else 0.0


def profile_case(case, reps):
    """A small, fixed case of one kernel for a profiler capture: few launches, no timing, no JSON.
    Sizes exceed the L2 (so DRAM counters mean something) and stay near 1 GiB on the device."""
    import cudadma_b200 as cd
    torch.cuda.set_device(0)
    if case == "stencil_512":
        nx, ny, nz = C4
        a, b = seeded_field(nx * ny * nz, 0xC4), torch.zeros(nx * ny * nz, device="cuda")
        for _ in range(reps):
            cd.stencil25_step(b, a, nx, ny, nz)
            a, b = b, a
    elif case == "stencil_c5":
        # the sharded configuration's whole grid on one GPU (8 GiB per array): only for captures that take ONE pass
        a, b = seeded_field(NX * NY * NZ, 0xC4), torch.zeros(NX * NY * NZ, device="cuda")
        for _ in range(reps):
            cd.stencil25_step(b, a, NX, NY, NZ)
            a, b = b, a
    elif case == "sequential":
        n = 1 << 27  # 512 MiB in, 512 MiB out
        a, b = seeded_field(n, 0xC1), torch.empty(n, device="cuda")
        for _ in range(reps):
            cd.seq_copy(b, a, n * 4)
    elif case == "strided":
        m = 8192     # 256 MiB in, 256 MiB out
        a, b = seeded_field(m * m, 0xC2), torch.empty(m * m, device="cuda")
        for _ in range(reps):
            cd.strided_transpose(b, a, m, m)
    elif case in ("indirect", "indirect_tma", "indirect_scatter4", "indirect_portable"):
        n, rec = 1 << 22, 1 << 24
        table = seeded_field(rec * 8, 0xC3, -1.0, 1.0)
        gi = cd.fill_index(torch.empty(n, dtype=torch.int32, device="cuda"), 0xC3A, rec)
        si = torch.randperm(n, device="cuda").to(torch.int32)
        out = torch.zeros(n * 8, device="cuda")
        for _ in range(reps):
            if case == "indirect":
                cd.gather_scatter(out, table, gi, si, n)
            elif case == "indirect_portable":
                cd.gather_scatter(out, table, gi, si, n, 32, "portable")
            else:
                cd.gather_scatter_tma(out, n, table, rec, gi, si, n, 32, 1 if case == "indirect_tma" else 2)
    else:
        raise SystemExit("unknown case " + case)
    torch.cuda.synchronize()
    if cd.device_status() != 0:
        raise SystemExit("a wait inside a kernel gave up")
    print("profile case %s: %d launches done" % (case, reps))


def claim_stdout():
    """Libraries underneath (NCCL's version banner, for one) write to file descriptor 1. Point it at
    stderr for the duration of the run and return a file on the real stdout for the JSON line."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    json_out = claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-patterns", action="store_true", help="skip the single-GPU data-movement patterns")
    ap.add_argument("--no-weak", action="store_true", help="skip the weak-scaling companion run")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--no-balance", dest="balance", action="store_false",
                    help="equal slabs on every GPU instead of slabs in proportion to the GPUs' measured rates")
    ap.add_argument("--exchange", default="p2p", choices=("p2p", "nccl"),
                    help="halo exchange at N > 1: peer-to-peer stores from the boundary kernel, or NCCL send/recv")
    ap.add_argument("--p2p-signal", default=None, choices=("trailing", "trailing-ascending", "fused"),
                    help="p2p exchange: the step count is published by a one-thread launch behind the step's kernel "
                         "(trailing, the library's default) or by the kernel's last boundary CTA (fused, one launch per step)")
    ap.add_argument("--profile-case", default=None,
                    help="run only a small case of one kernel (stencil_512, stencil_c5, sequential, strided, indirect, indirect_tma, "
                         "indirect_scatter4, indirect_portable) "
                         "--steps times, for a profiler capture")
    args = ap.parse_args()
    global EXCHANGE, P2P_SIGNAL
    EXCHANGE = args.exchange
    P2P_SIGNAL = args.p2p_signal
    peak, peak_kind = measured_peaks()
    if args.profile_case:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device")
        profile_case(args.profile_case, args.steps)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    rank, world, local = setup_dist(args.gpus)

    impl = args.impl
    ref_gpu = False
    if impl == "reference":
        from oracle import reference as ref
        ref_gpu = ref.available() and hasattr(ref.lib(), "cudadma_ref_stencil25_step_padded")
        if not ref_gpu:
            # the reference's classes were not compiled here: time the CPU restatement, rank 0 only
            if rank == 0:
                cb = cpu_baseline_stencil()
                cpu_line = {
                    "impl": "reference", "metric": "stencil Gpts/s (radius-4 25-point fp32, %dx%dx%d)" % (NX, NY, NZ),
                    "value": round(cb["value"], 4), "unit": "Gpts/s", "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": round(NX * NY * NZ / cb["value"] / 1e6, 2),
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                    "data": "synthetic", "config": {"workload": "CPU restatement, " + cb["sample"]},
                    "cpu_baseline": cb,
                    "e2e": {"value": round(cb["value"], 4), "unit": "Gpts/s", "h2d_bytes_per_step": 0,
                            "d2h_bytes_per_step": 0}}
                print(json.dumps(cpu_line), file=json_out, flush=True)
            if dist.is_initialized():
                dist.destroy_process_group()
            return

    import cudadma_b200 as cd
    before = cd.launch_count()
    line, st = run_stencil_job(impl, args, rank, world, local, peak, peak_kind)
    del st
    torch.cuda.empty_cache()
    if impl == "ours":
        # launches of this library per timed step: one kernel at one GPU; p2p: the kernel and the one-thread launch
        # that publishes the step count (fused: the kernel alone); the nccl form: two boundary runs and the interior
        if world > 1:
            line["config"]["host_threads"] = ("each rank bound to the %d cores NVML lists for its GPU" % len(HOST_CORES)) if HOST_CORES \
                else "not bound (no NVML core list)"
        line["gpu_launches"] = args.steps * (1 if (world == 1 or (EXCHANGE == "p2p" and P2P_SIGNAL == "fused")) else
                                             2 if EXCHANGE == "p2p" else 3)
        line["launches_total_this_process"] = cd.launch_count() - before
    else:
        line["impl"] = "reference"
        line["config"]["reference_build"] = ("reference CudaDMA classes compiled for sm_100a on zero-padded arrays; the fastest of: "
                                             "whole windows by CudaDMAStrided (cudaDMAv2.h) with BYTES_PER_THREAD 64 / 128 / 192, "
                                             "ring by v1 cudaDMAHalo + interior by cudaDMAStrided (cudaDMA.h)")
        line["config"]["reference_stencil_form"] = _REFERENCE_STENCIL.get("choice", _REFERENCE_STENCIL.get("best"))
    if rank == 0 and world == 1 and not args.no_patterns:
        if impl == "ours":
            line["patterns"] = {"native": run_patterns("native", peak), "portable": run_patterns("portable", peak)}
            line["patterns"]["examples"] = run_examples()
        else:
            line["patterns"] = {"reference": run_patterns("reference", peak)}
    if rank == 0 and not args.no_cpu and (world == 1 or impl == "reference"):
        line["cpu_baseline"] = cpu_baseline_stencil()
        if world == 1:
            line["cpu_baseline"]["patterns"] = cpu_baseline_patterns()
    if rank == 0:
        print(json.dumps(line), file=json_out, flush=True)
    if dist.is_initialized():
        barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
