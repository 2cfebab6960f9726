"""ctypes binding of libcudadma_b200.so (declarations: include/cudadma_b200.h).

The library is the product; this module only loads it and checks arguments and
status codes. There is no CPU fallback: a missing library raises at first use,
and every compute call needs a CUDA device.

Tensors are torch CUDA tensors (torch supplies device memory and streams);
raw integer device addresses are accepted too.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcudadma_b200.so")

OK, ERR_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_NOMEM, ERR_TIMEOUT = 0, -1, -2, -3, -4, 1
ERR_TOO_LARGE = -5
IMPL_NATIVE, IMPL_PORTABLE = 0, 1
_IMPLS = {"native": IMPL_NATIVE, "portable": IMPL_PORTABLE, IMPL_NATIVE: IMPL_NATIVE, IMPL_PORTABLE: IMPL_PORTABLE}

# every symbol include/cudadma_b200.h declares: (name, restype, argtypes)
_c = ctypes
SYMBOLS = [
    ("cudadma_version", _c.c_int, []),
    ("cudadma_status_string", _c.c_char_p, [_c.c_int]),
    ("cudadma_last_cuda_error", _c.c_int, []),
    ("cudadma_device_status", _c.c_int, [_c.c_void_p, _c.POINTER(_c.c_uint)]),
    ("cudadma_launch_count", _c.c_ulonglong, []),
    ("cudadma_seq_copy", _c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int, _c.c_int, _c.c_void_p]),
    ("cudadma_strided_transpose", _c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    ("cudadma_gather_scatter", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int, _c.c_int, _c.c_void_p]),
    ("cudadma_gather_scatter_tma", _c.c_int,
     [_c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int, _c.c_int,
      _c.c_void_p]),
    ("cudadma_make_tensor_map_2d", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_ulonglong, _c.c_ulonglong, _c.c_ulonglong, _c.c_uint, _c.c_uint, _c.c_int]),
    ("cudadma_make_tensor_map_3d", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_ulonglong, _c.c_ulonglong, _c.c_ulonglong, _c.c_ulonglong, _c.c_ulonglong,
      _c.c_uint, _c.c_uint, _c.c_uint]),
    ("cudadma_fill_uniform", _c.c_int,
     [_c.c_void_p, _c.c_size_t, _c.c_ulonglong, _c.c_ulonglong, _c.c_float, _c.c_float, _c.c_void_p]),
    ("cudadma_fill_index", _c.c_int,
     [_c.c_void_p, _c.c_size_t, _c.c_ulonglong, _c.c_ulonglong, _c.c_uint, _c.c_void_p]),
    ("cudadma_clock_probe", _c.c_int, [_c.c_void_p, _c.c_longlong, _c.c_void_p]),
    ("cudadma_stencil25_step", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_float), _c.c_int,
      _c.c_int, _c.c_void_p]),
    ("cudadma_stencil25_run", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_float), _c.c_int, _c.c_int,
      _c.c_void_p]),
    ("cudadma_stencil25_step_padded", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_float), _c.c_int,
      _c.c_int, _c.c_void_p]),
    ("cudadma_stencil25_step_noalloc", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_float), _c.c_void_p]),
    ("cudadma_slab_create", _c.c_int, [_c.POINTER(_c.c_void_p), _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int]),
    ("cudadma_slab_handle_bytes", _c.c_size_t, []),
    ("cudadma_slab_export", _c.c_int, [_c.c_void_p, _c.c_void_p]),
    ("cudadma_slab_connect", _c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p]),
    ("cudadma_slab_connect_local", _c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p]),
    ("cudadma_slab_set_wait_limit", _c.c_int, [_c.c_void_p, _c.c_longlong]),
    ("cudadma_slab_set_edge_planes", _c.c_int, [_c.c_void_p, _c.c_int]),
    ("cudadma_slab_set_signal_mode", _c.c_int, [_c.c_void_p, _c.c_int]),
    ("cudadma_slab_set_run_order", _c.c_int, [_c.c_void_p, _c.c_int]),
    ("cudadma_slab_buffer", _c.c_int, [_c.c_void_p, _c.c_int, _c.POINTER(_c.c_void_p)]),
    ("cudadma_slab_step", _c.c_int, [_c.c_void_p, _c.POINTER(_c.c_float), _c.c_void_p]),
    ("cudadma_slab_status", _c.c_int, [_c.c_void_p, _c.c_void_p]),
    ("cudadma_slab_destroy", _c.c_int, [_c.c_void_p]),
    ("cudadma_stencil25_multi_create", _c.c_int,
     [_c.POINTER(_c.c_void_p), _c.c_int, _c.POINTER(_c.c_int), _c.c_int, _c.c_int, _c.c_int]),
    ("cudadma_stencil25_multi_load", _c.c_int, [_c.c_void_p, _c.c_void_p]),
    ("cudadma_stencil25_multi_run", _c.c_int, [_c.c_void_p, _c.POINTER(_c.c_float), _c.c_int]),
    ("cudadma_stencil25_multi_store", _c.c_int, [_c.c_void_p, _c.c_void_p]),
    ("cudadma_stencil25_multi_slab", _c.c_int,
     [_c.c_void_p, _c.c_int, _c.POINTER(_c.c_void_p), _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    ("cudadma_stencil25_multi_destroy", _c.c_int, [_c.c_void_p]),
    ("cudadma_seq_copy_host", _c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int, _c.c_int]),
    ("cudadma_strided_transpose_host", _c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int]),
    ("cudadma_gather_scatter_host", _c.c_int,
     [_c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_int, _c.c_int]),
    ("cudadma_stencil25_run_host", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_float), _c.c_int, _c.c_int]),
    ("cudadma_stencil25_run_host_pipelined", _c.c_int,
     [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_float), _c.c_int, _c.c_int, _c.c_int]),
    ("cudadma_release_workspace", _c.c_int, []),
]

# the benchmark's stencil coefficients c0..c4
STENCIL_COEFFS = (-2.847, 1.6, -0.2, 0.0254, -0.00179)

_lib = None


class CudaDMAError(RuntimeError):
    def __init__(self, call, status, detail=""):
        self.status = status
        super().__init__("%s failed with status %d (%s)%s" % (call, status, detail, ""))


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU fallback)" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS:
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def _check(call, status):
    if status != OK:
        l = lib()
        detail = l.cudadma_status_string(status).decode()
        if status == ERR_CUDA:
            detail += ", cudaError %d" % l.cudadma_last_cuda_error()
        raise CudaDMAError(call, status, detail)


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):  # torch tensor
        return x.data_ptr()
    if hasattr(x, "ctypes"):  # numpy array (host-buffer forms)
        return x.ctypes.data
    raise TypeError("expected a tensor, an array or an address, got %r" % type(x))


def _stream(stream):
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _coeffs(coeff):
    coeff = STENCIL_COEFFS if coeff is None else coeff
    if len(coeff) != 5:
        raise ValueError("the stencil takes five coefficients c0..c4")
    return (ctypes.c_float * 5)(*[float(c) for c in coeff])


def _require_cuda(*tensors):
    for t in tensors:
        if hasattr(t, "is_cuda") and not t.is_cuda:
            raise ValueError("device calls take CUDA tensors; use the *_host form for host memory")
        if hasattr(t, "is_contiguous") and not t.is_contiguous():
            raise ValueError("tensors must be contiguous")


def version():
    return lib().cudadma_version()


def launch_count():
    return int(lib().cudadma_launch_count())


def device_status(stream=None):
    """Reads and clears the device status word (0 = no wait gave up). Synchronises the stream."""
    out = ctypes.c_uint(0)
    _check("cudadma_device_status", lib().cudadma_device_status(_stream(stream), ctypes.byref(out)))
    return out.value


def seq_copy(dst, src, nbytes=None, chunk_bytes=16384, impl="native", stream=None):
    _require_cuda(dst, src)
    if nbytes is None:
        nbytes = src.numel() * src.element_size()
    _check("cudadma_seq_copy",
           lib().cudadma_seq_copy(_ptr(dst), _ptr(src), nbytes, chunk_bytes, _IMPLS[impl], _stream(stream)))


def strided_transpose(dst, src, rows, cols, impl="native", stream=None):
    _require_cuda(dst, src)
    _check("cudadma_strided_transpose",
           lib().cudadma_strided_transpose(_ptr(dst), _ptr(src), rows, cols, _IMPLS[impl], _stream(stream)))


def gather_scatter(out, table, gather_idx, scatter_idx, n=None, record_bytes=32, impl="native", stream=None):
    _require_cuda(out, table, gather_idx, scatter_idx)
    if n is None:
        n = gather_idx.numel()
    _check("cudadma_gather_scatter",
           lib().cudadma_gather_scatter(_ptr(out), _ptr(table), _ptr(gather_idx), _ptr(scatter_idx), n, record_bytes,
                                        _IMPLS[impl], _stream(stream)))


def gather_scatter_tma(out, out_records, table, table_records, gather_idx, scatter_idx, n=None, record_bytes=32,
                       mode=1, stream=None):
    """gather_scatter with TMA row instructions, four records each: mode 1 = gather4 loads,
    2 = scatter4 stores, 3 = both."""
    _require_cuda(out, table, gather_idx, scatter_idx)
    if n is None:
        n = gather_idx.numel()
    _check("cudadma_gather_scatter_tma",
           lib().cudadma_gather_scatter_tma(_ptr(out), out_records, _ptr(table), table_records, _ptr(gather_idx),
                                            _ptr(scatter_idx), n, record_bytes, mode, _stream(stream)))


def make_tensor_map_2d(base, cols, rows, row_pitch_bytes, box_cols, box_rows, swizzle_128b=False):
    """A 128-byte CUtensorMap (as a ctypes buffer, 64-byte aligned) over a 2-D array of 4-byte words."""
    raw = ctypes.create_string_buffer(128 + 64)
    addr = (ctypes.addressof(raw) + 63) & ~63
    _check("cudadma_make_tensor_map_2d",
           lib().cudadma_make_tensor_map_2d(addr, _ptr(base), cols, rows, row_pitch_bytes, box_cols, box_rows,
                                            int(bool(swizzle_128b))))
    return ctypes.string_at(addr, 128)


def make_tensor_map_3d(base, nx, ny, nz, row_pitch_bytes, plane_pitch_bytes, box_x, box_y, box_z):
    raw = ctypes.create_string_buffer(128 + 64)
    addr = (ctypes.addressof(raw) + 63) & ~63
    _check("cudadma_make_tensor_map_3d",
           lib().cudadma_make_tensor_map_3d(addr, _ptr(base), nx, ny, nz, row_pitch_bytes, plane_pitch_bytes, box_x,
                                            box_y, box_z))
    return ctypes.string_at(addr, 128)


def fill_uniform(dst, seed, lo=0.0, hi=1.0, first_index=0, n=None, stream=None):
    """dst[i] = lo + (hi - lo) * u(seed + first_index + i): the seeded generator of the benchmark inputs."""
    _require_cuda(dst)
    n = dst.numel() if n is None else n
    _check("cudadma_fill_uniform", lib().cudadma_fill_uniform(_ptr(dst), n, seed, first_index, lo, hi, _stream(stream)))
    return dst


def fill_index(dst, seed, modulo, first_index=0, n=None, stream=None):
    _require_cuda(dst)
    n = dst.numel() if n is None else n
    _check("cudadma_fill_index", lib().cudadma_fill_index(_ptr(dst), n, seed, first_index, modulo, _stream(stream)))
    return dst


def clock_probe(out, spin_ns, stream=None):
    """out: int64 CUDA tensor of two elements; receives SM cycles and nanoseconds of a spin_ns spin."""
    _require_cuda(out)
    _check("cudadma_clock_probe", lib().cudadma_clock_probe(_ptr(out), spin_ns, _stream(stream)))


def stencil25_step(out, inp, nx, ny, nz, z_begin=0, z_end=None, coeff=None, z_chunk=0, impl="native", stream=None):
    _require_cuda(out, inp)
    if z_end is None:
        z_end = nz
    _check("cudadma_stencil25_step",
           lib().cudadma_stencil25_step(_ptr(out), _ptr(inp), nx, ny, nz, z_begin, z_end, _coeffs(coeff), z_chunk,
                                        _IMPLS[impl], _stream(stream)))


def stencil25_step_padded(out, inp, nx, ny, nz, z_begin=0, z_end=None, coeff=None, z_chunk=0, impl="portable",
                          stream=None):
    """One step on arrays padded by four zero cells on every side (portable kernels only)."""
    _require_cuda(out, inp)
    if z_end is None:
        z_end = nz
    _check("cudadma_stencil25_step_padded",
           lib().cudadma_stencil25_step_padded(_ptr(out), _ptr(inp), nx, ny, nz, z_begin, z_end, _coeffs(coeff),
                                               z_chunk, _IMPLS[impl], _stream(stream)))


def stencil25_step_noalloc(out, inp, nx, ny, nz, coeff=None, stream=None):
    """One full step through the entry point that allocates no device memory: for solvers whose
    framework owns all device memory, or whose time-step loop cannot afford the device-wide stall
    of cudaMalloc. The padded grid is limited to 2**21 cells; larger grids raise with status
    ERR_TOO_LARGE. Calls share one built-in scratch array, so keep them ordered on the GPU."""
    _require_cuda(out, inp)
    _check("cudadma_stencil25_step_noalloc",
           lib().cudadma_stencil25_step_noalloc(_ptr(out), _ptr(inp), nx, ny, nz, _coeffs(coeff), _stream(stream)))


def stencil25_run(a, b, nx, ny, nz, steps, coeff=None, impl="native", stream=None):
    """`steps` ping-pong steps starting from `a`; returns the tensor that holds the result."""
    _require_cuda(a, b)
    _check("cudadma_stencil25_run",
           lib().cudadma_stencil25_run(_ptr(a), _ptr(b), nx, ny, nz, _coeffs(coeff), steps, _IMPLS[impl],
                                       _stream(stream)))
    return a if steps % 2 == 0 else b


# ---- slabs of the z-sharded stencil with peer-to-peer halo pushes ----

SIGNAL_MODES = {"trailing": (0, 1), "trailing-ascending": (0, 0), "fused": (1, None)}


def _set_signal_mode(handle, mode):
    signal, highest_first = SIGNAL_MODES[mode]
    _check("cudadma_slab_set_signal_mode", lib().cudadma_slab_set_signal_mode(handle, signal))
    if highest_first is not None:
        _check("cudadma_slab_set_run_order", lib().cudadma_slab_set_run_order(handle, highest_first))


class Slab:
    """This rank's planes of a z-sharded grid, in two arrays the library allocates so that the
    z-neighbour processes can map them (CUDA IPC) and push their boundary planes into the ghost
    planes. export() bytes go to both neighbours by any means; connect() takes theirs."""

    def __init__(self, nx, ny, nzl, has_lower, has_upper):
        self.nx, self.ny, self.nzl = nx, ny, nzl
        h = ctypes.c_void_p()
        _check("cudadma_slab_create", lib().cudadma_slab_create(ctypes.byref(h), nx, ny, nzl, int(has_lower),
                                                                int(has_upper)))
        self._h = h

    def export(self):
        buf = ctypes.create_string_buffer(lib().cudadma_slab_handle_bytes())
        _check("cudadma_slab_export", lib().cudadma_slab_export(self._h, buf))
        return buf.raw

    def connect(self, lower, upper):
        _check("cudadma_slab_connect", lib().cudadma_slab_connect(self._h, lower, upper))

    def connect_local(self, lower, upper):
        """Joins slabs of this process: lower / upper are Slab objects (or None)."""
        _check("cudadma_slab_connect_local",
               lib().cudadma_slab_connect_local(self._h, lower._h if lower is not None else None,
                                                upper._h if upper is not None else None))

    def set_wait_limit(self, sm_cycles):
        _check("cudadma_slab_set_wait_limit", lib().cudadma_slab_set_wait_limit(self._h, int(sm_cycles)))

    def set_signal_mode(self, mode):
        """mode: "trailing" (a one-thread launch behind the step publishes the step count; the runs of
        planes are dispatched from the top down), "trailing-ascending" (the same with the runs from the
        bottom up) or "fused" (one launch per step; the last boundary CTA publishes)."""
        _set_signal_mode(self._h, mode)

    def set_edge_planes(self, planes):
        _check("cudadma_slab_set_edge_planes", lib().cudadma_slab_set_edge_planes(self._h, int(planes)))

    def status(self, stream=None):
        """Synchronises the stream; OK, or ERR_TIMEOUT once a wait for a neighbour has given up."""
        return lib().cudadma_slab_status(self._h, _stream(stream))

    def buffer_address(self, which=0):
        p = ctypes.c_void_p()
        _check("cudadma_slab_buffer", lib().cudadma_slab_buffer(self._h, which, ctypes.byref(p)))
        return p.value

    def tensor(self, which=0):
        """The array as a flat float32 torch tensor over the library's memory (no copy)."""
        import torch
        n = (self.nzl + 8) * self.ny * self.nx

        class _Raw:
            __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (self.buffer_address(which), False),
                                        "version": 2}
        return torch.as_tensor(_Raw(), device="cuda")

    def step(self, coeff=None, stream=None):
        _check("cudadma_slab_step", lib().cudadma_slab_step(self._h, _coeffs(coeff), _stream(stream)))

    def destroy(self):
        if self._h is not None:
            lib().cudadma_slab_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class MultiStencil:
    """The sharded stencil driven from this one process through cudadma_stencil25_multi_*: one slab
    per entry of `devices` (default: GPUs 0 .. n_gpus - 1; repeated entries put several slabs on
    one GPU), host fields in, host fields out."""

    def __init__(self, n_gpus, nx, ny, nz, devices=None, signal_mode=None):
        self.n, self.nx, self.ny, self.nz = n_gpus, nx, ny, nz
        h = ctypes.c_void_p()
        dev = None if devices is None else (ctypes.c_int * n_gpus)(*[int(d) for d in devices])
        _check("cudadma_stencil25_multi_create", lib().cudadma_stencil25_multi_create(ctypes.byref(h), n_gpus, dev, nx, ny, nz))
        self._h = h
        if signal_mode is not None:   # "trailing" or "fused", see Slab.set_signal_mode
            for r in range(n_gpus):
                s = ctypes.c_void_p()
                _check("cudadma_stencil25_multi_slab", lib().cudadma_stencil25_multi_slab(self._h, r, ctypes.byref(s), None, None))
                _set_signal_mode(s, signal_mode)

    def load(self, h_field):
        _check("cudadma_stencil25_multi_load", lib().cudadma_stencil25_multi_load(self._h, _ptr(h_field)))

    def run(self, steps, coeff=None):
        _check("cudadma_stencil25_multi_run", lib().cudadma_stencil25_multi_run(self._h, _coeffs(coeff), steps))

    def store(self, h_field):
        _check("cudadma_stencil25_multi_store", lib().cudadma_stencil25_multi_store(self._h, _ptr(h_field)))

    def planes(self, rank):
        lo, hi = ctypes.c_int(), ctypes.c_int()
        _check("cudadma_stencil25_multi_slab",
               lib().cudadma_stencil25_multi_slab(self._h, rank, None, ctypes.byref(lo), ctypes.byref(hi)))
        return lo.value, hi.value

    def destroy(self):
        if self._h is not None:
            lib().cudadma_stencil25_multi_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


# ---- host-buffer forms (numpy arrays or pinned CPU tensors) ----

def seq_copy_host(h_dst, h_src, nbytes, chunk_bytes=16384, impl="native"):
    _check("cudadma_seq_copy_host",
           lib().cudadma_seq_copy_host(_ptr(h_dst), _ptr(h_src), nbytes, chunk_bytes, _IMPLS[impl]))


def strided_transpose_host(h_dst, h_src, rows, cols, impl="native"):
    _check("cudadma_strided_transpose_host",
           lib().cudadma_strided_transpose_host(_ptr(h_dst), _ptr(h_src), rows, cols, _IMPLS[impl]))


def gather_scatter_host(h_out, out_records, h_table, table_records, h_gather_idx, h_scatter_idx, n, record_bytes=32,
                        impl="native"):
    _check("cudadma_gather_scatter_host",
           lib().cudadma_gather_scatter_host(_ptr(h_out), out_records, _ptr(h_table), table_records,
                                             _ptr(h_gather_idx), _ptr(h_scatter_idx), n, record_bytes, _IMPLS[impl]))


def stencil25_run_host(h_out, h_in, nx, ny, nz, steps, coeff=None, impl="native", chunk_planes=None):
    """`steps` steps from and to host memory. chunk_planes: piece size of the overlapped form
    (None = the library's choice, see cudadma_stencil25_run_host_pipelined)."""
    if chunk_planes is None:
        _check("cudadma_stencil25_run_host",
               lib().cudadma_stencil25_run_host(_ptr(h_out), _ptr(h_in), nx, ny, nz, _coeffs(coeff), steps, _IMPLS[impl]))
    else:
        _check("cudadma_stencil25_run_host_pipelined",
               lib().cudadma_stencil25_run_host_pipelined(_ptr(h_out), _ptr(h_in), nx, ny, nz, _coeffs(coeff), steps,
                                                          _IMPLS[impl], chunk_planes))


def release_workspace():
    _check("cudadma_release_workspace", lib().cudadma_release_workspace())
