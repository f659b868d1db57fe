"""`Nx.Backend` for B200 tensors.

Tensor storage is a device buffer owned by the native runtime; the callbacks
below are the ones nx/lib/nx/backend.ex:46-144 requires for the hot path:
``from_binary to_binary backend_copy backend_transfer backend_deallocate`` plus
every compute callback, which — exactly like EXLA.Backend
(exla/lib/exla/backend.ex:363-431) — is the compiler applied to a one-node
graph.  Anything the compiler does not implement raises; there is no host
implementation to fall back to.
"""
from __future__ import annotations

import ctypes as C
import math
import threading

from . import expr as E
from . import nif
from . import types as T

_state = threading.local()
_default = {"backend": None}


class DeviceBuffer:
    """``%EXLA.DeviceBuffer{ref, device_id, typespec}`` (exla/lib/exla/device_buffer.ex:9-10).
    Dropping the last reference releases the handle, as the BEAM's GC does for
    a NIF resource (exla/c_src/exla/exla_client.cc:22-26)."""
    __slots__ = ("handle", "device", "__weakref__")

    def __init__(self, handle, device):
        self.handle, self.device = handle, device

    def __del__(self):
        h, self.handle = self.handle, None
        if h and getattr(nif, "_LIB", None) is not None:
            try:
                nif._LIB.nxb200_buffer_release(h)
            except Exception:
                pass

    def __repr__(self):
        return f"B200.Backend<cuda:{self.device}>"


def set_default_backend(backend, device=0):
    """``Nx.default_backend/1`` (nx/lib/nx.ex:5006-5009).  ``backend`` is
    ``"b200"`` or None (host storage only)."""
    if backend not in (None, "b200"):
        raise ValueError(f"unknown backend {backend!r}")
    _default["backend"] = None if backend is None else ("b200", int(device))


def default_backend():
    return _default["backend"]


def tracing():
    return getattr(_state, "tracing", 0) > 0


class trace_scope:
    def __enter__(self):
        _state.tracing = getattr(_state, "tracing", 0) + 1

    def __exit__(self, *a):
        _state.tracing -= 1


def _device_of(opts_device=None):
    if opts_device is not None:
        return int(opts_device)
    d = default_backend()
    return d[1] if d else 0


# ---- storage callbacks ------------------------------------------------------------

def from_binary(raw, type, shape, device=None):
    """``from_binary/3`` (exla/lib/exla/backend.ex:43-50 -> binary_to_device_mem)."""
    from .nx import Tensor
    l = nif.lib()
    dev = _device_of(device)
    out = C.c_void_p()
    raw = bytes(raw)
    nif.check(l.nxb200_buffer_from_host(dev, T.DTYPE_CODES[type], nif.dims_array(shape), len(shape),
                                        raw, len(raw), C.byref(out)))
    return Tensor(DeviceBuffer(out.value, dev), type, shape)


def backend_transfer(t, device=None):
    """``backend_transfer/3``: host -> device copies; a tensor already on the
    target device is returned as is (exla/lib/exla/backend.ex:68-78)."""
    from .nx import HostData
    dev = _device_of(device)
    if isinstance(t.data, HostData):
        return from_binary(t.data.raw, t.type, t.shape, dev)
    if isinstance(t.data, DeviceBuffer):
        if t.data.device == dev:
            return t
        moved = backend_copy(t, dev)
        backend_deallocate(t)
        return moved
    raise TypeError("cannot transfer an expression")


def backend_copy(t, device=None):
    """``backend_copy/3`` (exla/lib/exla/backend.ex:53-66 -> copy_buffer_to_device)."""
    from .nx import Tensor, HostData
    dev = _device_of(device)
    if isinstance(t.data, HostData):
        return from_binary(t.data.raw, t.type, t.shape, dev)
    out = C.c_void_p()
    nif.check(nif.lib().nxb200_buffer_copy_to_device(t.data.handle, dev, C.byref(out)))
    return Tensor(DeviceBuffer(out.value, dev), t.type, t.shape)


def to_host(t):
    """Transfer to host storage (``Nx.backend_transfer(t, Nx.BinaryBackend)``)."""
    from .nx import Tensor, HostData, to_binary
    if isinstance(t.data, HostData):
        return t
    return Tensor(HostData(to_binary(t)), t.type, t.shape)


class Pointer:
    """``%Nx.Pointer{kind, address, handle, data_size}`` (nx/lib/nx/pointer.ex)."""
    __slots__ = ("kind", "address", "handle", "data_size")

    def __init__(self, kind, address=None, handle=None, data_size=0):
        self.kind, self.address, self.handle, self.data_size = kind, address, handle, data_size


def to_pointer(t, mode="local"):
    """``Nx.to_pointer/2`` (exla/lib/exla/backend.ex:86-134): ``"local"`` gives the device address,
    ``"ipc"`` a CUDA IPC handle another process can map (``address`` then holds the device id)."""
    if not isinstance(t.data, DeviceBuffer):
        raise ValueError("tensor must be allocated on the device")
    size = t.size * T.itemsize(t.type)
    l = nif.lib()
    if mode == "local":
        p = C.c_void_p()
        nif.check(l.nxb200_buffer_device_pointer(t.data.handle, C.byref(p)))
        return Pointer("local", address=p.value, data_size=size)
    if mode == "ipc":
        h = C.create_string_buffer(64)
        nif.check(l.nxb200_buffer_ipc_export(t.data.handle, h))
        return Pointer("ipc", address=t.data.device, handle=h.raw, data_size=size)
    raise ValueError(f"expected one of :local, :ipc, got: {mode!r}")


def from_pointer(pointer, type, shape, device=None):
    """``Nx.from_pointer/5`` (exla/lib/exla/backend.ex:137-181): a tensor over memory someone else
    owns - a device address of this process, or an IPC handle exported by another one."""
    from .nx import Tensor
    type = T.normalize(type)
    shape = tuple(int(d) for d in shape)
    want = math.prod(shape) * T.itemsize(type)
    if pointer.data_size != want:
        raise ValueError(f"invalid pointer data_size for shape, expected: {want}, got: {pointer.data_size}")
    dev = _device_of(device)
    l = nif.lib()
    h = C.c_void_p()
    dims = nif.dims_array(shape)
    if pointer.kind == "local":
        nif.check(l.nxb200_buffer_from_pointer(dev, T.DTYPE_CODES[type], dims, len(shape), C.c_void_p(pointer.address), C.byref(h)))
    elif pointer.kind == "ipc":
        nif.check(l.nxb200_buffer_from_ipc(dev, T.DTYPE_CODES[type], dims, len(shape), pointer.handle, C.byref(h)))
    else:
        raise ValueError(f"unknown pointer kind {pointer.kind!r}")
    return Tensor(DeviceBuffer(h.value, dev), type, shape)


def backend_deallocate(t):
    """``backend_deallocate/1``: ``"ok"`` or ``"already_deallocated"``
    (exla/lib/exla/backend.ex:81-83)."""
    if not isinstance(t.data, DeviceBuffer):
        return "ok"
    st = nif.lib().nxb200_buffer_deallocate(t.data.handle)
    if st == nif.ERR_DEALLOCATED:
        return "already_deallocated"
    nif.check(st)
    return "ok"


def to_binary(t, n_elems):
    """``to_binary/2`` (exla/lib/exla/backend.ex:222-226 -> read_device_mem)."""
    nbytes = n_elems * T.itemsize(t.type)
    buf = C.create_string_buffer(nbytes) if nbytes else C.create_string_buffer(1)
    nif.check(nif.lib().nxb200_buffer_to_host(t.data.handle, buf, nbytes))
    return buf.raw[:nbytes]


# ---- compute callbacks: one-node programs ---------------------------------------------

def to_expr(o):
    """Operand of a traced call -> expression tensor.  Host tensors captured by
    a traced function become literal nodes (nx/lib/nx/defn/expr.ex:1352-1357);
    scalars become constants."""
    from .nx import HostData, to_binary, to_numpy
    if isinstance(o.data, E.Expr):
        return o
    if o.shape == ():
        return E.constant(o.type, (), to_numpy(o).item())
    raw = o.data.raw if isinstance(o.data, HostData) else to_binary(o, o.size)
    return E.tensor_literal(o.type, o.shape, raw)


_eager_cache = {}
_eager_lock = threading.Lock()


def eager(builder, operands):
    """Run ``builder`` as a program whose parameters are the non-constant
    operands (exla/lib/exla/backend.ex:427-431)."""
    from . import defn
    from .nx import HostData
    params, args = [], []
    for o in operands:
        if isinstance(o.data, E.Expr):
            params.append(o)                       # a number: stays a constant node
        else:
            if isinstance(o.data, HostData):
                o = backend_transfer(o)
            params.append(E.parameter(o.type, o.shape, len(args)))
            args.append(o)
    with trace_scope():
        out = builder(*params)
    if not isinstance(out.data, E.Expr):           # builder returned an operand unchanged
        return out
    if out.data.op == "parameter":
        return args[out.data.ints[0]]
    blob = E.serialize([out])
    with _eager_lock:
        prog = _eager_cache.get(blob)
        if prog is None:
            prog = defn.Program(blob)
            _eager_cache[blob] = prog
    device = args[0].data.device if args else _device_of()
    return prog.run(args, device)[0]
