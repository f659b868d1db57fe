"""The slice of the ``Nx`` public API that sits above the hot path.

Every function does what nx/lib/nx.ex does before it reaches a backend: infer
the output type and shape, then hand ``(out_template, operands…)`` to the
implementation that owns the operands (nx/lib/nx/shared.ex:449-473):

* while a function is being traced (`nx_b200.defn`), operands are expression
  nodes and the call appends a node to the graph (``Nx.Defn.Expr``);
* otherwise operands live on a B200 (`nx_b200.backend.Backend`) and the call
  runs as a one-node program, the way EXLA.Backend runs eager ops
  (exla/lib/exla/backend.ex:409-431).

There is no host implementation of any operation: a tensor that is still in
host memory is storage only (the analogue of handing an ``Nx.BinaryBackend``
tensor to another backend, which transfers it).
"""
from __future__ import annotations

import builtins as _b
import math

import numpy as np

from . import expr as E
from . import types as T


class Tensor:
    """``%Nx.Tensor{data, type, shape}`` (nx/lib/nx/tensor.ex:41-42).  ``data``
    is an `expr.Expr` node, a `backend.DeviceBuffer`, or a `HostData`."""
    __slots__ = ("data", "type", "shape", "donatable")

    def __init__(self, data, type, shape, donatable=False):
        self.data, self.type, self.shape = data, type, tuple(int(d) for d in shape)
        self.donatable = donatable      # %Nx.Tensor{donatable?: ...} (nx/lib/nx/tensor.ex:41-42)

    @property
    def rank(self):
        return len(self.shape)

    @property
    def size(self):
        return math.prod(self.shape)

    def __repr__(self):
        dims = "".join(f"[{d}]" for d in self.shape)
        return f"#Nx.Tensor<{T.short(self.type)}{dims} {self.data!r}>"

    # the operators `defn` rewrites to Nx calls (nx/lib/nx/defn/kernel.ex)
    def __add__(self, o): return add(self, o)
    def __radd__(self, o): return add(o, self)
    def __sub__(self, o): return subtract(self, o)
    def __rsub__(self, o): return subtract(o, self)
    def __mul__(self, o): return multiply(self, o)
    def __rmul__(self, o): return multiply(o, self)
    def __truediv__(self, o): return divide(self, o)
    def __rtruediv__(self, o): return divide(o, self)
    def __neg__(self): return negate(self)
    def __pow__(self, o): return pow(self, o)
    def __gt__(self, o): return greater(self, o)
    def __ge__(self, o): return greater_equal(self, o)
    def __lt__(self, o): return less(self, o)
    def __le__(self, o): return less_equal(self, o)


class HostData:
    """Row-major little-endian bytes in host memory: what a tensor is before
    `backend_transfer` (the storage half of Nx.BinaryBackend)."""
    __slots__ = ("raw",)

    def __init__(self, raw):
        self.raw = bytes(raw)

    def __repr__(self):
        return f"host<{len(self.raw)} bytes>"


# ---- numpy <-> raw bytes (bf16 has no numpy dtype: it travels as uint16) ---------

_NP = {T.U8: np.uint8, T.U16: np.uint16, T.U32: np.uint32, T.U64: np.uint64,
       T.S8: np.int8, T.S16: np.int16, T.S32: np.int32, T.S64: np.int64,
       T.F16: np.float16, T.F32: np.float32, T.F64: np.float64, T.BF16: np.uint16}


def f32_to_bf16_bits(a):
    """Round-to-nearest-even f32 -> bf16 bit pattern (NaN stays NaN)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    rounded = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(a)
    if nan.any():
        rounded = np.where(nan, ((u >> np.uint32(16)) | np.uint32(0x40)).astype(np.uint16), rounded)
    return rounded


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def tensor(value, type=None):
    """``Nx.tensor/2``: build a tensor from a number, nested list or ndarray.
    With a default backend configured the data goes straight to the device
    (nx/lib/nx.ex:5006-5049)."""
    if isinstance(value, Tensor):
        return value if type is None else as_type(value, type)
    arr = np.asarray(value)
    if type is None:
        if arr.dtype.kind == "f":
            type = T.F32 if arr.dtype != np.float64 or not isinstance(value, np.ndarray) else T.F64
        elif arr.dtype.kind == "b":
            type = T.U8
        elif arr.dtype.kind in "iu" and isinstance(value, np.ndarray):
            type = {v: k for k, v in _NP.items() if k != T.BF16}[arr.dtype.type]
        else:
            type = T.S32
    type = T.normalize(type)
    if type == T.BF16:
        raw = f32_to_bf16_bits(arr.astype(np.float32)).tobytes()
    else:
        with np.errstate(invalid="ignore"):
            raw = np.ascontiguousarray(arr).astype(_NP[type]).tobytes()
    return from_binary(raw, type, arr.shape)


def donatable(t):
    """``Nx.donatable/1`` (nx/lib/nx.ex:1064-1068): marks a tensor (or every tensor of a tuple /
    list / dict) as one whose buffer a compiled function may take over for a result of the same
    type and shape.  The mark applies to that argument only; results are never donatable."""
    if isinstance(t, (tuple, list)):
        return type(t)(donatable(x) for x in t)
    if isinstance(t, dict):
        return {k: donatable(v) for k, v in t.items()}
    t = tensor(t)
    return Tensor(t.data, t.type, t.shape, donatable=True)


def is_donatable(t):
    """``Nx.donatable?/1``."""
    return bool(getattr(t, "donatable", False))


def from_binary(raw, type, shape=None):
    """``Nx.from_binary/3`` followed by placement on the default backend."""
    type = T.normalize(type)
    if shape is None:
        shape = (len(raw) // T.itemsize(type),)
    t = Tensor(HostData(raw), type, shape)
    if t.size * T.itemsize(type) != len(raw):
        raise ValueError(f"binary has {len(raw)} bytes, expected {t.size * T.itemsize(type)} "
                         f"for {T.short(type)}{list(t.shape)}")
    from . import backend
    if backend.default_backend() is not None:
        return backend.backend_transfer(t)
    return t


def to_binary(t, limit=None):
    """``Nx.to_binary/2`` (nx/lib/nx/backend.ex:56; EXLA: backend.ex:222-226)."""
    from . import backend
    n = t.size if limit is None else _b.min(int(limit), t.size)
    if isinstance(t.data, HostData):
        return t.data.raw[: n * T.itemsize(t.type)]
    if isinstance(t.data, E.Expr):
        raise TypeError("cannot read the value of a tensor inside defn")
    return backend.to_binary(t, n)


def to_numpy(t):
    """Convenience over `to_binary`: bf16 comes back widened to float32."""
    raw = to_binary(t)
    a = np.frombuffer(raw, dtype=_NP[t.type]).reshape(t.shape)
    return bf16_bits_to_f32(a).reshape(t.shape) if t.type == T.BF16 else a.copy()


def to_number(t):
    return to_numpy(t).reshape(()).item()


# ---- dispatch ----------------------------------------------------------------------

def _is_expr(x):
    return isinstance(x, Tensor) and isinstance(x.data, E.Expr)


def _as_operand(x):
    """Numbers become constant nodes typed by Nx.Type.infer (nx/lib/nx.ex to_tensor)."""
    if isinstance(x, Tensor):
        return x
    if isinstance(x, (bool, int, float, np.integer, np.floating)):
        x = x.item() if isinstance(x, np.generic) else x
        return E.constant(T.infer(x), (), x)
    return tensor(x)


def _dispatch(builder, operands):
    """Run ``builder(*operands)`` against the graph (tracing) or as a one-node
    program on the device (eager)."""
    from . import backend
    operands = [_as_operand(o) for o in operands]
    if _b.any(_is_expr(o) and o.data.op != "constant" for o in operands):
        return builder(*[backend.to_expr(o) for o in operands])
    if _b.all(_is_expr(o) for o in operands) and operands:
        return builder(*operands)          # constants only: folds at trace time
    if backend.tracing():
        # inside a traced function every operation is a graph node, also on tensors the function
        # captured from the host (they become literal nodes, nx/lib/nx/defn/expr.ex:1352-1357)
        return builder(*[backend.to_expr(o) for o in operands])
    return backend.eager(builder, operands)


def _out(type, shape):
    return Tensor(None, type, shape)


def _type_of(x):
    return x.type if isinstance(x, Tensor) else None


def _binary_type(a, b):
    """nx/lib/nx/shared.ex:383-388."""
    na, nb = not isinstance(a, Tensor), not isinstance(b, Tensor)
    if na and nb:
        return T.infer(a + b)
    if na:
        return T.merge_number(b.type, a)
    if nb:
        return T.merge_number(a.type, b)
    return T.merge(a.type, b.type)


def _num(x):
    if isinstance(x, np.generic):
        return x.item()
    if isinstance(x, (list, tuple, np.ndarray)):
        return tensor(x)
    return x


def _shape_of(x):
    return x.shape if isinstance(x, Tensor) else ()


def binary_broadcast(s1, s2):
    """nx/lib/nx/shape.ex binary_broadcast: right-aligned, size-1 stretches."""
    r = _b.max(len(s1), len(s2))
    a = (1,) * (r - len(s1)) + tuple(s1)
    b = (1,) * (r - len(s2)) + tuple(s2)
    out = []
    for x, y in zip(a, b):
        if x == y or y == 1:
            out.append(x)
        elif x == 1:
            out.append(y)
        else:
            raise ValueError(f"cannot broadcast tensor of dimensions {tuple(s1)} to {tuple(s2)}")
    return tuple(out)


def _bin(op, a, b, type_fun=lambda t: t, pred=False):
    a, b = _num(a), _num(b)
    type = T.U8 if pred else type_fun(_binary_type(a, b))
    shape = binary_broadcast(_shape_of(a), _shape_of(b))
    out = _out(type, shape)
    special = {"add": E.add, "multiply": E.multiply, "subtract": E.subtract, "divide": E.divide}
    if op in special:
        return _dispatch(lambda x, y: special[op](out, x, y), [a, b])
    return _dispatch(lambda x, y: E.binary_expr(out, op, x, y), [a, b])


def add(a, b): return _bin("add", a, b)
def subtract(a, b): return _bin("subtract", a, b)
def multiply(a, b): return _bin("multiply", a, b)
def divide(a, b): return _bin("divide", a, b, T.to_floating)
def pow(a, b): return _bin("pow", a, b)
def remainder(a, b): return _bin("remainder", a, b)
def atan2(a, b): return _bin("atan2", a, b, T.to_floating)
def min(a, b): return _bin("min", a, b)
def max(a, b): return _bin("max", a, b)


def _int_only(name, *xs):
    for x in xs:
        t = _type_of(x)
        if (t is not None and not T.is_integer(t)) or isinstance(x, float):
            raise ValueError(f"{name} expects integer tensors as inputs and outputs an integer tensor, "
                             f"got: {t}")


def quotient(a, b):
    _int_only("quotient", a, b)
    return _bin("quotient", a, b)


def bitwise_and(a, b): _int_only("bitwise_and", a, b); return _bin("bitwise_and", a, b)
def bitwise_or(a, b): _int_only("bitwise_or", a, b); return _bin("bitwise_or", a, b)
def bitwise_xor(a, b): _int_only("bitwise_xor", a, b); return _bin("bitwise_xor", a, b)
def left_shift(a, b): _int_only("left_shift", a, b); return _bin("left_shift", a, b)
def right_shift(a, b): _int_only("right_shift", a, b); return _bin("right_shift", a, b)

def equal(a, b): return _bin("equal", a, b, pred=True)
def not_equal(a, b): return _bin("not_equal", a, b, pred=True)
def greater(a, b): return _bin("greater", a, b, pred=True)
def less(a, b): return _bin("less", a, b, pred=True)
def greater_equal(a, b): return _bin("greater_equal", a, b, pred=True)
def less_equal(a, b): return _bin("less_equal", a, b, pred=True)
def logical_and(a, b): return _bin("logical_and", a, b, pred=True)
def logical_or(a, b): return _bin("logical_or", a, b, pred=True)
def logical_xor(a, b): return _bin("logical_xor", a, b, pred=True)


def _unary(op, x, type_fun):
    x = _as_operand(_num(x))
    out = _out(type_fun(x.type), x.shape)
    return _dispatch(lambda a: E.unary_expr(out, op, a), [x])


def _make_math(op):
    def f(x):
        return _unary(op, x, T.to_floating)      # nx/lib/nx.ex:8592-8598
    f.__name__ = op
    f.__doc__ = f"Element-wise {op} (nx/lib/nx/shared.ex:311-376)."
    return f


for _op in E.UNARY_MATH:
    globals()[_op] = _make_math(_op)


def negate(x): return _unary("negate", x, lambda t: t)
def abs(x): return _unary("abs", x, lambda t: t)
def sign(x): return _unary("sign", x, lambda t: t)
def is_nan(x): return _unary("is_nan", x, lambda t: T.U8)
def is_infinity(x): return _unary("is_infinity", x, lambda t: T.U8)


def _round_like(op, x):
    x = _as_operand(_num(x))
    return x if T.is_integer(x.type) else _unary(op, x, lambda t: t)


def floor(x): return _round_like("floor", x)
def ceil(x): return _round_like("ceil", x)
def round(x): return _round_like("round", x)


def bitwise_not(x):
    _int_only("bitwise_not", x)
    return _unary("bitwise_not", x, lambda t: t)


def population_count(x):
    _int_only("population_count", x)
    return _unary("population_count", x, lambda t: t)


def count_leading_zeros(x):
    _int_only("count_leading_zeros", x)
    return _unary("count_leading_zeros", x, lambda t: t)


def logical_not(x):
    """nx/lib/nx.ex logical_not: ``equal(x, 0)``."""
    return equal(x, 0)


def as_type(x, type):
    """nx/lib/nx.ex as_type -> backend.ex:68."""
    type = T.normalize(type)
    x = _as_operand(_num(x))
    if x.type == type:
        return x
    c = E.maybe_constant(x) if _is_expr(x) else None
    if c is not None:
        if T.is_integer(type) and isinstance(c, float):
            c = 0 if math.isnan(c) else (T.max_value(type) if c == math.inf else
                                         T.min_value(type) if c == -math.inf else int(c))
        return E.constant(type, x.shape, c)
    out = _out(type, x.shape)
    return _dispatch(lambda a: E.node(out, "as_type", [a]), [x])


def select(pred, on_true, on_false):
    """nx/lib/nx.ex:7782-7830."""
    type = _binary_type(_num(on_true), _num(on_false))
    pred, on_true, on_false = (_as_operand(_num(v)) for v in (pred, on_true, on_false))
    shape = binary_broadcast(on_true.shape, on_false.shape) if pred.shape == () else pred.shape
    for v in (on_true, on_false):
        if binary_broadcast(v.shape, shape) != shape:
            raise ValueError(f"cannot broadcast tensor of dimensions {v.shape} to {shape}")
    out = _out(type, shape)
    return _dispatch(lambda p, a, b: E.node(out, "select", [p, a, b]), [pred, on_true, on_false])


def clip(x, lo, hi):
    x, lo, hi = (_as_operand(_num(v)) for v in (x, lo, hi))
    if lo.shape != () or hi.shape != ():
        raise ValueError("min/max of clip must be scalars")
    out = _out(T.merge(T.merge(x.type, lo.type), hi.type), x.shape)
    return _dispatch(lambda a, b, c: E.node(out, "clip", [a, b, c]), [x, lo, hi])


# ---- shape operations --------------------------------------------------------------

def _norm_axis(rank, axis):
    a = axis + rank if axis < 0 else axis
    if not 0 <= a < rank:
        raise ValueError(f"given axis ({axis}) invalid for shape with rank {rank}")
    return a


def _norm_axes(rank, axes):
    out = [_norm_axis(rank, a) for a in axes]
    if len(set(out)) != len(out):
        raise ValueError(f"axes {list(axes)} must be unique integers between 0 and {rank - 1}")
    return out


def reshape(x, shape):
    x = _as_operand(x)
    shape = list(shape)
    if shape.count("auto") + shape.count(-1) == 1:
        i = shape.index("auto") if "auto" in shape else shape.index(-1)
        rest = math.prod(d for j, d in enumerate(shape) if j != i)
        shape[i] = x.size // rest if rest else 0
    shape = tuple(shape)
    if math.prod(shape) != x.size:
        raise ValueError(f"cannot reshape, current shape {x.shape} is not compatible with new shape {shape}")
    if shape == x.shape:
        return x
    out = _out(x.type, shape)
    return _dispatch(lambda a: E.node(out, "reshape", [a]), [x])


def squeeze(x, axes=None):
    x = _as_operand(x)
    if axes is None:
        axes = [i for i, d in enumerate(x.shape) if d == 1]
    axes = sorted(_norm_axes(x.rank, axes))
    for a in axes:
        if x.shape[a] != 1:
            raise ValueError(f"cannot squeeze dimensions whose sizes are not 1, got {x.shape[a]} for dimension {a}")
    if not axes:
        return x
    out = _out(x.type, tuple(d for i, d in enumerate(x.shape) if i not in axes))
    if _is_expr(x) and x.data.op == "squeeze":      # expr.ex:1092-1103 merges nested squeezes
        inner = x.data.args[0]
        inner_axes = x.data.ints[1:]
        kept = [i for i in range(inner.rank) if i not in inner_axes]
        merged = sorted(inner_axes + [kept[a] for a in axes])
        return E.node(out, "squeeze", [inner], ints=[len(merged)] + merged)
    return _dispatch(lambda a: E.node(out, "squeeze", [a], ints=[len(axes)] + axes), [x])


def new_axis(x, axis):
    x = _as_operand(x)
    a = axis + x.rank + 1 if axis < 0 else axis
    return reshape(x, x.shape[:a] + (1,) + x.shape[a:])


def broadcast(x, shape, axes=None):
    """``Nx.broadcast/3``: ``axes[i]`` is the output axis input axis i lands on;
    default is right alignment (nx/lib/nx/shape.ex broadcast_axes)."""
    x = _as_operand(_num(x))
    shape = tuple(shape)
    if axes is None:
        if x.shape == shape:
            return x
        axes = list(range(len(shape) - x.rank, len(shape)))
    axes = _norm_axes(len(shape), axes)
    if len(axes) != x.rank or _b.any(d != 1 and d != shape[a] for d, a in zip(x.shape, axes)):
        raise ValueError(f"cannot broadcast tensor of dimensions {x.shape} to {shape} with axes {axes}")
    if sorted(axes) != axes:
        raise ValueError("broadcast axes must be ordered")
    out = _out(x.type, shape)
    c = E.maybe_constant(x) if _is_expr(x) else None
    if c is not None:
        return E.constant(x.type, shape, c)
    return _dispatch(lambda a: E.node(out, "broadcast", [a], ints=[len(axes)] + axes), [x])


def transpose(x, axes=None):
    x = _as_operand(x)
    axes = list(range(x.rank))[::-1] if axes is None else _norm_axes(x.rank, axes)
    if len(axes) != x.rank:
        raise ValueError(f"expected length of permutation ({len(axes)}) to match rank of shape ({x.rank})")
    if axes == list(range(x.rank)):
        return x
    out = _out(x.type, tuple(x.shape[a] for a in axes))
    return _dispatch(lambda a: E.node(out, "transpose", [a], ints=axes), [x])


def _index_scalar(v):
    """A start index given as a tensor: must be an integer scalar."""
    v = _as_operand(v)
    if v.shape != () or not T.is_integer(v.type):
        raise ValueError(f"index must be an integer scalar tensor, got {v.type} {v.shape}")
    return v


def slice(x, starts, lengths, strides=None):
    """``Nx.slice/4`` (nx/lib/nx.ex slice).  Start indices may be integers or
    scalar integer tensors; either way a start is clamped so that the slice
    fits (``Nx.Shape.slice`` for static starts, the backend for dynamic ones)."""
    x = _as_operand(x)
    strides = [1] * x.rank if strides is None else ([strides] * x.rank if isinstance(strides, int) else list(strides))
    starts, lengths = list(starts), list(lengths)
    if not (len(starts) == len(lengths) == len(strides) == x.rank):
        raise ValueError("slice arguments must have one entry per axis")
    shape = []
    for d, l, st in zip(x.shape, lengths, strides):
        if l < 1 or l > d or st < 1:
            raise ValueError(f"length at axis must be in 1..{d} and strides positive, got length {l} stride {st}")
        shape.append(-(-l // st))
    if _b.any(isinstance(s, Tensor) for s in starts):
        dyn = [_index_scalar(s if isinstance(s, Tensor) else tensor(s, "s64")) for s in starts]
        out = _out(x.type, shape)
        return _dispatch(lambda a, *ss: E.node(out, "slice", [a, *ss], ints=[0] * x.rank + lengths + strides), [x] + dyn)
    starts = [_b.min(_b.max(s, 0), d - l) for s, d, l in zip(starts, x.shape, lengths)]
    if tuple(shape) == x.shape:
        return x
    out = _out(x.type, shape)
    return _dispatch(lambda a: E.node(out, "slice", [a], ints=starts + lengths + strides), [x])


def put_slice(x, start_indices, piece):
    """``Nx.put_slice/3`` (nx/lib/nx.ex put_slice; backend.ex put_slice): `x` with
    `piece` written at `start_indices` (integers or scalar integer tensors), each start
    clamped so that the piece fits.  The result type merges both types."""
    x, piece = _as_operand(x), _as_operand(piece)
    starts = list(start_indices)
    if len(starts) != x.rank or piece.rank != x.rank:
        raise ValueError("put_slice needs one start index per axis and a slice of the same rank")
    for d, l in zip(x.shape, piece.shape):
        if l > d:
            raise ValueError(f"slice shape {piece.shape} must be less than or equal to tensor shape {x.shape}")
    dyn = [_index_scalar(s if isinstance(s, Tensor) else tensor(s, "s64")) for s in starts]
    out = _out(T.merge(x.type, piece.type), x.shape)
    return _dispatch(lambda a, p, *ss: E.node(out, "put_slice", [a, p, *ss]), [x, piece] + dyn)


def gather(x, indices, axes=None):
    """``Nx.gather/3`` (nx/lib/nx.ex:15160-15203, shape rule nx/lib/nx/shape.ex:1643-1661):
    the last axis of `indices` holds one coordinate per indexed axis (default: the
    leading ones); the result has the batch shape of `indices` followed by the axes of
    `x` that are not indexed.  Out-of-range coordinates are clamped, as the compiled
    (XLA) path does."""
    x, indices = _as_operand(x), _as_operand(indices)
    if indices.rank < 1:
        raise ValueError("expected indices rank to be at least 1, got: 0")
    if not T.is_integer(indices.type):
        raise ValueError(f"indices must be an integer tensor, got {indices.type}")
    depth = indices.shape[-1]
    if depth > x.rank:
        raise ValueError(f"expected the last indices dimension size ({depth}) to be less than or equal to the tensor rank ({x.rank})")
    axes = list(range(depth)) if axes is None else _norm_axes(x.rank, axes)
    if len(axes) != depth or sorted(set(axes)) != sorted(axes):
        raise ValueError(f"expected {depth} distinct axes, got {axes}")
    if axes != sorted(axes):
        raise ValueError(":axes must be an ordered list")
    shape = tuple(indices.shape[:-1]) + tuple(d for i, d in enumerate(x.shape) if i not in axes)
    out = _out(x.type, shape)
    return _dispatch(lambda a, i: E.node(out, "gather", [a, i], ints=list(axes)), [x, indices])


def _indexed_op(op, target, indices, updates, axes):
    """``Nx.indexed_add/4`` / ``Nx.indexed_put/4`` (nx/lib/nx.ex:8277,8466; shape rules
    nx/lib/nx/shape.ex:937-973): `indices` {n, i} names, per row, a position along the i indexed
    axes (default: the leading ones); `updates` {n, ...} holds the slice that lands there, starting
    at 0 along the other axes.  The result has the merged type of target and updates
    (both are converted first, exla/lib/exla/defn.ex:1829-1848).  Rows with a coordinate outside the
    target are dropped, as the compiled (XLA) path does."""
    type = _binary_type(target if isinstance(target, Tensor) else _num(target), updates if isinstance(updates, Tensor) else _num(updates))
    target, indices, updates = _as_operand(target), _as_operand(indices), _as_operand(updates)
    if not T.is_integer(indices.type):
        raise ValueError(f"indices must be an integer tensor, got type: {indices.type}")
    if indices.rank == 1:
        # one index row, one scalar update (nx/lib/nx.ex:8470-8475)
        if updates.rank != 0 or indices.shape[0] != target.rank:
            raise ValueError("a rank-1 index updates a single entry: it needs one coordinate per axis and a scalar update")
        indices, updates = reshape(indices, (1,) + indices.shape), reshape(updates, (1,))
    if indices.rank != 2:
        raise ValueError(f"indices must be a rank 1 or 2 tensor, got: {indices.rank}")
    n, depth = indices.shape
    if axes is None:
        axes = list(range(depth))
    else:
        axes = _norm_axes(target.rank, axes)
        if axes != sorted(axes) or len(set(axes)) != len(axes):
            raise ValueError(":axes must be an ordered list")
        if len(axes) != depth:
            raise ValueError(":axes must have the same number of elements as the last dimension of indices")
    if updates.shape[:1] != (n,):
        raise ValueError(f"expected the leading axis of indices ({indices.shape}) and leading axis of updates ({updates.shape}) to match")
    if updates.rank - 1 + depth != target.rank:
        raise ValueError(f"expected the rank of the input ({target.rank}) to be equal to the rank of the updates ({updates.rank}) "
                         f"plus the trailing axis of indices ({indices.shape}) minus one")
    rest = [a for a in range(target.rank) if a not in axes]
    for j, a in enumerate(rest):
        if updates.shape[1 + j] > target.shape[a]:
            raise ValueError(f"axis ({1 + j}) of updates ({updates.shape}) must be less than or equal to the axis ({a}) of {target.shape})")
    out = _out(type, target.shape)
    if target.type != type:
        target = as_type(target, type)
    if updates.type != type:
        updates = as_type(updates, type)
    # the kernel reads 32- or 64-bit signed coordinates
    want = T.S64 if indices.type in (T.S64, T.U64, T.U32) else T.S32
    if indices.type != want:
        indices = as_type(indices, want)
    return _dispatch(lambda t, i, u: E.node(out, op, [t, i, u], ints=list(axes)), [target, indices, updates])


def indexed_add(target, indices, updates, axes=None):
    """``Nx.indexed_add/4``: adds the slices of `updates` at the positions in `indices`; repeated
    positions accumulate."""
    return _indexed_op("indexed_add", target, indices, updates, axes)


def indexed_put(target, indices, updates, axes=None):
    """``Nx.indexed_put/4``: writes the slices of `updates` at the positions in `indices`.  With
    repeated positions the result is one of the written values (nx/lib/nx.ex:8452-8454)."""
    return _indexed_op("indexed_put", target, indices, updates, axes)


def take(x, indices, axis=0):
    """``Nx.take/3`` (nx/lib/nx.ex:14731-14816): gather along one axis; the axes of
    `indices` replace `axis` in the result."""
    x, indices = _as_operand(x), _as_operand(indices)
    if not T.is_integer(indices.type):
        raise ValueError(f"indices must be an integer tensor, got {indices.type}")
    a = _norm_axis(x.rank, axis)
    g = gather(x, reshape(indices, indices.shape + (1,)), axes=[a])       # indices axes ++ remaining axes of x
    k = indices.rank
    lead = list(range(k, k + a))
    perm = lead + list(range(k)) + list(range(k + a, g.rank))
    return transpose(g, perm)


def _window(op, x, window_dimensions, strides, padding, window_dilations):
    """nx/lib/nx.ex:11007-11051 (aggregate_window_op) with Nx.Shape.pool (nx/lib/nx/shape.ex:860-886)."""
    x = _as_operand(x)
    win = [int(w) for w in window_dimensions]
    r = x.rank
    if len(win) != r:
        raise ValueError(f"invalid window dimensions, rank of shape ({r}) does not match rank of window ({len(win)})")
    strides = [strides] * r if isinstance(strides, int) else [int(s) for s in strides]
    dil = [window_dilations] * r if isinstance(window_dilations, int) else [int(d) for d in window_dilations]
    if len(strides) != r or len(dil) != r:
        raise ValueError("invalid stride or dilation dimensions, rank must match the shape")
    if _b.any(d < 1 for d in dil):
        raise ValueError(f"dilation rates must be greater than or equal to 1 got {dil}")
    kern = [(w - 1) * d + 1 for w, d in zip(win, dil)]
    if padding == "valid":
        pads = [(0, 0)] * r
    elif padding == "same":
        pads = [((k - 1) // 2, (k - 1) - (k - 1) // 2) for k in kern]
    else:
        pads = [(int(lo), int(hi)) for lo, hi in padding]
        if len(pads) != r or _b.any(lo < 0 or hi < 0 for lo, hi in pads):
            raise ValueError("padding must be a list of non-negative {low, high} pairs, one per axis")
    shape = []
    for d, k, s, (lo, hi) in zip(x.shape, kern, strides, pads):
        n = (d + lo + hi - k) // s + 1
        if n <= 0:
            raise ValueError("window dimensions would result in empty tensor which is not currently supported in Nx")
        shape.append(n)
    out = _out(x.type, shape)
    ints = win + strides + [p[0] for p in pads] + [p[1] for p in pads] + dil
    return _dispatch(lambda a: E.node(out, op, [a], ints=ints), [x])


def window_sum(x, window_dimensions, strides=1, padding="valid", window_dilations=1):
    """``Nx.window_sum/3``."""
    return _window("window_sum", x, window_dimensions, strides, padding, window_dilations)


def window_max(x, window_dimensions, strides=1, padding="valid", window_dilations=1):
    """``Nx.window_max/3``: padding contributes the type's minimum (-inf for floats)."""
    return _window("window_max", x, window_dimensions, strides, padding, window_dilations)


def window_min(x, window_dimensions, strides=1, padding="valid", window_dilations=1):
    """``Nx.window_min/3``."""
    return _window("window_min", x, window_dimensions, strides, padding, window_dilations)


def window_product(x, window_dimensions, strides=1, padding="valid", window_dilations=1):
    """``Nx.window_product/3``."""
    return _window("window_product", x, window_dimensions, strides, padding, window_dilations)


def window_mean(x, window_dimensions, strides=1, padding="valid", window_dilations=1):
    """``Nx.window_mean/3``: the window sum over the window's element count."""
    s = window_sum(x, window_dimensions, strides, padding, window_dilations)
    return divide(s, math.prod(int(w) for w in window_dimensions))


def _to_last(x, axis):
    a = _norm_axis(x.rank, axis)
    perm = [i for i in range(x.rank) if i != a] + [a]
    inv = [0] * x.rank
    for i, p in enumerate(perm):
        inv[p] = i
    return (x if a == x.rank - 1 else transpose(x, perm)), (None if a == x.rank - 1 else inv)


def _direction(direction):
    if direction not in ("asc", "desc"):
        raise ValueError(f"unknown value for :direction, expected :asc or :desc, got: {direction!r}")
    return 1 if direction == "desc" else 0


def sort(x, axis=0, direction="asc"):
    """``Nx.sort/2`` (nx/lib/nx.ex:15600-15720): NaN sorts higher than any other value.  The kernel
    sorts the last axis; another axis is moved there and back."""
    x = _as_operand(x)
    if x.rank == 0:
        raise ValueError("cannot sort a scalar")
    desc = _direction(direction)
    t, inv = _to_last(x, axis)
    out = _out(t.type, t.shape)
    r = _dispatch(lambda a: E.node(out, "sort", [a], ints=[desc]), [t])
    return r if inv is None else transpose(r, inv)


def argsort(x, axis=0, direction="asc", stable=False, type="s32"):
    """``Nx.argsort/2`` (nx/lib/nx.ex:15949-15990).  The result is always the stable permutation
    (ties keep their order), which is also a valid answer when ``stable`` is false."""
    x = _as_operand(x)
    if x.rank == 0:
        raise ValueError("cannot sort a scalar")
    desc = _direction(direction)
    t, inv = _to_last(x, axis)
    out = _out(T.normalize(type), t.shape)
    r = _dispatch(lambda a: E.node(out, "argsort", [a], ints=[desc, 1 if stable else 0]), [t])
    return r if inv is None else transpose(r, inv)


def top_k(x, k=1):
    """``Nx.top_k/2`` (nx/lib/nx.ex top_k): the k largest entries along the last axis and their
    indices (the first k of the descending sort / argsort)."""
    x = _as_operand(x)
    if x.rank == 0 or not 1 <= k <= x.shape[-1]:
        raise ValueError(f"top_k input must have at least rank 1 and k must be in 1..{x.shape[-1] if x.rank else 0}")
    last = x.rank - 1
    n = x.shape[-1]
    if n > SORT_LIMIT:
        return _top_k_of_long_rows(x, k)
    values = slice_along_axis(sort(x, axis=last, direction="desc"), 0, k, axis=last)
    indices = slice_along_axis(argsort(x, axis=last, direction="desc"), 0, k, axis=last)
    return values, indices


# ---- cumulative operations (nx/lib/nx.ex:12044-12057) --------------------------------------------
# The reference's default is a recursive pairwise scan (nx.ex:12186-12286) whose every level reads the
# level before twice; generated inline that doubles the arithmetic per level.  Here a row is cut into
# blocks: inside a block a running window (window reductions pad with the operation's identity) gives the
# running value, a reduction gives each block's total, the totals are scanned the same way, and every
# block adds what came before it.  Integers give the reference's result exactly (they wrap alike);
# floats differ from it by the order of summation only.

_CUMULATIVE_BLOCK = 32
_CUMULATIVE = {"sum": ("window_sum", "sum", "add", lambda t: 0),
               "product": ("window_product", "product", "multiply", lambda t: 1),
               "max": ("window_max", "reduce_max", "max", lambda t: float("-inf") if T.is_float(t) else T.min_value(t)),
               "min": ("window_min", "reduce_min", "min", lambda t: float("inf") if T.is_float(t) else T.max_value(t))}


def _running(kind, x):
    """Running `kind` along the last axis."""
    window_op, reduce_op, combine, identity = _CUMULATIVE[kind]
    g = globals()
    n, lead = x.shape[-1], list(x.shape[:-1])
    ones = [1] * len(lead)
    if n <= 2 * _CUMULATIVE_BLOCK:
        return g[window_op](x, ones + [n], padding=[(0, 0)] * len(lead) + [(n - 1, 0)])
    w = _CUMULATIVE_BLOCK
    blocks = -(-n // w)
    fill = identity(x.type)
    padded = pad(x, fill, [(0, 0, 0)] * len(lead) + [(0, blocks * w - n, 0)])
    tiles = reshape(padded, tuple(lead + [blocks, w]))
    inside = g[window_op](tiles, ones + [1, w], padding=[(0, 0)] * (len(lead) + 1) + [(w - 1, 0)])
    totals = as_type(g[reduce_op](tiles, axes=[-1]), x.type)
    before = _running(kind, totals)                                    # inclusive over the blocks
    before = pad(slice_along_axis(before, 0, blocks - 1, axis=-1), fill, [(0, 0, 0)] * len(lead) + [(1, 0, 0)])
    whole = g[combine](inside, new_axis(before, -1))
    return slice_along_axis(reshape(whole, tuple(lead + [blocks * w])), 0, n, axis=-1)


def _cumulative(kind, x, axis, reverse_):
    x = _as_operand(x)
    if x.rank == 0:
        raise ValueError("cumulative operations need a tensor of rank 1 or more")
    t, inv = _to_last(x, axis)
    if reverse_:
        t = reverse(t, axes=[t.rank - 1])
    r = as_type(_running(kind, t), x.type)
    if reverse_:
        r = reverse(r, axes=[r.rank - 1])
    return r if inv is None else transpose(r, inv)


def cumulative_sum(x, axis=0, reverse=False):
    """``Nx.cumulative_sum/2`` (nx/lib/nx.ex:11742-11786): same type and shape as the input."""
    return _cumulative("sum", x, axis, reverse)


def cumulative_product(x, axis=0, reverse=False):
    """``Nx.cumulative_product/2`` (nx/lib/nx.ex:11819-11863)."""
    return _cumulative("product", x, axis, reverse)


def cumulative_min(x, axis=0, reverse=False):
    """``Nx.cumulative_min/2``."""
    return _cumulative("min", x, axis, reverse)


def cumulative_max(x, axis=0, reverse=False):
    """``Nx.cumulative_max/2``."""
    return _cumulative("max", x, axis, reverse)


# the row kernel of sort / argsort keeps a whole row in shared memory
SORT_LIMIT = 16384


def _top_k_of_long_rows(x, k):
    """top_k over rows longer than one sorted row may be (a vocabulary): every row is cut into equal
    chunks, each chunk gives its own k best, and the k best of those candidates are the answer.  The
    sorts are stable and the candidates stay in chunk order, so among equal values the lowest position
    wins, exactly as in the one-pass form.  Positions past the end of a row are filled with the lowest
    value of the type; they lie behind every real position and can never be among the first k."""
    n, last = x.shape[-1], x.rank - 1
    chunks = -(-n // SORT_LIMIT)
    width = -(-n // chunks)
    if k > width or chunks * k > SORT_LIMIT:
        raise ValueError(f"top_k over {n} entries supports k up to {min(width, SORT_LIMIT // chunks)}, got {k}")
    lowest = float("-inf") if T.is_float(x.type) else T.min_value(x.type)
    padded = pad(x, lowest, [(0, 0, 0)] * last + [(0, chunks * width - n, 0)])
    pieces = reshape(padded, x.shape[:-1] + (chunks, width))
    best = slice_along_axis(sort(pieces, axis=last + 1, direction="desc"), 0, k, axis=last + 1)
    where = slice_along_axis(argsort(pieces, axis=last + 1, direction="desc"), 0, k, axis=last + 1)
    where = where + iota(where.shape, axis=last, type="s32") * width            # position in the whole row
    best, where = (reshape(t, x.shape[:-1] + (chunks * k,)) for t in (best, where))
    order = slice_along_axis(argsort(best, axis=last, direction="desc"), 0, k, axis=last)
    return take_along_axis(best, order, axis=last), take_along_axis(where, order, axis=last)


def conv(x, kernel, strides=1, padding="valid", input_dilation=1, kernel_dilation=1, feature_group_size=1,
         batch_group_size=1, input_permutation=None, kernel_permutation=None, output_permutation=None):
    """``Nx.conv/3`` (nx/lib/nx.ex:13757-13860; shape rule nx/lib/nx/shape.ex conv): input {N, C, spatial…},
    kernel {Cout, C / groups, spatial…}, result {N, Cout, spatial…} in the floating type both merge to.

    Lowered to ops the compiler already has: the input is padded (interior padding is the input
    dilation), one strided slice per kernel position gives the patches, and a `dot` over (channel,
    kernel position) does the arithmetic - on the tensor cores for 16-bit types."""
    x, kernel = _as_operand(x), _as_operand(kernel)
    if x.rank < 3 or kernel.rank != x.rank:
        raise ValueError(f"input and kernel must have the same rank of at least 3, got {x.shape} and {kernel.shape}")
    if batch_group_size != 1:
        raise NotImplementedError("conv with batch_group_size > 1 is not implemented")
    type = T.to_floating(T.merge(x.type, kernel.type))
    nsp = x.rank - 2
    if input_permutation is not None:
        x = transpose(x, list(input_permutation))
    if kernel_permutation is not None:
        kernel = transpose(kernel, list(kernel_permutation))
    x, kernel = as_type(x, type), as_type(kernel, type)
    many = lambda v: [int(v)] * nsp if isinstance(v, int) else [int(i) for i in v]
    strides, idil, kdil = many(strides), many(input_dilation), many(kernel_dilation)
    n, c = x.shape[:2]
    cout, cin = kernel.shape[:2]
    ks = list(kernel.shape[2:])
    groups = int(feature_group_size)
    if c != cin * groups or cout % groups != 0:
        raise ValueError(f"size of input channels divided by feature groups must match size of kernel channels, got {c} / {groups} != {cin}")
    kd = [(k - 1) * d + 1 for k, d in zip(ks, kdil)]
    if padding == "valid":
        pads = [(0, 0)] * nsp
    elif padding == "same":
        pads = [((k - 1) // 2, (k - 1) - (k - 1) // 2) for k in kd]
    else:
        pads = [(int(lo), int(hi)) for lo, hi in padding]
        if len(pads) != nsp:
            raise ValueError("padding must have one {low, high} pair per spatial dimension")
    xp = pad(x, 0.0, [(0, 0, 0), (0, 0, 0)] + [(lo, hi, d - 1) for (lo, hi), d in zip(pads, idil)])
    xp = as_type(xp, type)
    osp = []
    for d, k, s in zip(xp.shape[2:], kd, strides):
        o = (d - k) // s + 1
        if o <= 0:
            raise ValueError("convolution would result in an empty tensor")
        osp.append(o)
    import itertools
    patches = []
    for pos in itertools.product(*[range(k) for k in ks]):
        starts = [0, 0] + [p * d for p, d in zip(pos, kdil)]
        lengths = [n, c] + [(o - 1) * s + 1 for o, s in zip(osp, strides)]
        patches.append(slice(xp, starts, lengths, [1, 1] + strides))
    kvol = len(patches)
    cols = stack(patches, axis=2)                                        # {N, C, K, spatial…}
    w = reshape(kernel, (cout, cin, kvol))
    outs = []
    cg = cout // groups
    for g in range(groups):
        xg = cols if groups == 1 else slice_along_axis(cols, g * cin, cin, axis=1)
        wg = w if groups == 1 else slice_along_axis(w, g * cg, cg, axis=0)
        outs.append(dot(xg, [1, 2], [], wg, [1, 2], []))                 # {N, spatial…, Cout / groups}
    y = outs[0] if groups == 1 else concatenate(outs, axis=nsp + 1)
    y = transpose(y, [0, nsp + 1] + list(range(1, nsp + 1)))             # {N, Cout, spatial…}
    if output_permutation is not None:
        perm = list(output_permutation)
        inv = [0] * len(perm)
        for i, p in enumerate(perm):
            inv[p] = i
        y = transpose(y, inv)
    return y


def pad(x, pad_value, padding_config):
    """``Nx.pad/3`` (nx/lib/nx.ex pad; shape rule nx/lib/nx/shape.ex:1038-1090): per axis
    ``(low, high, interior)``; negative edges crop."""
    x, pv = _as_operand(x), _as_operand(_num(pad_value))
    if pv.shape != ():
        raise ValueError("padding value must be a scalar")
    cfg = [tuple(int(v) for v in c) for c in padding_config]
    if len(cfg) != x.rank or _b.any(len(c) != 3 for c in cfg):
        raise ValueError("invalid padding configuration, rank of padding configuration and shape must match")
    shape = []
    for d, (lo, hi, it) in zip(x.shape, cfg):
        if it < 0:
            raise ValueError("interior padding must be non-negative")
        n = d + lo + hi + _b.max(d - 1, 0) * it
        if n < 0:
            raise ValueError("invalid padding widths, padding width can't be less than the dimension it pads")
        shape.append(n)
    out = _out(_binary_type(x, pv if not isinstance(pad_value, Tensor) else pad_value), shape)
    ints = [c[0] for c in cfg] + [c[1] for c in cfg] + [c[2] for c in cfg]
    if x.rank == 0:
        return as_type(x, out.type)
    return _dispatch(lambda a, v: E.node(out, "pad", [a, v], ints=ints), [x, pv])


def reverse(x, axes=None):
    """``Nx.reverse/2`` (nx/lib/nx.ex reverse): all axes by default."""
    x = _as_operand(x)
    axes = list(range(x.rank)) if axes is None else sorted(set(_norm_axes(x.rank, axes)))
    axes = [a for a in axes if x.shape[a] > 1]
    if not axes:
        return x
    out = _out(x.type, x.shape)
    return _dispatch(lambda a: E.node(out, "reverse", [a], ints=axes), [x])


def stack(tensors, axis=0):
    """``Nx.stack/2``: a new axis, then concatenate."""
    ts = [_as_operand(t) for t in tensors]
    a = axis if axis >= 0 else axis + ts[0].rank + 1
    return concatenate([reshape(t, t.shape[:a] + (1,) + t.shape[a:]) for t in ts], axis=a)


def new_axis(x, axis):
    """``Nx.new_axis/2``."""
    x = _as_operand(x)
    a = axis if axis >= 0 else axis + x.rank + 1
    return reshape(x, x.shape[:a] + (1,) + x.shape[a:])


def take_along_axis(x, indices, axis=0):
    """``Nx.take_along_axis/3`` (nx/lib/nx.ex take_along_axis): `indices` has the shape of `x`
    except along `axis`; lowered to `gather` over iotas like the reference does."""
    x, indices = _as_operand(x), _as_operand(indices)
    if not T.is_integer(indices.type):
        raise ValueError(f"indices must be an integer tensor, got {indices.type}")
    a = _norm_axis(x.rank, axis)
    if indices.rank != x.rank or _b.any(i != a and indices.shape[i] != x.shape[i] for i in range(x.rank)):
        raise ValueError(f"expected indices shape {indices.shape} to match tensor shape {x.shape} except along axis {a}")
    cols = [indices if i == a else as_type(iota(indices.shape, axis=i), indices.type) for i in range(x.rank)]
    full = concatenate([reshape(c, indices.shape + (1,)) for c in cols], axis=x.rank)
    return gather(x, full)


def slice_along_axis(x, start, length, axis=0, strides=1):
    x = _as_operand(x)
    a = _norm_axis(x.rank, axis)
    starts = [0] * x.rank
    lengths = list(x.shape)
    st = [1] * x.rank
    starts[a], lengths[a], st[a] = start, length, strides
    return slice(x, starts, lengths, st)


def concatenate(tensors, axis=0):
    tensors = [_as_operand(t) for t in tensors]
    a = _norm_axis(tensors[0].rank, axis)
    type = tensors[0].type
    for t in tensors[1:]:
        type = T.merge(type, t.type)
        if t.rank != tensors[0].rank or _b.any(i != a and d != e for i, (d, e) in enumerate(zip(t.shape, tensors[0].shape))):
            raise ValueError("expected all shapes to match except on the concatenation axis")
    if len(tensors) == 1:
        return as_type(tensors[0], type)
    shape = list(tensors[0].shape)
    shape[a] = _b.sum(t.shape[a] for t in tensors)
    out = _out(type, shape)
    from . import backend
    if backend.tracing() and _b.all(_is_expr(t) and t.data.id == tensors[0].data.id for t in tensors):
        # k copies of ONE traced value side by side (the angle table of a rotary embedding,
        # ``concatenate([freqs, freqs])``): a broadcast over a new axis folded into the concatenation
        # axis, i.e. index arithmetic inside whatever reads it, with no buffer and no kernel of its own
        x = tensors[0]
        k, n = len(tensors), x.shape[a]
        tiled = broadcast(reshape(x, x.shape[:a] + (1,) + x.shape[a:]), x.shape[:a] + (k,) + x.shape[a:])
        return as_type(reshape(tiled, tuple(shape)), type)
    if _rearranges_one_source(tensors):
        return _concatenate_by_selection(tensors, a, type, shape)
    return _dispatch(lambda *ts: E.node(out, "concatenate", list(ts), ints=[a]), tensors)


_POINTWISE_VIEWS = set(E.UNARY_MATH) | set(E.UNARY_OTHER) | {"as_type", "slice"}


def _rearranges_one_source(tensors):
    """True inside a traced function when every piece is a static slice of the same tensor, possibly under
    pointwise functions (the rotate-half of a rotary embedding: ``concatenate([-x2, x1])``).  Such a
    concatenation is an index selection on one source: it is traced as selects over padded pieces, which
    the compiler generates inside the consumer's kernel, instead of a node of its own whose pieces are
    written to memory first.  (Different whole tensors side by side stay a concatenate node.)"""
    from . import backend
    if not backend.tracing() or len(tensors) > 4 or not _b.all(_is_expr(t) for t in tensors):
        return False
    roots = set()
    for t in tensors:
        e, sliced = t.data, False
        while e.op in _POINTWISE_VIEWS and len(e.args) == 1:
            sliced = sliced or e.op == "slice"
            e = e.args[0].data
        if e.op == "constant" or not sliced:
            return False
        roots.add(e.id)
    return len(roots) == 1


def _concatenate_by_selection(tensors, a, type, shape):
    position = iota(shape, axis=a)
    total, offsets, off = shape[a], [], 0
    for t in tensors:
        offsets.append(off)
        off += t.shape[a]
    padded = []
    for t, o in zip(tensors, offsets):
        t = as_type(t, type) if t.type != type else t
        cfg = [(0, 0, 0)] * len(shape)
        cfg[a] = (o, total - o - t.shape[a], 0)
        padded.append(pad(t, 0, cfg))
    acc = padded[-1]
    for k in range(len(tensors) - 2, -1, -1):
        acc = select(less(position, offsets[k + 1]), padded[k], acc)
    return acc


def iota(shape, axis=None, type=T.S32):
    """``Nx.iota/2`` (nx/lib/nx.ex iota; backend.ex:51)."""
    shape = tuple(shape)
    type = T.normalize(type)
    a = -1 if axis is None else _norm_axis(len(shape), axis)
    out = _out(type, shape)
    from . import backend
    t = E.node(out, "iota", [], ints=[a])
    if backend.tracing():
        return t
    return backend.eager(lambda: E.node(out, "iota", [], ints=[a]), [])


def eye(shape, type=T.S32):
    """``Nx.eye/2`` (nx/lib/nx.ex:1262-1390): the identity on the last two axes of ``shape`` (an integer
    ``n`` means ``{n, n}``), repeated over the leading ones.  The reference's compilers lower it to
    ``iota(rows) == iota(columns)`` (exla/lib/exla/defn.ex:1126-1130); so does this front-end: it is index
    arithmetic inside whatever kernel reads it."""
    shape = (shape, shape) if isinstance(shape, int) else tuple(shape)
    if len(shape) < 2:
        raise ValueError(f"eye/2 expects a shape with at least 2 dimensions or an integer, got: {shape!r}")
    rank = len(shape)
    return as_type(equal(iota(shape, axis=rank - 2), iota(shape, axis=rank - 1)), type)


# ---- aggregates ---------------------------------------------------------------------



def _aggregate(op, x, type, axes, keep_axes):
    """nx/lib/nx.ex aggregate_axes_op (:9622-9660)."""
    x = _as_operand(x)
    if axes is not None:
        axes = sorted(_norm_axes(x.rank, axes))
        if axes == []:
            return as_type(x, type)
        shape = tuple((1 if i in axes else d) for i, d in enumerate(x.shape) if keep_axes or i not in axes)
    else:
        axes = list(range(x.rank))
        shape = (1,) * x.rank if keep_axes else ()
    out = _out(type, shape)
    ints = [int(bool(keep_axes)), len(axes)] + axes
    return _dispatch(lambda a: E.node(out, op, [a], ints=ints), [x])


def sum(x, axes=None, keep_axes=False):
    x = _as_operand(x)
    return _aggregate("sum", x, T.to_aggregate(x.type), axes, keep_axes)


def product(x, axes=None, keep_axes=False):
    x = _as_operand(x)
    return _aggregate("product", x, T.to_aggregate(x.type), axes, keep_axes)


def reduce_max(x, axes=None, keep_axes=False):
    x = _as_operand(x)
    return _aggregate("reduce_max", x, x.type, axes, keep_axes)


def reduce_min(x, axes=None, keep_axes=False):
    x = _as_operand(x)
    return _aggregate("reduce_min", x, x.type, axes, keep_axes)


def all(x, axes=None, keep_axes=False):
    return _aggregate("all", x, T.U8, axes, keep_axes)


def any(x, axes=None, keep_axes=False):
    return _aggregate("any", x, T.U8, axes, keep_axes)


def mean(x, axes=None, keep_axes=False):
    """nx/lib/nx.ex:9745-9756: ``sum / count``."""
    x = _as_operand(x)
    den = x.size if axes is None else math.prod(x.shape[a] for a in _norm_axes(x.rank, axes))
    return divide(sum(x, axes=axes, keep_axes=keep_axes), den)


def _arg_reduce(op, x, axis, keep_axis, tie_break, type):
    """nx/lib/nx.ex:10948-11006."""
    x = _as_operand(x)
    if tie_break not in ("low", "high"):
        raise ValueError(f"unknown value for :tie_break, expected :high or :low, got: {tie_break!r}")
    type = T.normalize(type)
    if axis is None:
        shape = (1,) * x.rank if keep_axis else ()
        a = -1
    else:
        a = _norm_axis(x.rank, axis)
        shape = tuple((1 if i == a else d) for i, d in enumerate(x.shape) if keep_axis or i != a)
    out = _out(type, shape)
    ints = [int(tie_break == "high"), a, int(bool(keep_axis))]
    return _dispatch(lambda t: E.node(out, op, [t], ints=ints), [x])


def argmax(x, axis=None, keep_axis=False, tie_break="low", type=T.S32):
    return _arg_reduce("argmax", x, axis, keep_axis, tie_break, type)


def argmin(x, axis=None, keep_axis=False, tie_break="low", type=T.S32):
    return _arg_reduce("argmin", x, axis, keep_axis, tie_break, type)


def logsumexp(x, axes=None, keep_axes=False, exp_scaling_factor=None):
    """nx/lib/nx.ex:18400-18433, node for node (minus the gradient-only
    ``stop_grad`` metadata wrapper, which is an identity for evaluation)."""
    x = _as_operand(x)
    mx = reduce_max(x, axes=axes, keep_axes=True)
    if _is_expr(mx):
        mx = E.node(mx, "metadata", [mx])
    mask = is_infinity(mx)
    mx = select(mask, E.constant(x.type, (), 0), mx)
    ex = exp(subtract(x, mx))
    if exp_scaling_factor is not None:
        ex = multiply(exp_scaling_factor, ex)
    if not keep_axes:
        ax = list(range(x.rank)) if axes is None else axes
        mx = squeeze(mx, axes=ax)
    return add(log(sum(ex, axes=axes, keep_axes=keep_axes)), mx)


# ---- dot ------------------------------------------------------------------------------

def dot(a, *args):
    """``Nx.dot/2``, ``dot/4`` and ``dot/6`` (nx/lib/nx.ex:12836-13161)."""
    if len(args) == 1:
        b = args[0]
        a, b = _as_operand(_num(a)), _as_operand(_num(b))
        if a.rank == 0 or b.rank == 0:
            return multiply(a, b)
        if b.rank == 1:
            return dot(a, [a.rank - 1], [], b, [0], [])
        if a.rank == 1:
            return dot(a, [0], [], b, [b.rank - 2], [])
        return dot(a, [a.rank - 1], [], b, [b.rank - 2], [])
    if len(args) == 3:
        c1, b, c2 = args
        return dot(a, c1, [], b, c2, [])
    c1, b1, b, c2, b2 = args
    a, b = _as_operand(_num(a)), _as_operand(_num(b))
    c1, b1 = _norm_axes(a.rank, c1), _norm_axes(a.rank, b1)
    c2, b2 = _norm_axes(b.rank, c2), _norm_axes(b.rank, b2)
    # nx/lib/nx/shape.ex:1801-1850
    if b1 and not b2:
        raise ValueError("right tensor must be batched if left tensor is batched")
    if b2 and not b1:
        raise ValueError("left tensor must be batched if right tensor is batched")
    if b1 != list(range(len(b1))):
        raise ValueError("invalid dot batch axis for the left tensor, batch axes must be successive "
                         f"dimensions starting from 0, got {b1}")
    if b2 != list(range(len(b2))):
        raise ValueError("invalid dot batch axis for the right tensor, batch axes must be successive "
                         f"dimensions starting from 0, got {b2}")
    if set(b1) & set(c1):
        raise ValueError(f"dot batch axes for left tensor ({b1}) cannot be in contract axes ({c1})")
    if set(b2) & set(c2):
        raise ValueError(f"dot batch axes for right tensor ({b2}) cannot be in contract axes ({c2})")
    if [a.shape[i] for i in c1] != [b.shape[i] for i in c2]:
        raise ValueError("dot/zip expects shapes to be compatible, dimensions "
                         f"{[a.shape[i] for i in c1]} of left do not match {[b.shape[i] for i in c2]} of right")
    if [a.shape[i] for i in b1] != [b.shape[i] for i in b2]:
        raise ValueError("dot batch dimensions must match")
    shape = tuple([a.shape[i] for i in b1]
                  + [d for i, d in enumerate(a.shape) if i not in c1 and i not in b1]
                  + [d for i, d in enumerate(b.shape) if i not in c2 and i not in b2])
    out = _out(T.merge(a.type, b.type), shape)
    ints = [len(c1)] + c1 + [len(b1)] + b1 + [len(c2)] + c2 + [len(b2)] + b2
    return _dispatch(lambda x, y: E.node(out, "dot", [x, y], ints=ints), [a, b])


def runtime_call(output, tensor_or_container, fun, opts=None):
    """``Nx.runtime_call/4`` (nx/lib/nx.ex:2394-2419); the graph cutting lives with the compiler mirror."""
    from . import defn
    return defn.runtime_call(output, tensor_or_container, fun, opts)
