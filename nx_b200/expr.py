"""The `defn` expression graph and its wire format.

Host-side mirror of ``Nx.Defn.Expr`` (nx/lib/nx/defn/expr.ex:17-60): a node is
``{id, op, args}`` attached to a tensor that carries the node's *result* type
and shape.  The same trace-time rewrites the reference applies are applied
here, so the graphs the compiler sees look like the ones an Elixir caller
produces: ``x + 0`` / ``x * 1`` folding, constant folding, constants commuted
to the left operand of add/multiply (expr.ex:889-962, :1597-1646) and float
constants retagged to the operation's output type (expr.ex:1648-1664).

``serialize`` flattens a DAG into the byte string `nxb200_program_build`
consumes (layout documented in include/nxb200.h).
"""
from __future__ import annotations

import itertools
import math
import struct

from . import types as T

_ids = itertools.count(1)

UNARY_MATH = ["exp", "expm1", "log", "log1p", "sigmoid", "cos", "sin", "tan", "cosh",
              "sinh", "tanh", "acos", "asin", "atan", "acosh", "asinh", "atanh",
              "sqrt", "rsqrt", "cbrt", "erf", "erfc", "erf_inv"]
UNARY_OTHER = ["abs", "bitwise_not", "ceil", "floor", "negate", "round", "sign",
               "count_leading_zeros", "population_count", "is_nan", "is_infinity"]
BINARY_ARITH = ["add", "subtract", "multiply", "divide", "pow", "remainder", "atan2",
                "min", "max", "quotient", "bitwise_and", "bitwise_or", "bitwise_xor",
                "left_shift", "right_shift"]
BINARY_PRED = ["equal", "not_equal", "greater", "less", "greater_equal", "less_equal",
               "logical_and", "logical_or", "logical_xor"]
AGGREGATES = ["sum", "product", "reduce_max", "reduce_min", "all", "any"]


class Expr:
    """One node of the graph (expr.ex:59-60)."""
    __slots__ = ("id", "op", "args", "ints", "flts", "blob", "payload")

    def __init__(self, op, args=(), ints=(), flts=(), blob=b"", id=None, payload=None):
        self.id = next(_ids) if id is None else id
        self.payload = payload      # host-side attachment of control-flow nodes (never serialised)
        self.op = op
        self.args = list(args)      # Tensor operands (each with .data an Expr)
        self.ints = [int(i) for i in ints]
        self.flts = [float(f) for f in flts]
        self.blob = blob

    def __repr__(self):
        return f"Expr<{self.op}#{self.id}>"


def watermark():
    """An id larger than every node created so far (nodes made later have larger ids)."""
    return next(_ids)


def substitute(outputs, repl):
    """Copy of the DAG under ``outputs`` with the nodes whose id is in ``repl`` replaced by the given
    tensors (sub-graphs that contain none of them are shared, not copied)."""
    from .nx import Tensor
    memo = {}

    def go(t):
        e = t.data
        if e.id in repl:
            return repl[e.id]
        if e.id in memo:
            return memo[e.id]
        new_args = [go(a) for a in e.args]
        if all(n is a for n, a in zip(new_args, e.args)):
            r = t
        else:
            r = Tensor(Expr(e.op, new_args, e.ints, e.flts, e.blob, payload=e.payload), t.type, t.shape)
        memo[e.id] = r
        return r
    return [go(o) for o in outputs]


def _tensor(data, type, shape):
    from .nx import Tensor
    return Tensor(data, type, tuple(shape))


def parameter(type, shape, index):
    """expr.ex:72-90."""
    return _tensor(Expr("parameter", ints=[index]), type, shape)


def constant(type, shape, number):
    """expr.ex:1553-1576: the id of a constant is its value, so equal constants
    are the same node."""
    if T.is_float(type):
        number = float(number)
    elif not isinstance(number, int):
        if isinstance(number, float) and number == int(number) and math.isfinite(number):
            number = int(number)
        else:
            raise ValueError(f"value {number!r} is not valid for constant of type {type}")
    ints, flts = ((), (number,)) if T.is_float(type) else ((number,), ())
    key = ("c", repr(number), type, tuple(shape))
    return _tensor(Expr("constant", ints=ints, flts=flts, id=key), type, shape)


def tensor_literal(type, shape, raw_bytes):
    """expr.ex:1352-1357: a host tensor captured by the traced function."""
    return _tensor(Expr("tensor", blob=bytes(raw_bytes)), type, shape)


def maybe_constant(t):
    e = t.data
    if isinstance(e, Expr) and e.op == "constant":
        return e.flts[0] if e.flts else e.ints[0]
    return None


def node(out, op, args, ints=(), flts=()):
    return _tensor(Expr(op, args, ints, flts), out.type, out.shape)


# ---- constant folding helpers -------------------------------------------------

def _fold_scalar(op, type, *vals):
    """Evaluate ``op`` on python numbers the way the reference folds constants
    through Nx.BinaryBackend (expr.ex:1617-1626, :1666-1674): f64 math, one
    rounding into ``type``."""
    import numpy as np
    with np.errstate(all="ignore"):
        a = vals[0]
        b = vals[1] if len(vals) > 1 else None
        f = {
            "add": lambda: a + b, "subtract": lambda: a - b, "multiply": lambda: a * b,
            "divide": lambda: np.float64(a) / np.float64(b),
            "max": lambda: max(a, b), "min": lambda: min(a, b),
            "pow": lambda: (a ** b) if T.is_integer(type) else float(np.power(np.float64(a), np.float64(b))),
            "negate": lambda: -a, "abs": lambda: abs(a),
            "exp": lambda: float(np.exp(np.float64(a))), "log": lambda: float(np.log(np.float64(a))),
            "sqrt": lambda: float(np.sqrt(np.float64(a))),
            "rsqrt": lambda: float(1.0 / np.sqrt(np.float64(a))),
            "tanh": lambda: float(np.tanh(np.float64(a))),
            "sigmoid": lambda: float(1.0 / (1.0 + np.exp(-np.float64(a)))),
            "cos": lambda: float(np.cos(np.float64(a))), "sin": lambda: float(np.sin(np.float64(a))),
        }.get(op)
        if f is None:
            return None
        v = f()
    if T.is_float(type):
        v = float(v)
        if type == T.F32:
            v = float(np.float32(v))
        elif type == T.BF16:
            bits = np.float32(v).view(np.uint32) & np.uint32(0xFFFF0000)
            v = float(bits.view(np.float32))
        elif type == T.F16:
            v = float(np.float16(v))
    else:
        v = int(v)
    return v


def _retag_float_constant(arg, out_type):
    """expr.ex:1648-1664."""
    c = maybe_constant(arg)
    if c is not None and T.is_float(arg.type) and T.is_float(out_type) and arg.type != out_type:
        return constant(out_type, arg.shape, c)
    return arg


def ensure_compatible(t, out):
    """expr.ex:1591-1596."""
    from . import nx
    t = nx.as_type(t, out.type)
    if t.shape != out.shape:
        t = nx.broadcast(t, out.shape)
    return t


def binary_expr(out, op, a, b):
    """expr.ex:1614-1639."""
    c1, c2 = maybe_constant(a), maybe_constant(b)
    if c1 is not None and c2 is not None:
        v = _fold_scalar(op, out.type, c1, c2)
        if v is not None:
            return constant(out.type, out.shape, v)
    if c1 is not None:
        a = _retag_float_constant(a, out.type)
    if c2 is not None:
        b = _retag_float_constant(b, out.type)
    return node(out, op, [a, b])


def unary_expr(out, op, a):
    """expr.ex:1666-1674."""
    c = maybe_constant(a)
    if c is not None:
        v = _fold_scalar(op, out.type, c)
        if v is not None:
            return constant(out.type, out.shape, v)
    return node(out, op, [a])


def _commute(out, op, s1, t1, t2):
    """expr.ex:1597-1612: put the constant on the left, merging nested
    constants of the same commutative op."""
    from . import nx
    fold = (lambda x, y: x + y) if op == "add" else (lambda x, y: x * y)

    def const_lhs_of(t):
        e = t.data
        if isinstance(e, Expr) and e.op == op:
            return maybe_constant(e.args[0]), e.args[1]
        return None, None

    s2, t3 = const_lhs_of(t2)
    scalar_out = _tensor(None, out.type, ())
    if s2 is not None:
        if s1 is not None:
            a1 = constant(scalar_out.type, (), _fold_scalar(op, out.type, s1, s2))
            a2 = nx.broadcast(t3, out.shape) if t3.shape != out.shape else t3
        else:
            a1 = constant(scalar_out.type, (), s2)
            inner = getattr(nx, op)(t1, t3)
            a2 = nx.broadcast(inner, out.shape) if inner.shape != out.shape else inner
        return binary_expr(out, op, a1, a2)
    s1b, t3b = const_lhs_of(t1)
    if s1b is not None and s1 is None:
        a1 = constant(scalar_out.type, (), s1b)
        inner = getattr(nx, op)(t2, t3b)
        a2 = nx.broadcast(inner, out.shape) if inner.shape != out.shape else inner
        return binary_expr(out, op, a1, a2)
    return binary_expr(out, op, t1, t2)


def add(out, t1, t2):
    """expr.ex:889-918."""
    c1, c2 = maybe_constant(t1), maybe_constant(t2)
    if c1 == 0 and c1 is not None:
        return ensure_compatible(t2, out)
    if c2 == 0 and c2 is not None:
        return ensure_compatible(t1, out)
    if c2 is not None:
        return _commute(out, "add", c2, t2, t1)
    return _commute(out, "add", c1, t1, t2)


def multiply(out, t1, t2):
    """expr.ex:934-962."""
    c1, c2 = maybe_constant(t1), maybe_constant(t2)
    if c1 == 1 and c1 is not None:
        return ensure_compatible(t2, out)
    if c2 == 1 and c2 is not None:
        return ensure_compatible(t1, out)
    if c2 is not None:
        return _commute(out, "multiply", c2, t2, t1)
    return _commute(out, "multiply", c1, t1, t2)


def subtract(out, t1, t2):
    """expr.ex:921-931."""
    c2 = maybe_constant(t2)
    if c2 == 0 and c2 is not None:
        return ensure_compatible(t1, out)
    return binary_expr(out, "subtract", t1, t2)


def divide(out, t1, t2):
    """expr.ex:965-973."""
    c2 = maybe_constant(t2)
    if c2 == 1 and c2 is not None:
        return ensure_compatible(t1, out)
    return binary_expr(out, "divide", t1, t2)


# ---- serialisation ------------------------------------------------------------

MAGIC = b"NXB1"


def topo_order(outputs):
    """Depth-first post-order over the DAG, memoised by node id exactly like
    the reference's lowering (exla/lib/exla/defn.ex:659-668)."""
    order, seen = [], {}
    stack = [(t, False) for t in reversed(outputs)]
    while stack:
        t, done = stack.pop()
        e = t.data
        if e.id in seen and not done:
            continue
        if done:
            if e.id not in seen:
                seen[e.id] = len(order)
                order.append(t)
            continue
        stack.append((t, True))
        for a in reversed(e.args):
            if a.data.id not in seen:
                stack.append((a, False))
    return order, seen


def serialize(outputs, params=None, aliases=None):
    """Flatten the DAG reachable from ``outputs`` (a list of tensors whose data
    are Expr nodes) into the program wire format.  ``params`` (the function's
    parameter nodes) are written even when no output depends on them, so that
    the program keeps the function's arity (EXLA likewise accepts arguments it
    does not use, exla/lib/exla/defn.ex used-inputs handling)."""
    order, index = topo_order(outputs)
    for p in params or []:
        if p.data.id not in index:
            index[p.data.id] = len(order)
            order.append(p)
    buf = bytearray(MAGIC)
    buf += struct.pack("<I", len(order))
    for t in order:
        e = t.data
        # a host tap that was not lowered by the runner is an identity on the device
        name = ("metadata" if e.op == "io_call" else e.op).encode("ascii")
        buf += struct.pack("<B", len(name)) + name
        buf += struct.pack("<BB", T.DTYPE_CODES[t.type], len(t.shape))
        buf += struct.pack(f"<{len(t.shape)}q", *t.shape)
        buf += struct.pack("<H", len(e.args))
        buf += struct.pack(f"<{len(e.args)}I", *[index[a.data.id] for a in e.args])
        buf += struct.pack("<H", len(e.ints)) + struct.pack(f"<{len(e.ints)}q", *e.ints)
        buf += struct.pack("<H", len(e.flts)) + struct.pack(f"<{len(e.flts)}d", *e.flts)
        buf += struct.pack("<Q", len(e.blob)) + e.blob
    buf += struct.pack("<I", len(outputs))
    buf += struct.pack(f"<{len(outputs)}I", *[index[t.data.id] for t in outputs])
    if aliases:
        # buffer donation: (parameter index, output index) pairs, the result takes over the argument's memory
        buf += struct.pack("<I", len(aliases))
        for p, o in aliases:
            buf += struct.pack("<II", p, o)
    return bytes(buf)
