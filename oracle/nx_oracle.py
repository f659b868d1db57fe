"""CPU oracle for the Nx hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product may import this module: it exists so that tests, the
smoke check and the benchmark's CPU-baseline leg can compare the CUDA path with
an independent restatement of the reference's semantics.  It interprets the
same serialised expression graph the runtime compiles, one node at a time, the
way Nx.Defn.Evaluator walks a graph over a backend
(nx/lib/nx/defn/evaluator.ex:363-388).

Two numerics modes:

``binary_backend``  restates Nx.BinaryBackend: every scalar is read into a
    64-bit float or an integer, the operation runs at that width, and the
    result is rounded once when it is written (nx/lib/nx/binary_backend.ex
    element_wise_bin_op :662-706, unary :936-939, bin_reduce :2342-2360,
    dot :477-599).  A bf16 store keeps the upper 16 bits of the f32 encoding,
    i.e. truncates (nx/lib/nx/shared.ex:136-152, nx/lib/nx/floating.ex:60-64).

``xla_like``  restates the lowering rules of exla/lib/exla/defn.ex: operands
    are converted to the merged type before a binary op and the result to the
    node's type after it (:2380-2410), unary ops run in the node's type
    (:1374-1377), reductions convert their input first (:2148), arithmetic is
    IEEE in that type (bf16 values are widened to f32 for the operation and
    rounded to nearest-even after every node; dot accumulates in f32).

Parity status: pinned against the known-answer vectors of the reference's own
tests (tests/golden/reference_vectors.py lists them with file:line).  The
reference itself cannot run where this was written (no Erlang/Elixir, no XLA),
so full-size parity against the EXLA host client is unpinned.
"""
from __future__ import annotations

import math
import struct

import numpy as np

try:                                    # scipy is only needed for erf-family ops
    from scipy import special as _sp
except Exception:                       # pragma: no cover
    _sp = None

KINDS = {0: ("u", 8), 1: ("u", 16), 2: ("u", 32), 3: ("u", 64), 4: ("s", 8), 5: ("s", 16),
         6: ("s", 32), 7: ("s", 64), 8: ("f", 16), 9: ("bf", 16), 10: ("f", 32), 11: ("f", 64)}
NP = {("u", 8): np.uint8, ("u", 16): np.uint16, ("u", 32): np.uint32, ("u", 64): np.uint64,
      ("s", 8): np.int8, ("s", 16): np.int16, ("s", 32): np.int32, ("s", 64): np.int64,
      ("f", 16): np.float16, ("f", 32): np.float32, ("f", 64): np.float64,
      ("bf", 16): np.float32}          # bf16 values are held widened, exactly representable


def is_float(t):
    return t[0] in ("f", "bf")


def type_merge(a, b):
    """nx/lib/nx/type.ex:463-473."""
    order = {"u": 0, "s": 1, "bf": 2, "f": 3}
    if a[0] == b[0]:
        return (a[0], max(a[1], b[1]))
    lo, hi = (a, b) if order[a[0]] < order[b[0]] else (b, a)
    if lo[0] == "u" and hi[0] == "s":
        return ("s", max(min(lo[1] * 2, 64), hi[1]))
    return hi


# ---- bf16 ------------------------------------------------------------------------

def bf16_round_rne(a):
    """f32 -> nearest-even bf16, returned widened to f32 (XLA convert)."""
    shape = np.shape(a)
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    u = a.view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    out = r.view(np.float32)
    return np.where(np.isnan(a), np.float32(np.nan), out).astype(np.float32).reshape(shape)


def bf16_truncate(a):
    """f32 -> bf16 by dropping the low 16 bits (nx/lib/nx/floating.ex:60-64)."""
    shape = np.shape(a)
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    out = (a.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    return np.where(np.isnan(a), np.float32(np.nan), out).astype(np.float32).reshape(shape)


def decode(raw, t, shape):
    """Raw little-endian bytes -> oracle array."""
    if t == ("bf", 16):
        u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << np.uint32(16)
        return u.view(np.float32).reshape(shape).copy()
    return np.frombuffer(raw, dtype=NP[t]).reshape(shape).copy()


def encode(arr, t):
    """Oracle array -> raw bytes (bf16 arrays are already exactly representable)."""
    if t == ("bf", 16):
        a = np.ascontiguousarray(arr, dtype=np.float32)
        bits = (a.view(np.uint32) >> np.uint32(16)).astype(np.uint16)
        bits = np.where(np.isnan(a), np.uint16(0x7FC0), bits)
        return bits.tobytes()
    return np.ascontiguousarray(arr, dtype=NP[t]).tobytes()


# ---- conversion ("store") rules --------------------------------------------------

def _int_limits(t):
    if t[0] == "u":
        return 0, (1 << t[1]) - 1
    return -(1 << (t[1] - 1)), (1 << (t[1] - 1)) - 1


def convert(arr, src, dst, mode):
    """as_type semantics.  float -> int truncates, NaN -> 0, +inf -> max,
    -inf -> min (nx/lib/nx/binary_backend.ex:2056-2069; pinned by
    exla/test/exla/defn/expr_test.exs:1117-1130)."""
    if src == dst:
        return arr
    with np.errstate(all="ignore"):
        if is_float(dst):
            if dst == ("bf", 16):
                f = arr.astype(np.float32)
                return bf16_truncate(f) if mode == "binary_backend" else bf16_round_rne(f)
            return arr.astype(NP[dst])
        lo, hi = _int_limits(dst)
        if is_float(src):
            a = arr.astype(np.float64)
            tr = np.trunc(np.where(np.isfinite(a), a, 0.0))
            if mode == "binary_backend":      # integer written modulo 2^bits (shared.ex:190-194)
                ints = np.array([int(v) for v in tr.ravel()], dtype=object)
                span = 1 << dst[1]
                wrapped = np.array([((int(v) - lo) % span) + lo for v in ints], dtype=object)
                res = wrapped.astype(NP[dst]).reshape(a.shape)
            else:                              # saturating, like a hardware convert
                # the limits of the 64-bit types are not doubles: compare first, convert what lies inside
                inside = (tr > float(lo)) & (tr < float(hi))
                res = np.where(inside, tr, 0.0).astype(NP[dst])
                res = np.where(tr >= float(hi), np.array(hi, NP[dst]), res)
                res = np.where(tr <= float(lo), np.array(lo, NP[dst]), res)
            res = np.where(np.isnan(a), np.array(0, NP[dst]), res)
            res = np.where(a == np.inf, np.array(hi, NP[dst]), res)
            res = np.where(a == -np.inf, np.array(lo, NP[dst]), res)
            return res.astype(NP[dst])
        return arr.astype(NP[dst])             # int -> int wraps


def _compute_dtype(t, mode):
    """The width arithmetic runs at."""
    if mode == "binary_backend":
        return np.float64 if is_float(t) else np.int64
    if t in (("bf", 16), ("f", 16)):
        # 16-bit floats are computed in f32 and rounded once (for + - * / that IS the correctly rounded 16-bit
        # result; numpy's own float16 functions are a few units off for the transcendental ones)
        return np.float32
    return NP[t]


def _store(v, t, mode):
    """Round a value computed at `_compute_dtype` into type t."""
    with np.errstate(all="ignore"):
        if t == ("bf", 16):
            f = np.asarray(v).astype(np.float32)
            return bf16_truncate(f) if mode == "binary_backend" else bf16_round_rne(f)
        return np.asarray(v).astype(NP[t])


def _load(arr, src, t, mode):
    """Bring an operand to the compute representation of type t."""
    if mode == "binary_backend":
        # BinaryBackend reads each operand in its own type into a number
        return arr.astype(np.float64) if (is_float(src) or is_float(t)) else arr.astype(np.int64)
    return convert(arr, src, t, mode).astype(_compute_dtype(t, mode))


# ---- scalar function tables -----------------------------------------------------

def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _round_half_away(x):
    return np.where(x >= 0, np.floor(x + 0.5), np.ceil(x - 0.5)).astype(x.dtype)


def _erf_family(name):
    if _sp is None:
        raise RuntimeError("scipy is required for " + name)
    return {"erf": _sp.erf, "erfc": _sp.erfc, "erf_inv": _sp.erfinv}[name]


UNARY_FLOAT = {
    "exp": np.exp, "expm1": np.expm1, "log": np.log, "log1p": np.log1p, "sigmoid": _sigmoid,
    "cos": np.cos, "sin": np.sin, "tan": np.tan, "cosh": np.cosh, "sinh": np.sinh,
    "tanh": np.tanh, "acos": np.arccos, "asin": np.arcsin, "atan": np.arctan,
    "acosh": np.arccosh, "asinh": np.arcsinh, "atanh": np.arctanh, "sqrt": np.sqrt,
    "rsqrt": lambda x: 1.0 / np.sqrt(x), "cbrt": np.cbrt,
    "erf": lambda x: _erf_family("erf")(x), "erfc": lambda x: _erf_family("erfc")(x),
    "erf_inv": lambda x: _erf_family("erf_inv")(x),
}


def _popcount(a):
    u = a.astype(np.uint64) & np.uint64((1 << (a.dtype.itemsize * 8)) - 1 if a.dtype.itemsize < 8 else 0xFFFFFFFFFFFFFFFF)
    out = np.zeros(a.shape, dtype=np.uint64)
    for _ in range(64):
        out += u & np.uint64(1)
        u >>= np.uint64(1)
    return out


def _clz(a, bits):
    u = a.astype(np.uint64) & np.uint64((1 << bits) - 1 if bits < 64 else 0xFFFFFFFFFFFFFFFF)
    out = np.full(a.shape, bits, dtype=np.int64)
    for i in range(bits):
        has = (u >> np.uint64(i)) & np.uint64(1)
        out = np.where(has == 1, bits - 1 - i, out)
    return out


def _int_pow(a, b):
    """Integer power by squaring, wrapping; a negative exponent gives 1 for base 1, +-1 for base -1 and 0
    otherwise (what XLA's integer pow returns; Nx.BinaryBackend raises there)."""
    res = np.ones_like(a)
    base = a.copy()
    e = np.where(b < 0, 0, b).astype(b.dtype) if b.dtype.kind == "i" else b.copy()
    with np.errstate(all="ignore"):
        for _ in range(64):
            res = np.where(e & 1, res * base, res)
            base = base * base
            e = e >> 1
        if b.dtype.kind == "i":
            minus_one = a == np.array(-1).astype(a.dtype)
            negative = np.where(a == 1, 1, np.where(minus_one, np.where(b & 1, -1, 1), 0)).astype(a.dtype)
            res = np.where(b < 0, negative, res)
    return res


def _quotient(a, b):
    """Truncating integer division at the operands' own width; x / 0 is all ones (-1) and the most
    negative value divided by -1 is itself, as XLA defines them (Nx.BinaryBackend raises for a zero divisor)."""
    with np.errstate(all="ignore"):
        safe = np.where(b == 0, 1, b).astype(b.dtype)
        q = a // safe
        if a.dtype.kind == "i":
            r = a - q * safe
            q = np.where((r != 0) & ((a < 0) != (safe < 0)), q + 1, q)
        return np.where(b == 0, np.array(-1).astype(a.dtype), q).astype(a.dtype)


def _int_remainder(a, b):
    """Sign of the dividend; x rem 0 is x (XLA)."""
    with np.errstate(all="ignore"):
        safe = np.where(b == 0, 1, b).astype(b.dtype)
        return np.where(b == 0, a, np.fmod(a, safe)).astype(a.dtype)


def _binary(op, a, b, t):
    """a, b already at compute width."""
    fl = a.dtype.kind == "f"
    with np.errstate(all="ignore"):
        if op == "add": return a + b
        if op == "subtract": return a - b
        if op == "multiply": return a * b
        if op == "divide": return a / b
        if op == "max": return np.maximum(a, b)          # NaN wins (binary_backend.ex:719-725)
        if op == "min": return np.minimum(a, b)
        if op == "pow": return np.power(a, b) if fl else _int_pow(a, b)
        if op == "remainder": return np.fmod(a, b) if fl else _int_remainder(a, b)    # sign of the dividend (rem / :math.fmod)
        if op == "atan2": return np.arctan2(a, b)
        if op == "quotient": return _quotient(a, b)
        if op == "bitwise_and": return a & b
        if op == "bitwise_or": return a | b
        if op == "bitwise_xor": return a ^ b
        if op == "left_shift": return a << b
        if op == "right_shift": return a >> b             # arithmetic for signed, logical for unsigned
        if op == "equal": return (a == b).astype(np.uint8)
        if op == "not_equal": return (a != b).astype(np.uint8)
        if op == "greater": return (a > b).astype(np.uint8)
        if op == "less": return (a < b).astype(np.uint8)
        if op == "greater_equal": return (a >= b).astype(np.uint8)
        if op == "less_equal": return (a <= b).astype(np.uint8)
        if op == "logical_and": return ((a != 0) & (b != 0)).astype(np.uint8)
        if op == "logical_or": return ((a != 0) | (b != 0)).astype(np.uint8)
        if op == "logical_xor": return ((a != 0) ^ (b != 0)).astype(np.uint8)
    raise NotImplementedError(op)


BINARY_OPS = {"add", "subtract", "multiply", "divide", "max", "min", "pow", "remainder", "atan2",
              "quotient", "bitwise_and", "bitwise_or", "bitwise_xor", "left_shift", "right_shift",
              "equal", "not_equal", "greater", "less", "greater_equal", "less_equal",
              "logical_and", "logical_or", "logical_xor"}
PRED_OPS = {"equal", "not_equal", "greater", "less", "greater_equal", "less_equal",
            "logical_and", "logical_or", "logical_xor"}
UNARY_OTHER = {"abs", "bitwise_not", "ceil", "floor", "negate", "round", "sign",
               "count_leading_zeros", "population_count", "is_nan", "is_infinity"}
REDUCE_OPS = {"sum", "product", "reduce_max", "reduce_min", "all", "any"}


# ---- program parsing ----------------------------------------------------------------

class Node:
    __slots__ = ("op", "type", "shape", "args", "ints", "flts", "blob")


def parse_program(blob):
    if blob[:4] != b"NXB1":
        raise ValueError("bad magic")
    pos = 4

    def take(fmt):
        nonlocal pos
        vals = struct.unpack_from("<" + fmt, blob, pos)
        pos += struct.calcsize("<" + fmt)
        return vals

    (n,) = take("I")
    nodes = []
    for _ in range(n):
        nd = Node()
        (l,) = take("B")
        nd.op = blob[pos:pos + l].decode("ascii"); pos += l
        code, rank = take("BB")
        nd.type = KINDS[code]
        nd.shape = tuple(take(f"{rank}q"))
        (na,) = take("H"); nd.args = list(take(f"{na}I"))
        (ni,) = take("H"); nd.ints = list(take(f"{ni}q"))
        (nf,) = take("H"); nd.flts = list(take(f"{nf}d"))
        (nb,) = take("Q"); nd.blob = blob[pos:pos + nb]; pos += nb
        nodes.append(nd)
    (no,) = take("I")
    outs = list(take(f"{no}I"))
    return nodes, outs


# ---- evaluation ----------------------------------------------------------------------

def _bcast(arr, shape):
    """Right-aligned broadcast (nx/lib/nx/binary_backend.ex:224-276)."""
    return np.broadcast_to(arr, shape)


def _reduce(op, x, src_t, out_t, axes, keep, mode):
    axes = tuple(axes)
    with np.errstate(all="ignore"):
        if op in ("all", "any"):
            b = x != 0
            r = b.all(axis=axes, keepdims=keep) if op == "all" else b.any(axis=axes, keepdims=keep)
            return r.astype(np.uint8)
        a = _load(x, src_t, out_t, mode)
        if op == "sum":
            if mode == "binary_backend" and a.dtype.kind == "f":
                # sequential accumulation in f64 (bin_reduce, :2342-2360)
                moved = np.moveaxis(a, axes, tuple(range(-len(axes), 0)))
                flat = moved.reshape(moved.shape[: a.ndim - len(axes)] + (-1,))
                r = np.cumsum(flat, axis=-1)[..., -1] if flat.shape[-1] else np.zeros(flat.shape[:-1])
                if keep:
                    r = r.reshape([1 if i in axes else d for i, d in enumerate(a.shape)])
            else:
                r = a.sum(axis=axes, keepdims=keep, dtype=a.dtype)
        elif op == "product":
            r = a.prod(axis=axes, keepdims=keep, dtype=a.dtype)
        elif op == "reduce_max":
            r = a.max(axis=axes, keepdims=keep)           # NaN propagates (:1349-1355)
        else:
            r = a.min(axis=axes, keepdims=keep)
        return _store(r, out_t, mode)


def _arg_reduce(op, x, tie_high, axis, keep, out_t, mode):
    """argmax/argmin.  NaN-free data: the extreme value, lowest (tie_break
    :low) or highest index among equals.  A NaN beats every number
    (binary_backend.ex:1415-1431, exla/lib/exla/lib.ex:118-146).  With several
    NaNs in one slice BinaryBackend's sequential scan returns the LAST one
    (pinned by nx/test/nx_test.exs:1778-1798, row [:nan, :nan, 1] -> 1), while
    EXLA's reducer keeps whichever NaN reaches the left operand first; in
    `xla_like` mode that is modelled as a left-to-right fold (first NaN)."""
    shape = x.shape
    if axis < 0:
        x = x.reshape(-1)
        axis = 0
    a = np.moveaxis(x, axis, -1)
    n = a.shape[-1]
    fl = a.dtype.kind == "f"
    key = a.astype(np.float64) if fl else a
    if op == "argmin":
        key = -key if fl else (-(key.astype(np.int64)) if key.dtype.kind == "i" else key.max(initial=0) - key)
    if fl:
        nan = np.isnan(key)
        key = np.where(nan, -np.inf, key)
    if tie_high:
        idx = n - 1 - np.argmax(key[..., ::-1], axis=-1)
    else:
        idx = np.argmax(key, axis=-1)
    if fl and nan.any():
        has = nan.any(axis=-1)
        first = np.argmax(nan, axis=-1)
        last = n - 1 - np.argmax(nan[..., ::-1], axis=-1)
        idx = np.where(has, last if mode == "binary_backend" else first, idx)
    if keep:
        if len(shape) and x.ndim == len(shape):
            idx = np.expand_dims(idx, axis)
        else:
            idx = idx.reshape((1,) * len(shape))
    return np.asarray(idx).astype(NP[out_t])


def _dot(a, ta, c1, b1, b, tb, c2, b2, out_t, mode):
    """nx/lib/nx/binary_backend.ex:477-599: batch axes lead, then the free axes
    of the left operand, then those of the right."""
    f1 = [i for i in range(a.ndim) if i not in c1 and i not in b1]
    f2 = [i for i in range(b.ndim) if i not in c2 and i not in b2]
    A = np.transpose(a, list(b1) + f1 + list(c1))
    B = np.transpose(b, list(b2) + list(c2) + f2)
    bs = [a.shape[i] for i in b1]
    m = [a.shape[i] for i in f1]
    n = [b.shape[i] for i in f2]
    k = int(np.prod([a.shape[i] for i in c1], dtype=np.int64))
    A = A.reshape(bs + [int(np.prod(m, dtype=np.int64)), k])
    B = B.reshape(bs + [k, int(np.prod(n, dtype=np.int64))])
    with np.errstate(all="ignore"):
        if is_float(out_t):
            if mode == "binary_backend":
                acc = np.matmul(A.astype(np.float64), B.astype(np.float64))
            elif out_t == ("f", 64):
                acc = np.matmul(A.astype(np.float64), B.astype(np.float64))
            else:
                # products of f32 operands accumulated in f32; the wider f64
                # accumulation differs from any f32 order by far less than the
                # test tolerance and does not depend on a BLAS build
                Ac = convert(A, ta, out_t, mode).astype(np.float64)
                Bc = convert(B, tb, out_t, mode).astype(np.float64)
                acc = np.matmul(Ac, Bc).astype(np.float32)
            r = _store(acc, out_t, mode)
        else:
            # Exact integer sums.  When every partial sum is below 2^53 in magnitude the same
            # integers come out of a float64 product (every term and every partial sum is then
            # exactly representable), which runs through BLAS; otherwise int64 arithmetic.
            amax = int(np.abs(A.astype(np.int64)).max(initial=0))
            bmax = int(np.abs(B.astype(np.int64)).max(initial=0))
            if k * amax * bmax < (1 << 53) and A.size * B.shape[-1] > (1 << 22):
                acc = np.matmul(A.astype(np.float64), B.astype(np.float64)).astype(np.int64)
            else:
                acc = np.matmul(A.astype(np.int64), B.astype(np.int64))
            r = acc.astype(NP[out_t])          # wraps modulo 2^bits (shared.ex:190-194)
    return r.reshape(bs + m + n)


def evaluate(nodes, outs, params, mode="xla_like", all_reduce=None):
    """params: list of oracle arrays (see `decode`). Returns list of arrays.
    ``all_reduce(array, mesh_axis)`` supplies the cross-partition sum for the
    programs of sharded runs (tests pass a gloo all-reduce)."""
    if mode not in ("xla_like", "binary_backend"):
        raise ValueError(mode)
    vals = [None] * len(nodes)
    for i, nd in enumerate(nodes):
        op, t = nd.op, nd.type
        arg = [vals[j] for j in nd.args]
        at = [nodes[j].type for j in nd.args]
        if op == "parameter":
            v = params[nd.ints[0]]
            if tuple(v.shape) != nd.shape:
                raise ValueError(f"parameter {nd.ints[0]}: shape {v.shape} != {nd.shape}")
        elif op == "constant":
            c = nd.flts[0] if nd.flts else nd.ints[0]
            with np.errstate(all="ignore"):
                v = _store(np.full(nd.shape, c, dtype=np.float64 if nd.flts else np.int64), t, mode) \
                    if t != ("bf", 16) else _store(np.full(nd.shape, c, dtype=np.float64), t, mode)
        elif op == "tensor":
            v = decode(nd.blob, t, nd.shape)
        elif op == "metadata":
            v = arg[0]
        elif op == "all_reduce":
            if all_reduce is None:
                raise ValueError("program contains all_reduce but no reducer was given")
            v = _store(all_reduce(arg[0].astype(np.float64 if is_float(t) else np.int64), nd.ints[0]), t, mode)
        elif op == "iota":
            ax = nd.ints[0]
            if ax < 0:
                v = np.arange(int(np.prod(nd.shape, dtype=np.int64))).reshape(nd.shape)
            else:
                sh = [1] * len(nd.shape); sh[ax] = nd.shape[ax]
                v = np.broadcast_to(np.arange(nd.shape[ax]).reshape(sh), nd.shape)
            v = _store(v, t, mode)
        elif op == "as_type":
            v = convert(arg[0], at[0], t, mode)
        elif op in UNARY_FLOAT:
            x = _load(arg[0], at[0], t, mode)
            with np.errstate(all="ignore"):
                v = _store(UNARY_FLOAT[op](x), t, mode)
        elif op in UNARY_OTHER:
            x = arg[0]
            with np.errstate(all="ignore"):
                if op == "is_nan":
                    v = (np.isnan(x) if x.dtype.kind == "f" else np.zeros(x.shape, bool)).astype(np.uint8)
                elif op == "is_infinity":
                    v = (np.isinf(x) if x.dtype.kind == "f" else np.zeros(x.shape, bool)).astype(np.uint8)
                elif op == "population_count":
                    v = _popcount(x).astype(NP[t])
                elif op == "count_leading_zeros":
                    v = _clz(x, at[0][1]).astype(NP[t])
                else:
                    xc = _load(x, at[0], t, mode)
                    f = {"abs": np.abs, "negate": np.negative, "floor": np.floor, "ceil": np.ceil,
                         "sign": np.sign, "bitwise_not": np.invert, "round": _round_half_away}[op]
                    v = _store(f(xc), t, mode)
        elif op in BINARY_OPS:
            ct = type_merge(type_merge(at[0], at[1]), t) if op not in PRED_OPS else type_merge(at[0], at[1])
            if op in ("logical_and", "logical_or", "logical_xor"):
                a, b = arg[0], arg[1]
            else:
                a, b = _load(arg[0], at[0], ct, mode), _load(arg[1], at[1], ct, mode)
                if mode == "binary_backend" and a.dtype != b.dtype:
                    a, b = a.astype(np.float64), b.astype(np.float64)
            if op == "right_shift" and mode == "xla_like" and t[0] == "u" and a.dtype.kind == "i":
                # The reference shifts logically when the RESULT type is unsigned, whatever signed type the
                # operands were merged to (exla/lib/exla/defn.ex:1328-1335): a u64 tensor shifted by a
                # number is computed in s64, and its values with the top bit set are not sign-extended.
                wide = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize]
                bits = np.asarray(_bcast(b, nd.shape)).astype(wide)
                shifted = np.where(bits >= a.dtype.itemsize * 8, wide(0), _bcast(a, nd.shape).astype(wide) >> np.minimum(bits, wide(a.dtype.itemsize * 8 - 1)))
                r = shifted.astype(a.dtype)
            else:
                r = _binary(op, _bcast(a, nd.shape), _bcast(b, nd.shape), ct)
            if op in PRED_OPS:
                v = r.astype(np.uint8)
            elif mode == "binary_backend":
                v = convert(r, ("f", 64) if r.dtype.kind == "f" else ("s", 64), t, mode) \
                    if (r.dtype.kind == "f") != is_float(t) else _store(r, t, mode)
            else:
                v = convert(_store(r, ct, mode), ct, t, mode)
        elif op == "select":
            p = _bcast(arg[0] != 0, nd.shape)
            a = _bcast(convert(arg[1], at[1], t, mode), nd.shape)
            b = _bcast(convert(arg[2], at[2], t, mode), nd.shape)
            v = np.where(p, a, b)
        elif op == "clip":
            x, lo, hi = (convert(arg[k], at[k], t, mode) for k in range(3))
            v = np.minimum(np.maximum(x, lo), hi)
        elif op in REDUCE_OPS:
            keep, n = nd.ints[0], nd.ints[1]
            v = _reduce(op, arg[0], at[0], t, nd.ints[2:2 + n], bool(keep), mode)
        elif op in ("argmax", "argmin"):
            v = _arg_reduce(op, arg[0], bool(nd.ints[0]), nd.ints[1], bool(nd.ints[2]), t, mode)
        elif op == "dot":
            it = iter(nd.ints)
            lists = []
            for _ in range(4):
                k = next(it)
                lists.append([next(it) for _ in range(k)])
            c1, b1, c2, b2 = lists
            v = _dot(arg[0], at[0], c1, b1, arg[1], at[1], c2, b2, t, mode)
        elif op in ("reshape", "squeeze"):
            v = arg[0].reshape(nd.shape)
        elif op == "broadcast":
            n = nd.ints[0]
            axes = nd.ints[1:1 + n]
            sh = [1] * len(nd.shape)
            for d, ax in zip(arg[0].shape, axes):
                sh[ax] = d
            v = np.broadcast_to(arg[0].reshape(sh), nd.shape)
        elif op == "transpose":
            v = np.transpose(arg[0], nd.ints)
        elif op == "slice":
            r = arg[0].ndim
            st, ln, sd = nd.ints[:r], nd.ints[r:2 * r], nd.ints[2 * r:3 * r]
            if len(arg) > 1:      # dynamic starts, clamped so that the window fits
                st = [min(max(int(s), 0), d - l) for s, d, l in zip(arg[1:], arg[0].shape, ln)]
            v = arg[0][tuple(slice(s, s + l, d) for s, l, d in zip(st, ln, sd))]
        elif op in ("window_sum", "window_max", "window_min", "window_product"):
            # nx/lib/nx/binary_backend.ex:1447-1530: pad with the identity, then reduce each window
            r = arg[0].ndim
            win, st, lo, hi, dil = (nd.ints[i * r:(i + 1) * r] for i in range(5))
            npt = NP[t]
            if op == "window_sum":
                ident = 0
            elif op == "window_product":
                ident = 1
            elif np.issubdtype(npt, np.floating):
                ident = -np.inf if op == "window_max" else np.inf
            else:
                ident = np.iinfo(npt).min if op == "window_max" else np.iinfo(npt).max
            x = np.pad(arg[0], list(zip(lo, hi)), constant_values=ident)
            fn = {"window_sum": np.add, "window_product": np.multiply, "window_max": np.maximum, "window_min": np.minimum}[op]
            acc = None
            for pos in np.ndindex(*win):
                sl = tuple(slice(p * d, p * d + (n - 1) * s + 1, s) for p, d, n, s in zip(pos, dil, nd.shape, st))
                term = x[sl].astype(npt)
                with np.errstate(over="ignore"):
                    acc = term if acc is None else fn(acc, term).astype(npt)
            v = _store(acc.astype(np.float64) if is_float(t) else acc, t, mode) if is_float(t) else acc
        elif op in ("sort", "argsort"):
            # nx/lib/nx.ex:15676-15689: NaN sorts higher than any other value; ties keep their order
            a = arg[0]
            desc = bool(nd.ints[0])
            pos = np.broadcast_to(np.arange(a.shape[-1]), a.shape)
            if is_float(at[0]):
                nan = np.isnan(a)
                val = np.where(nan, 0.0, a).astype(np.float64)
                order = np.lexsort((pos, -val, ~nan) if desc else (pos, val, nan), axis=-1)
            else:
                order = np.lexsort((pos, ~a if desc else a), axis=-1)       # ~v reverses integer order without overflow
            v = np.take_along_axis(a, order, axis=-1) if op == "sort" else order.astype(NP[t])
        elif op == "reverse":
            v = np.flip(arg[0], axis=tuple(nd.ints))
        elif op == "pad":
            # nx/lib/nx/binary_backend.ex:326-348: interior, then edges (negative edges crop)
            r = arg[0].ndim
            lo, hi, it = nd.ints[:r], nd.ints[r:2 * r], nd.ints[2 * r:3 * r]
            x = convert(arg[0], at[0], t, mode)
            pv = convert(arg[1], at[1], t, mode)
            for ax in range(r):
                d = x.shape[ax]
                n = d + max(d - 1, 0) * it[ax]
                sh = list(x.shape)
                sh[ax] = n
                y = np.full(sh, pv, dtype=x.dtype)
                sl = [slice(None)] * r
                sl[ax] = slice(0, n, it[ax] + 1)
                y[tuple(sl)] = x
                pads = [(0, 0)] * r
                pads[ax] = (max(lo[ax], 0), max(hi[ax], 0))
                y = np.pad(y, pads, constant_values=pv)
                sl[ax] = slice(max(-lo[ax], 0), y.shape[ax] - max(-hi[ax], 0))
                x = y[tuple(sl)]
            v = x
        elif op == "gather":
            # nx/lib/nx/binary_backend.ex:1903-1940 (indexed axes first, then a contiguous
            # copy per index row); coordinates clamped as XLA's gather does
            axes = list(nd.ints)
            rest = [j for j in range(arg[0].ndim) if j not in axes]
            tt = np.transpose(arg[0], axes + rest)
            idx = arg[1].astype(np.int64) if arg[1].dtype != np.uint64 else np.minimum(arg[1], np.uint64(2 ** 62)).astype(np.int64)
            coords = tuple(np.clip(idx[..., i], 0, tt.shape[i] - 1) for i in range(len(axes)))
            v = tt[coords]
        elif op == "put_slice":
            base, piece = convert(arg[0], at[0], t, mode), convert(arg[1], at[1], t, mode)
            st = [min(max(int(s), 0), d - l) for s, d, l in zip(arg[2:], base.shape, piece.shape)]
            v = np.array(base, copy=True)
            v[tuple(slice(s, s + l) for s, l in zip(st, piece.shape))] = piece
        elif op in ("indexed_add", "indexed_put"):
            # nx/lib/nx/binary_backend.ex indexed_op: every row of `indices` names a position along the
            # indexed axes; the matching slice of `updates` lands there (starting at 0 along the other
            # axes) and is added to, or replaces, what the target holds.  Rows are applied in order (with
            # repeated indices indexed_put keeps the last row, what a sequential evaluator does); rows
            # with a coordinate outside the target are dropped, as XLA's scatter drops them.
            axes = list(nd.ints)
            base, upd = convert(arg[0], at[0], t, mode), convert(arg[2], at[2], t, mode)
            idx = arg[1].astype(np.int64)
            rest = [j for j in range(base.ndim) if j not in axes]
            v = np.array(base, copy=True)
            work = v.astype(_compute_dtype(t, mode)) if op == "indexed_add" else v
            for row in range(idx.shape[0]):
                if any(idx[row, k] < 0 or idx[row, k] >= base.shape[a] for k, a in enumerate(axes)):
                    continue
                sl = [None] * base.ndim
                for k, a in enumerate(axes):
                    sl[a] = int(idx[row, k])
                piece = upd[row]
                for j, a in enumerate(rest):
                    sl[a] = slice(0, piece.shape[j])
                if op == "indexed_add":
                    with np.errstate(all="ignore"):
                        work[tuple(sl)] = _store(work[tuple(sl)] + piece.astype(work.dtype), t, mode).astype(work.dtype)
                else:
                    work[tuple(sl)] = piece
            v = _store(work, t, mode) if op == "indexed_add" else work
        elif op == "concatenate":
            v = np.concatenate([convert(a, ta, t, mode) for a, ta in zip(arg, at)], axis=nd.ints[0])
        else:
            raise NotImplementedError(f"oracle: op {op}")
        v = np.asarray(v)
        if tuple(v.shape) != nd.shape:
            raise AssertionError(f"{op}: produced {v.shape}, node says {nd.shape}")
        vals[i] = np.ascontiguousarray(v).reshape(nd.shape)
    return [vals[o] for o in outs]


def run_program(blob, params_raw, mode="xla_like", all_reduce=None):
    """Evaluate a serialised program.  ``params_raw`` are raw byte strings (one
    per parameter, in parameter order).  Returns a list of
    ``(array, type, raw_bytes)`` per output."""
    nodes, outs = parse_program(blob)
    ptypes = {}
    for nd in nodes:
        if nd.op == "parameter":
            ptypes[nd.ints[0]] = (nd.type, nd.shape)
    params = [None] * (max(ptypes) + 1 if ptypes else 0)
    for i, (t, s) in ptypes.items():
        params[i] = decode(params_raw[i], t, s)
    res = evaluate(nodes, outs, params, mode, all_reduce)
    return [(r, nodes[o].type, encode(r, nodes[o].type)) for r, o in zip(res, outs)]
