"""The front-end plus the oracle against an independent statement of the same operations in numpy.

Every random step is applied twice: through `nx_b200.nx` (traced, serialised, interpreted by the oracle in
its f64 `binary_backend` mode) and directly on the numpy arrays with numpy's own functions.  The two must
agree to rounding for floats and exactly for integers and predicates.  This pins the oracle's
index arithmetic (slices with strides, padding with interior and negative edges, lookups, window
reductions, scatters, sorts, general products, reductions over any axes) with something that shares no
code with it."""
import math
import random

import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import defn, nx

DIMS = [1, 2, 3, 4, 5, 7]
KINDS = ["unary", "binary", "binary", "compare", "reduce", "arg", "reshape", "transpose", "broadcast", "slice", "pad",
         "reverse", "concat", "stack", "select", "clip", "dot", "take", "take_along", "put_slice", "window", "sort",
         "argsort", "scatter", "iota", "logsumexp", "mean", "squeeze", "allany", "top_k", "slice_along"]


def _np_pad(a, value, config):
    """Nx.pad: (low, high, interior) per axis; negative edges crop (nx/lib/nx.ex pad)."""
    for axis, (lo, hi, interior) in enumerate(config):
        n = a.shape[axis]
        if interior and n > 0:
            shape = list(a.shape)
            shape[axis] = n + (n - 1) * interior
            spread = np.full(shape, value, dtype=a.dtype)
            index = [slice(None)] * a.ndim
            index[axis] = slice(0, None, interior + 1)
            spread[tuple(index)] = a
            a = spread
        for edge, at_start in ((lo, True), (hi, False)):
            if edge > 0:
                shape = list(a.shape)
                shape[axis] = edge
                block = np.full(shape, value, dtype=a.dtype)
                a = np.concatenate([block, a] if at_start else [a, block], axis=axis)
            elif edge < 0:
                index = [slice(None)] * a.ndim
                index[axis] = slice(-edge, None) if at_start else slice(0, a.shape[axis] + edge)
                a = a[tuple(index)]
    return a


def _np_window(a, win, strides, padding, how):
    identity = {"sum": 0.0, "max": -np.inf, "min": np.inf}[how]
    if padding == "same":                  # nx/lib/nx/shape.ex:547-552: window - 1 in all, the odd one behind
        pads = [((w - 1) // 2, (w - 1) - (w - 1) // 2) for w in win]
    else:
        pads = [(0, 0)] * a.ndim
    a = np.pad(a, pads, constant_values=identity)
    view = np.lib.stride_tricks.sliding_window_view(a, win)
    view = view[tuple(slice(0, None, s) for s in strides)]
    axes = tuple(range(a.ndim, 2 * a.ndim))
    return {"sum": np.sum, "max": np.max, "min": np.min}[how](view, axis=axes)


def _broadcastable(a, b):
    try:
        np.broadcast_shapes(a, b)
        return True
    except ValueError:
        return False


def _step(r, kind, x, a, vals):
    """(traced value, numpy value) of one random operation on (x, a); None when it does not apply."""
    if kind == "unary":
        if a.dtype != np.float64:
            return nx.negate(x), -a
        name, twin = r.choice([("exp", np.exp), ("tanh", np.tanh), ("negate", np.negative), ("abs", np.abs),
                               ("cos", np.cos), ("sin", np.sin), ("floor", np.floor), ("ceil", np.ceil), ("sign", np.sign),
                               ("sigmoid", lambda t: 1.0 / (1.0 + np.exp(-t))), ("atan", np.arctan), ("expm1", np.expm1),
                               ("erf", np.vectorize(math.erf, otypes=[np.float64])), ("asinh", np.arcsinh)])
        return getattr(nx, name)(x), twin(a)
    if kind == "binary":
        cands = [(v, w) for v, w in vals if w.dtype == a.dtype and _broadcastable(w.shape, a.shape)]
        y, b = r.choice(cands)
        if a.dtype == np.float64:
            name, twin = r.choice([("add", np.add), ("subtract", np.subtract), ("multiply", np.multiply), ("max", np.maximum),
                                   ("min", np.minimum), ("atan2", np.arctan2),
                                   ("divide", lambda p, q: p / (np.abs(q) + 1.0))])
            if name == "divide":
                return x / (nx.abs(y) + 1.0), twin(a, b)
            return getattr(nx, name)(x, y), twin(a, b)
        name, twin = r.choice([("add", np.add), ("subtract", np.subtract), ("multiply", np.multiply), ("max", np.maximum),
                               ("min", np.minimum), ("bitwise_and", np.bitwise_and), ("bitwise_xor", np.bitwise_xor),
                               ("remainder", lambda p, q: np.fmod(p, np.abs(q) + 1)),
                               ("quotient", lambda p, q: np.trunc(p / (np.abs(q) + 1)).astype(np.int64))])
        if name in ("remainder", "quotient"):
            return getattr(nx, name)(x, nx.abs(y) + 1), twin(a, b)
        return getattr(nx, name)(x, y), twin(a, b)
    if kind == "compare":
        cands = [(v, w) for v, w in vals if w.dtype == a.dtype and _broadcastable(w.shape, a.shape)]
        y, b = r.choice(cands)
        name, twin = r.choice([("greater", np.greater), ("less_equal", np.less_equal), ("equal", np.equal), ("not_equal", np.not_equal)])
        return nx.as_type(getattr(nx, name)(x, y), "s64"), twin(a, b).astype(np.int64)
    if kind == "select":
        cands = [(v, w) for v, w in vals if w.shape == a.shape and w.dtype == a.dtype]
        (y, b), (z, c) = r.choice(cands), r.choice(cands)
        return nx.select(nx.greater(x, 0), y, z), np.where(a > 0, b, c)
    if kind == "clip":
        return (nx.clip(x, -0.5, 0.75), np.clip(a, -0.5, 0.75)) if a.dtype == np.float64 else (nx.clip(x, -3, 4), np.clip(a, -3, 4))
    if kind == "reshape":
        n = a.size
        shape = r.choice([(n,), (1, n), (n, 1)] + [(d, n // d) for d in (2, 3, 4, 5) if n % d == 0])
        return nx.reshape(x, shape), a.reshape(shape)
    if kind == "broadcast":
        if a.ndim >= 3:
            return None
        shape = (r.choice([1, 2, 3]),) + a.shape
        return nx.broadcast(x, shape), np.broadcast_to(a, shape)
    if kind == "stack":
        cands = [(v, w) for v, w in vals if w.shape == a.shape and w.dtype == a.dtype]
        y, b = r.choice(cands)
        axis = r.randint(0, a.ndim)
        return nx.stack([x, y], axis=axis), np.stack([a, b], axis=axis)
    if kind == "squeeze":
        ones = [i for i, d in enumerate(a.shape) if d == 1]
        if not ones:
            return None
        axis = r.choice(ones)
        return nx.squeeze(x, [axis]), np.squeeze(a, axis)
    if kind == "dot":
        cands = [(v, w) for v, w in vals if w.dtype == a.dtype and w.ndim >= 1 and a.ndim >= 1 and w.shape[0 if w.ndim == 1 else -2] == a.shape[-1]]
        if not cands:
            return None
        y, b = r.choice(cands)
        want = np.tensordot(a, b, axes=([a.ndim - 1], [0 if b.ndim == 1 else b.ndim - 2]))
        return nx.dot(x, [a.ndim - 1], y, [0 if b.ndim == 1 else b.ndim - 2]), want
    if a.ndim == 0:
        return None
    last = a.ndim - 1
    if kind == "reduce":
        axes = sorted(r.sample(range(a.ndim), r.randint(1, a.ndim)))
        keep = r.random() < 0.5
        name, twin = r.choice([("sum", np.sum), ("product", np.prod), ("reduce_max", np.max), ("reduce_min", np.min)])
        if name == "product" and a.dtype == np.float64:
            x, a = nx.tanh(x), np.tanh(a)
        return getattr(nx, name)(x, axes=axes, keep_axes=keep), twin(a, axis=tuple(axes), keepdims=keep)
    if kind == "mean":
        if a.dtype != np.float64:
            return None
        axis = r.randrange(a.ndim)
        return nx.mean(x, axes=[axis]), np.mean(a, axis=axis)
    if kind == "allany":
        axis = r.randrange(a.ndim)
        name, twin = r.choice([("all", np.all), ("any", np.any)])
        return nx.as_type(getattr(nx, name)(x, axes=[axis]), "s64"), twin(a != 0, axis=axis).astype(np.int64)
    if kind == "arg":
        axis = r.randrange(a.ndim)
        name, twin = r.choice([("argmax", np.argmax), ("argmin", np.argmin)])     # first occurrence = tie_break: :low
        return nx.as_type(getattr(nx, name)(x, axis=axis), "s64"), twin(a, axis=axis).astype(np.int64)
    if kind == "transpose":
        if a.ndim < 2:
            return None
        perm = list(range(a.ndim))
        r.shuffle(perm)
        return nx.transpose(x, axes=perm), np.transpose(a, perm)
    if kind == "slice":
        starts = [r.randrange(d) for d in a.shape]
        lengths = [r.randint(1, d - s) for d, s in zip(a.shape, starts)]
        strides = [r.choice([1, 1, 2, 3]) for _ in a.shape]
        index = tuple(slice(s, s + n, k) for s, n, k in zip(starts, lengths, strides))
        return nx.slice(x, starts, lengths, strides=strides), a[index]
    if kind == "slice_along":
        axis = r.randrange(a.ndim)
        start = r.randrange(a.shape[axis])
        length = r.randint(1, a.shape[axis] - start)
        return nx.slice_along_axis(x, start, length, axis=axis), np.take(a, range(start, start + length), axis=axis)
    if kind == "pad":
        config = [(r.randint(-1 if d > 2 else 0, 2), r.randint(-1 if d > 2 else 0, 2), r.choice([0, 0, 1, 2])) for d in a.shape]
        value = 0.5 if a.dtype == np.float64 else 9
        return nx.pad(x, value, config), _np_pad(a, value, config)
    if kind == "reverse":
        axes = sorted(r.sample(range(a.ndim), r.randint(1, a.ndim)))
        return nx.reverse(x, axes=axes), np.flip(a, axis=tuple(axes))
    if kind == "concat":
        axis = r.randrange(a.ndim)
        cands = [(v, w) for v, w in vals if w.dtype == a.dtype and w.ndim == a.ndim
                 and all(i == axis or p == q for i, (p, q) in enumerate(zip(w.shape, a.shape)))]
        y, b = r.choice(cands)
        return nx.concatenate([x, y], axis=axis), np.concatenate([a, b], axis=axis)
    if kind == "iota":
        axis = r.randrange(a.ndim)
        steps = np.indices(a.shape)[axis]
        return nx.add(x, nx.as_type(nx.iota(a.shape, axis=axis, type="s64"), "f64" if a.dtype == np.float64 else "s64")), a + steps.astype(a.dtype)
    if kind == "logsumexp":
        if a.dtype != np.float64:
            return None
        m = np.max(a, axis=last, keepdims=True)
        return nx.logsumexp(x, axes=[last]), np.squeeze(np.log(np.sum(np.exp(a - m), axis=last, keepdims=True)) + m, last)
    if kind == "take":
        axis = r.randrange(a.ndim)
        picks = np.array([r.randrange(a.shape[axis]) for _ in range(r.choice([1, 3, 4]))], dtype=np.int64)
        return nx.take(x, nx.tensor(picks, "s64"), axis=axis), np.take(a, picks, axis=axis)
    if kind == "take_along":
        axis = r.randrange(a.ndim)
        picks = np.random.default_rng(r.randrange(1 << 30)).integers(0, a.shape[axis], a.shape).astype(np.int64)
        return nx.take_along_axis(x, nx.tensor(picks, "s64"), axis=axis), np.take_along_axis(a, picks, axis=axis)
    if kind == "put_slice":
        cands = [(v, w) for v, w in vals if w.dtype == a.dtype and w.ndim == a.ndim and all(p <= q for p, q in zip(w.shape, a.shape))]
        y, b = r.choice(cands)
        starts = [r.randrange(d - n + 1) for d, n in zip(a.shape, b.shape)]
        out = a.copy()
        out[tuple(slice(s, s + n) for s, n in zip(starts, b.shape))] = b
        return nx.put_slice(x, starts, y), out
    if kind == "window":
        if a.ndim > 2 or a.dtype != np.float64:
            return None
        win = tuple(r.randint(1, min(3, d)) for d in a.shape)
        stride = r.choice([1, 2])
        padding = r.choice(["valid", "same"])
        how = r.choice(["sum", "max", "min"])
        got = getattr(nx, "window_" + how)(x, win, strides=stride, padding=padding)
        return got, _np_window(a, win, [stride] * a.ndim, padding, how)
    if kind in ("sort", "argsort"):
        descending = r.random() < 0.5
        order = np.argsort(-a if descending else a, axis=last, kind="stable")
        if kind == "sort":
            return nx.sort(x, axis=last, direction="desc" if descending else "asc"), np.take_along_axis(a, order, axis=last)
        got = nx.argsort(x, axis=last, direction="desc" if descending else "asc", stable=True)
        return nx.as_type(got, "s64"), order.astype(np.int64)
    if kind == "top_k":
        k = r.randint(1, a.shape[last])
        order = np.argsort(-a, axis=last, kind="stable")[..., :k]
        values, _ = nx.top_k(x, k=k)
        return values, np.take_along_axis(a, order, axis=last)
    if kind == "scatter":
        if a.ndim != 1:
            return None
        k = r.choice([1, 3, 5])
        where = np.array([[r.randrange(a.shape[0])] for _ in range(k)], dtype=np.int64)
        updates = (np.arange(k) + 1).astype(a.dtype)
        out = a.copy()
        if r.random() < 0.5:
            np.add.at(out, where[:, 0], updates)
            return nx.indexed_add(x, nx.tensor(where, "s64"), nx.tensor(updates, "f64" if a.dtype == np.float64 else "s64")), out
        if len(set(where[:, 0].tolist())) != k:
            return None                      # which of two writes to one place wins is not specified
        out[where[:, 0]] = updates
        return nx.indexed_put(x, nx.tensor(where, "s64"), nx.tensor(updates, "f64" if a.dtype == np.float64 else "s64")), out
    raise AssertionError(kind)


def _case(seed):
    rng = random.Random(seed)
    data = np.random.default_rng(seed)
    arrays = []
    for _ in range(rng.randint(1, 3)):
        shape = tuple(rng.choice(DIMS) for _ in range(rng.choice([1, 2, 2, 3])))
        arrays.append(data.standard_normal(shape) * 1.5 if rng.random() < 0.7 else data.integers(-6, 7, shape).astype(np.int64))
    types = ["f64" if a.dtype == np.float64 else "s64" for a in arrays]
    host = [host_tensor(a, t) for a, t in zip(arrays, types)]
    steps = rng.randint(2, 12)
    op_seed = seed * 2654435761 % (1 << 31)
    expected = []

    def fun(*tensors):
        r = random.Random(op_seed)
        vals = list(zip(tensors, arrays))
        for _ in range(steps):
            kind = r.choice(KINDS)
            x, a = r.choice(vals)
            made = _step(r, kind, x, a, vals)
            if made is not None and made[1].size <= 4096:
                assert tuple(made[0].shape) == tuple(made[1].shape), (kind, made[0].shape, made[1].shape)
                vals.append((made[0], np.asarray(made[1])))
        made = vals[len(tensors):] or [(tensors[0] + 1, arrays[0] + 1)]
        del expected[:]
        expected.extend(w for _, w in made)
        return tuple(v for v, _ in made)

    blob, _ = defn.build_program(fun, host)
    with np.errstate(all="ignore"):
        results = O.run_program(blob, [h.data.raw for h in host], "binary_backend")
    return results, list(expected)


@pytest.mark.parametrize("seed", range(300))
def test_the_oracle_agrees_with_numpy_on_a_random_composition(seed):
    with np.errstate(all="ignore"):
        results, expected = _case(seed)
    assert len(results) == len(expected)
    for (value, type_, _raw), want in zip(results, expected):
        value = np.asarray(value)
        assert value.shape == want.shape
        if want.dtype == np.float64:
            assert type_ == ("f", 64)
            np.testing.assert_allclose(value.astype(np.float64), want, rtol=1e-9, atol=1e-12, equal_nan=True)
        else:
            np.testing.assert_array_equal(value.astype(np.int64), want.astype(np.int64))
