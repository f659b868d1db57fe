"""Random compositions of the differentiable operations: the gradient graph of `nx_b200.grad`, evaluated
by the oracle in f64, against central finite differences of the function itself (what the reference's
`check_grads!` does, nx/test/support/grad_helpers.ex), for functions nobody wrote by hand.  Kinks
(max / min / abs / clip / select / sort ties) are re-checked with a smaller step before a difference
counts."""
import random

import numpy as np
import pytest

from helpers import host_tensor, oracle_run
from nx_b200 import nx
from nx_b200.grad import grad

DIMS = [1, 2, 3, 4, 5]
UNARY = ["exp", "tanh", "sigmoid", "cos", "sin", "negate", "sqrt_abs", "log1p_abs", "square", "abs"]
KINDS = ["unary", "binary", "binary", "reduce", "reshape", "transpose", "broadcast", "slice", "pad", "reverse", "concat",
         "select", "dot", "softmax", "take", "put_slice", "window", "clip", "logsumexp", "stack", "mean", "max_reduce", "squeeze",
         "sort", "take_along", "dynslice", "scatter", "product", "invtrig", "remainder"]


def bc(a, b):
    try:
        np.broadcast_shapes(a, b)
        return True
    except ValueError:
        return False


def apply(r, kind, x, vals):
    if kind == "unary":
        op = r.choice(UNARY)
        if op == "sqrt_abs":
            return nx.sqrt(nx.abs(x) + 0.5)
        if op == "log1p_abs":
            return nx.log1p(nx.abs(x))
        if op == "square":
            return x * x
        return getattr(nx, op)(x)
    if kind == "binary":
        cands = [v for v in vals if bc(v.shape, x.shape)]
        other = r.choice(cands) if cands and r.random() < 0.8 else r.choice([2.0, 0.5, 3.0])
        op = r.choice(["add", "subtract", "multiply", "divide_safe", "max", "min", "pow2", "atan2"])
        if op == "divide_safe":
            return x / (nx.abs(other) + 1.0) if not isinstance(other, float) else x / other
        if op == "pow2":
            return nx.pow(nx.abs(x) + 0.5, 1.5)
        return getattr(nx, op)(x, other)
    if kind == "select":
        cands = [v for v in vals if v.shape == x.shape]
        return nx.select(nx.greater(x, 0.1), r.choice(cands), r.choice(cands))
    if kind == "clip":
        return nx.clip(x, -0.7, 0.9)
    if kind == "invtrig":
        op = r.choice(["asin", "acos", "atanh", "asinh", "acosh", "erf_inv", "atan"])
        if op in ("asin", "acos", "atanh", "erf_inv"):
            return getattr(nx, op)(nx.tanh(x) * 0.9)
        if op == "acosh":
            return nx.acosh(nx.abs(x) + 1.5)
        return getattr(nx, op)(x)
    if kind == "remainder":
        return nx.remainder(x, r.choice([0.7, 1.3, 2.9]))
    if kind == "as_type":
        return nx.as_type(nx.as_type(x, "f32"), "f64")
    if kind == "reshape":
        n = int(np.prod(x.shape)) if x.rank else 1
        return nx.reshape(x, r.choice([(n,), (1, n), (n, 1)] + [(d, n // d) for d in (2, 3, 4) if n % d == 0]))
    if kind == "broadcast":
        return None if x.rank >= 3 else nx.broadcast(x, (r.choice([2, 3]),) + tuple(x.shape))
    if kind == "stack":
        cands = [v for v in vals if v.shape == x.shape]
        return nx.stack([x, r.choice(cands)], axis=r.randint(0, x.rank))
    if kind == "squeeze":
        ones = [i for i, d in enumerate(x.shape) if d == 1]
        return nx.squeeze(x, [r.choice(ones)]) if ones else None
    if kind == "dot":
        cands = [v for v in vals if v.rank == 2 and x.rank == 2 and v.shape[0] == x.shape[1]]
        return nx.dot(x, r.choice(cands)) if cands else None
    if x.rank == 0:
        return None
    last = x.rank - 1
    if kind == "reduce":
        axes = sorted(r.sample(range(x.rank), r.randint(1, x.rank)))
        return nx.sum(x, axes=axes, keep_axes=r.random() < 0.5)
    if kind == "product":
        return nx.product(x, axes=[r.randrange(x.rank)], keep_axes=r.random() < 0.5)
    if kind == "mean":
        return nx.mean(x, axes=[r.randrange(x.rank)])
    if kind == "max_reduce":
        return getattr(nx, r.choice(["reduce_max", "reduce_min"]))(x, axes=[r.randrange(x.rank)], keep_axes=r.random() < 0.5)
    if kind == "transpose":
        if x.rank < 2:
            return None
        perm = list(range(x.rank))
        r.shuffle(perm)
        return nx.transpose(x, axes=perm)
    if kind == "slice":
        starts = [r.randrange(d) for d in x.shape]
        lengths = [r.randint(1, d - s) for d, s in zip(x.shape, starts)]
        return nx.slice(x, starts, lengths, strides=[r.choice([1, 1, 2]) for _ in x.shape])
    if kind == "pad":
        return nx.pad(x, 0.0, [(r.randint(-1 if d > 2 else 0, 2), r.randint(0, 2), r.choice([0, 0, 1])) for d in x.shape])
    if kind == "reverse":
        return nx.reverse(x, axes=[r.randrange(x.rank)])
    if kind == "concat":
        ax = r.randrange(x.rank)
        cands = [v for v in vals if v.rank == x.rank and all(i == ax or a == b for i, (a, b) in enumerate(zip(v.shape, x.shape)))]
        return nx.concatenate([x, r.choice(cands)], axis=ax)
    if kind == "softmax":
        e = nx.exp(x - nx.reduce_max(x, axes=[last], keep_axes=True))
        return e / nx.sum(e, axes=[last], keep_axes=True)
    if kind == "logsumexp":
        return nx.logsumexp(x, axes=[last])
    if kind == "take":
        ax = r.randrange(x.rank)
        idx = nx.remainder(nx.iota((r.choice([1, 3, 4]),), type="s32") * 3, x.shape[ax])
        return nx.take(x, idx, axis=ax)
    if kind == "take_along":
        ax = r.randrange(x.rank)
        idx = nx.remainder(nx.iota(x.shape, axis=ax, type="s32") * 2 + 1, x.shape[ax])
        return nx.take_along_axis(x, idx, axis=ax)
    if kind == "put_slice":
        cands = [v for v in vals if v.rank == x.rank and all(a <= b for a, b in zip(v.shape, x.shape))]
        if not cands:
            return None
        piece = r.choice(cands)
        starts = [r.randrange(d - n + 1) for d, n in zip(x.shape, piece.shape)]
        return nx.put_slice(x, starts, piece)
    if kind == "dynslice":
        lengths = [r.randint(1, d) for d in x.shape]
        start = nx.as_type(nx.sum(nx.iota((2,), type="s32")), "s32")
        return nx.slice(x, [start] + [0] * (x.rank - 1), lengths)
    if kind == "window":
        if x.rank > 2:
            return None
        win = tuple(r.randint(1, min(2, d)) for d in x.shape)
        return nx.window_sum(x, win, strides=r.choice([1, 2]), padding=r.choice(["valid", "same"]))
    if kind == "sort":
        return nx.sort(x, axis=last, direction=r.choice(["asc", "desc"]))
    if kind == "scatter":
        if x.rank != 1:
            return None
        k = r.choice([1, 3])
        idx = nx.reshape(nx.remainder(nx.iota((k,), type="s32") * 2, x.shape[0]), (k, 1))
        cands = [v for v in vals if v.shape == (k,)]
        upd = r.choice(cands) if cands else nx.broadcast(nx.as_type(2.0, "f64"), (k,))
        scatter = r.choice([nx.indexed_add, nx.indexed_put])
        if scatter is nx.indexed_put and len({(2 * j) % x.shape[0] for j in range(k)}) < k:
            scatter = nx.indexed_add                  # two writes to one place: which one stays is not specified
        return scatter(x, idx, upd)
    raise AssertionError(kind)


def make(seed):
    rng = random.Random(seed)
    n_args = rng.randint(1, 2)
    shapes = [tuple(rng.choice(DIMS) for _ in range(rng.choice([1, 2, 2, 3]))) for _ in range(n_args)]
    data = np.random.default_rng(seed)
    arrays = [data.standard_normal(s) * 1.3 for s in shapes]
    op_seed = seed * 104729 + 7
    steps = rng.randint(2, 10)
    log = []

    def fun(*tensors):
        r = random.Random(op_seed)
        vals = list(tensors)
        del log[:]
        for _ in range(steps):
            kind = r.choice(KINDS)
            x = r.choice(vals)
            try:
                y = apply(r, kind, x, vals)
            except (ValueError, TypeError):
                continue                      # the front-end refused the combination
            if y is not None and int(np.prod(y.shape)) <= 4096:
                log.append((kind, vals.index(x), x.shape, y.shape))
                vals.append(y)
        out = vals[-1]
        # a weighted sum so that every element matters differently
        w = nx.cos(nx.as_type(nx.iota((int(np.prod(out.shape)) or 1,), type="s32"), "f64") * 0.37) + 1.5
        return nx.sum(nx.reshape(out, (int(np.prod(out.shape)) or 1,)) * w)

    return fun, arrays, log


def run(fun, arrays):
    host = [host_tensor(a, "f64") for a in arrays]
    blob, res = oracle_run(fun, host)
    return [np.asarray(r[0], dtype=np.float64) for r in res]


def fd(fun, arrays, wrt, eps=1e-6):
    base = [np.asarray(a, dtype=np.float64) for a in arrays]
    out = np.zeros_like(base[wrt])
    it = np.nditer(base[wrt], flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        hi = [b.copy() for b in base]
        lo = [b.copy() for b in base]
        hi[wrt][i] += eps
        lo[wrt][i] -= eps
        out[i] = (run(fun, hi)[0] - run(fun, lo)[0]) / (2 * eps)
    return out


@pytest.mark.parametrize("seed", range(200))
def test_gradient_of_a_random_composition_matches_finite_differences(seed):
    fun, arrays, log = make(seed)
    with np.errstate(all="ignore"):
        for wrt in range(len(arrays)):
            got = run(lambda *xs: grad(fun, wrt)(*xs), arrays)[0]
            want = fd(fun, arrays, wrt)
            ok = (np.abs(got - want) <= 2e-4 * (1 + np.abs(want))) | ~np.isfinite(want)
            if not np.all(ok):
                want = fd(fun, arrays, wrt, eps=1e-7)
                ok = (np.abs(got - want) <= 2e-3 * (1 + np.abs(want))) | ~np.isfinite(want)
            assert np.all(ok), (wrt, [step[0] for step in log], got, want)
