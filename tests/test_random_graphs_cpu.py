"""Random graphs of the supported operations must trace, plan, generate and compile (no GPU needed),
and the oracle must be able to interpret the same bytes.  The generator draws shapes around the
vector / warp / row boundaries and mixes element-wise operations, reductions, shape operations,
lookups, window reductions, sorts, scatters and products.

Seeds in `ONCE_REJECTED` produced fused row kernels the runtime compiler rejected (a `put_slice`, or a
slice at a computed position, applied to the result of a reduction of the same kernel); such graphs are
planned again with one kernel per materialised value (`NXB200_NO_REPLAN=1` shows the rejected kernel)."""
import random

import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import defn, nx

DIMS = [1, 2, 3, 4, 5, 8, 16, 17, 32, 33, 64, 128, 256, 1000]
TYPES = ["f32", "bf16", "s32", "u8", "f16", "s64"]
UNARY = ["exp", "tanh", "negate", "abs", "sigmoid", "sqrt", "floor", "sign", "log1p", "cos"]
BINARY = ["add", "subtract", "multiply", "max", "min", "divide", "greater", "equal", "less_equal"]
REDUCE = ["sum", "reduce_max", "reduce_min", "product"]
KINDS = ["unary", "binary", "binary", "reduce", "reshape", "transpose", "broadcast", "slice", "pad", "reverse", "concat",
         "select", "as_type", "argmax", "dot", "iota", "softmax", "squeeze", "take", "put_slice", "window", "sort",
         "clip", "logsumexp", "intop", "scatter", "dynslice", "stack"]
ONCE_REJECTED = [92, 284, 311, 412, 664, 815, 855, 993, 1191, 1227, 1278, 1385, 1482]


def _broadcastable(a, b):
    try:
        np.broadcast_shapes(a, b)
        return True
    except ValueError:
        return False


def _apply(r, kind, x, vals):
    """One random operation on `x` (other operands drawn from `vals`); None when it does not apply."""
    if kind == "unary":
        return getattr(nx, r.choice(UNARY))(x)
    if kind == "binary":
        cands = [v for v in vals if _broadcastable(v.shape, x.shape)]
        other = r.choice(cands) if cands and r.random() < 0.8 else r.choice([2, 0.5, 3])
        return getattr(nx, r.choice(BINARY))(x, other)
    if kind == "as_type":
        return nx.as_type(x, r.choice(TYPES))
    if kind == "clip":
        return nx.clip(x, -1, 1)
    if kind == "select":
        cands = [v for v in vals if v.shape == x.shape]
        return nx.select(nx.greater(x, 0), r.choice(cands), r.choice(cands))
    if kind == "intop":
        xi = nx.as_type(x, r.choice(["s32", "u8", "s64"]))
        op = r.choice(["bitwise_and", "bitwise_or", "bitwise_xor", "left_shift", "right_shift", "remainder", "quotient"])
        return getattr(nx, op)(xi, r.choice([1, 3, 5]))
    if kind == "reshape":
        n = int(np.prod(x.shape)) if x.rank else 1
        return nx.reshape(x, r.choice([(n,), (1, n), (n, 1)] + [(d, n // d) for d in (2, 3, 4, 8) if n % d == 0]))
    if kind == "broadcast":
        return None if x.rank >= 3 else nx.broadcast(x, (r.choice([2, 3, 4]),) + tuple(x.shape))
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
        return getattr(nx, r.choice(REDUCE))(x, axes=axes, keep_axes=r.random() < 0.5)
    if kind == "argmax":
        return getattr(nx, r.choice(["argmax", "argmin"]))(x, axis=r.randrange(x.rank), keep_axis=r.random() < 0.3)
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
        return nx.pad(x, 0, [(r.randint(0, 2), r.randint(0, 2), r.choice([0, 0, 1])) for _ in x.shape])
    if kind == "reverse":
        return nx.reverse(x, axes=[r.randrange(x.rank)])
    if kind == "concat":
        ax = r.randrange(x.rank)
        cands = [v for v in vals if v.rank == x.rank and all(i == ax or a == b for i, (a, b) in enumerate(zip(v.shape, x.shape)))]
        return nx.concatenate([x, r.choice(cands)], axis=ax)
    if kind == "iota":
        return nx.add(x, nx.iota(x.shape, axis=r.randrange(x.rank), type="s32"))
    if kind == "softmax":
        xf = nx.as_type(x, "f32")
        e = nx.exp(xf - nx.reduce_max(xf, axes=[last], keep_axes=True))
        return e / nx.sum(e, axes=[last], keep_axes=True)
    if kind == "logsumexp":
        return nx.logsumexp(nx.as_type(x, "f32"), axes=[last])
    if kind == "take":
        ax = r.randrange(x.rank)
        idx = nx.as_type(nx.abs(nx.iota((r.choice([1, 3, 7]),), type="s32") * 3), "s32")
        return nx.take(x, nx.remainder(idx, x.shape[ax]), axis=ax)
    if kind == "put_slice":
        lengths = [r.randint(1, d) for d in x.shape]
        starts = [r.randrange(d - n + 1) for d, n in zip(x.shape, lengths)]
        return nx.put_slice(x, starts, nx.broadcast(nx.as_type(7, x.type), tuple(lengths)))
    if kind == "dynslice":
        lengths = [r.randint(1, d) for d in x.shape]
        start = nx.as_type(nx.sum(nx.iota((3,), type="s32")), "s32")
        return nx.slice(x, [start] + [0] * (x.rank - 1), lengths)
    if kind == "window":
        if x.rank > 2:
            return None
        win = tuple(r.randint(1, min(3, d)) for d in x.shape)
        op = r.choice(["window_sum", "window_max", "window_min"])
        return getattr(nx, op)(x, win, strides=r.choice([1, 2]), padding=r.choice(["valid", "same"]))
    if kind == "sort":
        return r.choice([nx.sort, nx.argsort])(x, axis=last, direction=r.choice(["asc", "desc"]))
    if kind == "scatter":
        if x.rank != 1:
            return None
        k = r.choice([1, 4])
        idx = nx.reshape(nx.remainder(nx.iota((k,), type="s32") * 5, x.shape[0]), (k, 1))
        return r.choice([nx.indexed_add, nx.indexed_put])(x, idx, nx.broadcast(nx.as_type(2, x.type), (k,)))
    raise AssertionError(kind)


def random_program(seed):
    """(program bytes, host arguments) of a random function of one to three tensors."""
    rng = random.Random(seed)
    n_args = rng.randint(1, 3)
    specs = [(tuple(rng.choice(DIMS) for _ in range(rng.choice([1, 2, 2, 3]))), rng.choice(TYPES)) for _ in range(n_args)]
    data = np.random.default_rng(seed)
    args = []
    for shape, ty in specs:
        if ty in ("f32", "bf16", "f16"):
            value = data.standard_normal(shape)
        elif ty == "u8":
            value = data.integers(0, 200, shape)
        else:
            value = data.integers(-50, 50, shape)
        args.append(host_tensor(value, ty))
    op_seed = seed * 7919 + 13
    steps = rng.randint(2, 16)

    def fun(*tensors):
        r = random.Random(op_seed)
        vals = list(tensors)
        for _ in range(steps):
            kind = r.choice(KINDS)
            x = r.choice(vals)
            try:
                y = _apply(r, kind, x, vals)
            except (ValueError, TypeError):
                continue                      # the front-end refused the combination (as the reference's would)
            if y is not None and int(np.prod(y.shape)) <= 1 << 20:
                vals.append(y)
        made = vals[len(tensors):]
        return tuple(r.sample(made, min(len(made), r.randint(1, 3)))) if made else (tensors[0] + 1,)

    blob, _ = defn.build_program(fun, args)
    return blob, args


@pytest.mark.parametrize("seed", sorted(set(range(120)) | set(ONCE_REJECTED)))
def test_random_graph_compiles_and_the_oracle_interprets_it(seed):
    blob, args = random_program(seed)
    prog = defn.Program(blob)
    assert prog.launch_count() >= 1
    with np.errstate(all="ignore"):
        results = O.run_program(blob, [a.data.raw for a in args], "xla_like")
    assert len(results) == prog.n_outputs


def test_a_window_update_of_a_reduction_result_gets_a_kernel_of_its_own():
    """`put_slice` on the result of a reduction cannot live in the reduction's row kernel (its value
    depends on the position along the reduced tensor's remaining axes); the plan is two kernels."""
    x = host_tensor(np.random.default_rng(0).standard_normal((33, 17)), "f32")
    piece = lambda: nx.broadcast(nx.as_type(7.0, "f32"), (5,))
    cases = [(lambda t: nx.put_slice(nx.sum(t, axes=[1]), [3], piece()), 7.0),
             (lambda t: nx.exp(nx.put_slice(nx.sum(t, axes=[1]), [3], piece())), float(np.exp(np.float32(7.0)))),
             (lambda t: nx.put_slice(nx.as_type(nx.argmax(t, axis=1), "f32"), [3], piece()), 7.0)]
    for fun, inside in cases:
        blob, _ = defn.build_program(fun, [x])
        prog = defn.Program(blob)
        assert prog.launch_count() == 2, prog.describe()
        value, _type, _raw = O.run_program(blob, [x.data.raw], "xla_like")[0]
        value = np.asarray(value, dtype=np.float64)
        assert value.shape == (33,)
        np.testing.assert_allclose(value[3:8], inside, rtol=1e-6)
