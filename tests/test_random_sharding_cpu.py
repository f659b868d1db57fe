"""Random programs over randomly split arguments: the partitioner's per-partition programs, interpreted by
the oracle (one thread per partition; an `all_reduce` node sums over the partitions that differ only in its
mesh axis), stitched by the result shardings it reports, must equal the oracle's evaluation of the global
program — or the partitioner must refuse with `ShardingError` (anything that would need another
collective).  Meshes {2}, {4} and {2,2}.

`ONCE_WRONG`: seeds whose result was split twice over one mesh axis (`x + transpose(x)` with x split by
rows and the like): every partition computed a diagonal block and the stitched result was wrong; the
partitioner now refuses them."""
import random
import threading

import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import defn, nx, sharding

DIMS = [2, 4, 6, 8]
KINDS = ["unary", "binary", "binary", "reduce", "reshape", "transpose", "broadcast", "slice", "pad", "reverse", "concat",
         "select", "dot", "dot", "softmax", "iota", "clip", "logsumexp", "max_reduce", "argmax", "as_type", "take", "stack", "squeeze"]


def bc(a, b):
    try:
        np.broadcast_shapes(a, b)
        return True
    except ValueError:
        return False


def apply(r, kind, x, vals):
    if kind == "unary":
        return getattr(nx, r.choice(["exp", "tanh", "negate", "abs", "sigmoid", "cos"]))(x)
    if kind == "binary":
        cands = [v for v in vals if bc(v.shape, x.shape)]
        other = r.choice(cands) if cands and r.random() < 0.8 else r.choice([2.0, 0.5])
        return getattr(nx, r.choice(["add", "subtract", "multiply", "max", "min"]))(x, other)
    if kind == "select":
        cands = [v for v in vals if v.shape == x.shape]
        return nx.select(nx.greater(x, 0.1), r.choice(cands), r.choice(cands))
    if kind == "clip":
        return nx.clip(x, -0.7, 0.9)
    if kind == "as_type":
        return nx.as_type(x, r.choice(["f32", "f64"]))
    if kind == "reshape":
        n = int(np.prod(x.shape)) if x.rank else 1
        return nx.reshape(x, r.choice([(n,), (1, n), (n, 1)] + [(d, n // d) for d in (2, 3, 4) if n % d == 0]))
    if kind == "broadcast":
        return None if x.rank >= 3 else nx.broadcast(x, (r.choice([2, 4]),) + tuple(x.shape))
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
    if kind == "max_reduce":
        return getattr(nx, r.choice(["reduce_max", "reduce_min"]))(x, axes=[r.randrange(x.rank)], keep_axes=r.random() < 0.5)
    if kind == "argmax":
        return nx.as_type(nx.argmax(x, axis=r.randrange(x.rank)), "f32")
    if kind == "transpose":
        if x.rank < 2:
            return None
        perm = list(range(x.rank))
        r.shuffle(perm)
        return nx.transpose(x, axes=perm)
    if kind == "slice":
        starts = [r.randrange(d) for d in x.shape]
        lengths = [r.randint(1, d - s) for d, s in zip(x.shape, starts)]
        return nx.slice(x, starts, lengths)
    if kind == "pad":
        return nx.pad(x, 0.0, [(r.randint(0, 1), r.randint(0, 1), 0) for d in x.shape])
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
    if kind == "iota":
        return x + nx.as_type(nx.iota(x.shape, axis=r.randrange(x.rank), type="s32"), x.type)
    if kind == "take":
        ax = r.randrange(x.rank)
        idx = nx.remainder(nx.iota((r.choice([1, 2, 4]),), type="s32") * 3, x.shape[ax])
        return nx.take(x, idx, axis=ax)
    raise AssertionError(kind)


def make(seed):
    rng = random.Random(seed)
    mesh_shape = rng.choice([(2,), (2,), (4,), (2, 2)])
    mesh = sharding.Mesh("m", mesh_shape)
    n_args = rng.randint(1, 3)
    shapes = [tuple(rng.choice(DIMS) for _ in range(rng.choice([1, 2, 2, 3]))) for _ in range(n_args)]
    # matching shapes for dot: make arg1 {k, n} for arg0 {m, k} sometimes
    if n_args >= 2 and len(shapes[0]) == 2 and rng.random() < 0.6:
        shapes[1] = (shapes[0][1], rng.choice(DIMS))
        if n_args == 3 and rng.random() < 0.6:
            shapes[2] = (shapes[1][1], rng.choice(DIMS))
    shardings = []
    for s in shapes:
        sh = {}
        free_axes = list(range(len(mesh_shape)))
        for dim in range(len(s)):
            if free_axes and rng.random() < 0.4:
                a = rng.choice(free_axes)
                if s[dim] % mesh_shape[a] == 0:
                    sh[dim] = [a]
                    free_axes.remove(a)
        shardings.append(sh)
    data = np.random.default_rng(seed)
    arrays = [data.standard_normal(s).astype(np.float32) for s in shapes]
    op_seed = seed * 31337 + 5
    steps = rng.randint(1, 8)
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
                continue
            if y is not None and int(np.prod(y.shape)) <= 4096:
                log.append((kind, vals.index(x), x.shape, y.shape))
                vals.append(y)
        k = min(len(vals) - len(tensors), 2)
        return tuple(vals[-k:]) if k else (tensors[0] + 1.0,)

    return mesh, shardings, arrays, fun, log


def local_slice(a, sh, mesh, coords):
    for dim, axes in sh.items():
        ax = axes[0]
        n = a.shape[dim] // mesh.shape[ax]
        a = np.take(a, range(coords[ax] * n, (coords[ax] + 1) * n), axis=dim)
    return np.ascontiguousarray(a)


def run_case(seed):
    mesh, shardings, arrays, fun, log = make(seed)
    host = [host_tensor(a, "f32") for a in arrays]
    blob, _ = defn.build_program(fun, host)
    with np.errstate(all="ignore"):
        full = [np.asarray(r[0]) for r in O.run_program(blob, [h.data.raw for h in host], "xla_like")]
    P = mesh.size
    progs = []
    for p in range(P):
        coords = mesh.coords(p)
        local = [host_tensor(local_slice(a, sh, mesh, coords), "f32") for a, sh in zip(arrays, shardings)]
        pblob, _, out_specs = sharding.partition(fun, mesh, shardings, local, p)
        progs.append((pblob, local, out_specs, coords))
    # run the partitions in threads so that all_reduce can meet
    results = [None] * P
    errors = []
    lock = threading.Lock()
    barrier = threading.Barrier(P)
    pending = {}

    def worker(p):
        pblob, local, out_specs, coords = progs[p]
        calls = [0]

        def all_reduce(arr, axis):
            # group = partitions that differ only in mesh coordinate `axis`
            key = (calls[0], tuple(c for i, c in enumerate(coords) if i != axis))
            calls[0] += 1
            with lock:
                pending.setdefault(key, []).append(np.array(arr, copy=True))
            barrier.wait()
            with lock:
                total = sum(pending[key][1:], pending[key][0].copy())
            barrier.wait()
            return total.astype(arr.dtype)

        try:
            with np.errstate(all="ignore"):
                results[p] = [np.asarray(r[0]) for r in O.run_program(pblob, [h.data.raw for h in local], "xla_like", all_reduce=all_reduce)]
        except Exception as e:
            errors.append(e)
            barrier.abort()
    ts = [threading.Thread(target=worker, args=(p,)) for p in range(P)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    if errors:
        raise errors[0]
    # stitch
    for oi, want in enumerate(full):
        spec = progs[0][2][oi]
        got = np.zeros_like(want)
        for p in range(P):
            coords = progs[p][3]
            part = results[p][oi]
            idx = []
            for dim, a in enumerate(spec):
                if a is None:
                    idx.append(slice(None))
                else:
                    n = want.shape[dim] // mesh.shape[a]
                    idx.append(slice(coords[a] * n, (coords[a] + 1) * n))
            if part.shape != got[tuple(idx)].shape:
                raise AssertionError(f"shape of partition {p} output {oi}: {part.shape} vs {got[tuple(idx)].shape} spec {spec}")
            got[tuple(idx)] = part
        if not np.allclose(got, want, rtol=2e-5, atol=1e-5, equal_nan=True):
            raise AssertionError(f"output {oi} differs: max {np.nanmax(np.abs(got - want))} spec {spec}")
    return log


ONCE_WRONG = [708, 1101, 1693, 1802, 2709, 2869, 2977]


@pytest.mark.parametrize("seed", sorted(set(range(500)) | set(ONCE_WRONG)))
def test_partitions_of_a_random_program_stitch_to_the_global_result(seed):
    try:
        run_case(seed)
    except sharding.ShardingError:
        pass                                   # refused: the pattern needs a collective the partitioner does not insert


def test_one_mesh_axis_cannot_split_two_dimensions_of_a_result():
    mesh = sharding.Mesh("m", (2,))
    x = defn.template((4, 8), "f32")           # local shape of an {8,8} tensor split by rows
    with pytest.raises(sharding.ShardingError, match="two dimensions"):
        sharding.partition(lambda t: t + nx.transpose(t), mesh, [{0: [0]}], [x], 0)
    for seed in ONCE_WRONG:
        with pytest.raises(sharding.ShardingError):
            run_case(seed)
