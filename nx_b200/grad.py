"""Reverse-mode differentiation over the traced graph: the host-side mirror of ``Nx.Defn.Grad``
(nx/lib/nx/defn/grad.ex).  The gradient is built as ordinary graph nodes, so the compiler sees
nothing new: backward products arrive as `dot` with other contracted axes (served by the
MN-major operand path of the tensor-core kernel), un-broadcasting as `sum`, and so on.

Rules follow the reference's (file:line quoted per rule).  Lookups differentiate into scatters:
gather / take / take_along_axis into `indexed_add`, a slice at computed positions into `put_slice`,
and the scatters back into gathers.  Not differentiable here (raises): window max / min / product
(the reference scatters through `window_scatter_max/min`, which the device lacks) and loops.  An
integer-valued node (`quotient`, comparisons, `argmax` …) carries no gradient: the walk stops there,
where the reference raises for `quotient`.
"""
from . import backend as B
from . import expr as E
from . import nx
from . import types as T
from .nx import Tensor


def _unbroadcast(x, res, ans_shape):
    """grad.ex:1698-1745: the gradient of an operand that was broadcast to `ans_shape`."""
    if x.shape == tuple(ans_shape):
        return res
    res = nx.broadcast(res, ans_shape) if res.shape != tuple(ans_shape) else res
    lead = len(ans_shape) - x.rank
    axes = list(range(lead)) + [lead + i for i, d in enumerate(x.shape) if d == 1 and ans_shape[lead + i] != 1]
    out = nx.sum(res, axes=axes) if axes else res
    return nx.reshape(out, x.shape)


def _reduce_g(x, ints, g):
    """grad.ex:1811-1822: spread the gradient of a reduction back over the reduced axes."""
    keep, n = ints[0], ints[1]
    if keep:
        return nx.broadcast(g, x.shape)                       # unit axes are still in place
    axes = list(ints[2:2 + n]) or list(range(x.rank))
    return nx.broadcast(g, x.shape, axes=[i for i in range(x.rank) if i not in axes])


def _dot_axes(ints):
    it = iter(ints)
    out = []
    for _ in range(4):
        k = next(it)
        out.append([next(it) for _ in range(k)])
    return out


def _argsort(xs):
    return sorted(range(len(xs)), key=lambda i: xs[i])


def _rule(t, g):
    """Contributions ``[(operand tensor, gradient)]`` of node `t` given the gradient `g` of its result."""
    e = t.data
    op, a = e.op, e.args
    if op in ("parameter", "constant", "tensor", "iota", "metadata"):
        return []                                                        # leaves; metadata = stop_grad (nx.ex:18407-18414)
    if op == "io_call":
        return [(a[0], g)]                                               # grad_test.exs:72-86: a tap is transparent
    if not T.is_float(t.type):
        return []                                                        # integer / predicate results carry no gradient
    ans = t
    if op == "add":                                                      # grad.ex:990-996
        if a[0].data.id == a[1].data.id:
            return [(a[0], g * 2.0)]
        return [(a[0], _unbroadcast(a[0], g, ans.shape)), (a[1], _unbroadcast(a[1], g, ans.shape))]
    if op == "subtract":                                                 # :998-1000
        return [(a[0], _unbroadcast(a[0], g, ans.shape)), (a[1], _unbroadcast(a[1], nx.negate(g), ans.shape))]
    if op == "multiply":                                                 # :1002-1011
        if a[0].data.id == a[1].data.id:
            return [(a[0], g * (a[0] * 2.0))]
        return [(a[0], _unbroadcast(a[0], g * a[1], ans.shape)), (a[1], _unbroadcast(a[1], g * a[0], ans.shape))]
    if op == "divide":                                                   # :1013-1018
        return [(a[0], _unbroadcast(a[0], g / a[1], ans.shape)),
                (a[1], _unbroadcast(a[1], g * nx.negate(ans / a[1]), ans.shape))]
    if op == "pow":                                                      # :1027-1046
        x, y = a
        gx = g * y * nx.pow(x, y - 1.0)
        gy = g * ans * nx.log(nx.select(nx.equal(x, 0.0), 1.0, x))
        return [(x, _unbroadcast(x, gx, ans.shape)), (y, _unbroadcast(y, gy, ans.shape))]
    if op == "atan2":                                                    # :1048-1055
        x, y = a
        den = x * x + y * y
        return [(x, _unbroadcast(x, g * (y / den), ans.shape)), (y, _unbroadcast(y, g * nx.negate(x / den), ans.shape))]
    if op == "remainder":                                                # :1020-1025
        x, y = a
        return [(x, _unbroadcast(x, g, ans.shape)), (y, _unbroadcast(y, g * nx.negate(nx.floor(x / y)), ans.shape))]
    if op in ("max", "min"):                                             # :1057-1075
        x, y = a
        lhs = nx.select(nx.equal(x, ans), 1.0, 0.0) / nx.select(nx.equal(y, ans), 2.0, 1.0)
        rhs = nx.select(nx.equal(y, ans), 1.0, 0.0) / nx.select(nx.equal(x, ans), 2.0, 1.0)
        return [(x, _unbroadcast(x, g * lhs, ans.shape)), (y, _unbroadcast(y, g * rhs, ans.shape))]
    if op == "select":                                                   # :675-683
        p, x, y = a
        return [(x, _unbroadcast(x, nx.select(p, g, 0.0), ans.shape)), (y, _unbroadcast(y, nx.select(p, 0.0, g), ans.shape))]
    if op == "clip":                                                     # :689-716 (operand only: the limits are constants here)
        x, lo, hi = a
        inside = nx.logical_and(nx.greater_equal(x, lo), nx.less_equal(x, hi))
        return [(x, nx.select(inside, g, 0.0))]
    unary = {
        "negate": lambda x: nx.negate(g),                                # :1166
        "exp": lambda x: g * ans,                                        # :1139
        "expm1": lambda x: g * (ans + 1.0),                              # :1143
        "log": lambda x: g / x,                                          # :1147
        "log1p": lambda x: g / (x + 1.0),                                # :1151
        "sigmoid": lambda x: g * ans * (1.0 - ans),                      # :1155-1164
        "tanh": lambda x: g * (1.0 - ans * ans),                         # :1219-1224
        "sqrt": lambda x: g / (ans * 2.0),                               # :1131
        "rsqrt": lambda x: g * -0.5 * ans / x,                           # :1170
        "cbrt": lambda x: g / (ans * ans * 3.0),                         # :1135
        "sin": lambda x: g * nx.cos(x),                                  # :1174
        "cos": lambda x: g * nx.negate(nx.sin(x)),                       # :1198
        "tan": lambda x: g * (1.0 + ans * ans),                          # :1210
        "sinh": lambda x: g * nx.cosh(x),
        "cosh": lambda x: g * nx.sinh(x),
        "atan": lambda x: g / (1.0 + x * x),
        "asin": lambda x: g * nx.rsqrt(1.0 - x * x),                     # :1178
        "acos": lambda x: g * nx.negate(nx.rsqrt(1.0 - x * x)),          # :1202
        "asinh": lambda x: g * nx.rsqrt(x * x + 1.0),                    # :1186
        "acosh": lambda x: g * nx.rsqrt(x * x - 1.0),                    # :1190
        "atanh": lambda x: g / (1.0 - x * x),                            # :1194
        "erf_inv": lambda x: g * (nx.exp(ans * ans) * 0.886226925452758),        # :1248-1251  (sqrt(pi) / 2)
        "abs": lambda x: g * nx.select(nx.greater_equal(x, 0.0), 1.0, -1.0),     # :1127
        "erf": lambda x: g * nx.exp(nx.negate(x * x)) * 1.1283791670955126,      # :1226-1235  (2 / sqrt(pi))
        "erfc": lambda x: g * nx.exp(nx.negate(x * x)) * -1.1283791670955126,
    }
    if op in unary:
        return [(a[0], unary[op](a[0]))]
    if op in ("floor", "ceil", "round", "sign"):
        return []                                                        # piecewise constant
    if op == "as_type":                                                  # :1088
        return [(a[0], nx.as_type(g, a[0].type))] if T.is_float(a[0].type) else []
    if op in ("reshape", "squeeze"):                                     # :718-732
        return [(a[0], nx.reshape(g, a[0].shape))]
    if op == "broadcast":                                                # :685-687, 1732-1760
        x = a[0]
        n = e.ints[0]
        axes = list(e.ints[1:1 + n])
        summed = [i for i in range(ans.rank) if i not in axes]
        implicit = [ax for i, ax in enumerate(axes) if x.shape[i] == 1 and ans.shape[ax] != 1]
        gx = nx.sum(g, axes=sorted(summed + implicit)) if summed or implicit else g
        return [(x, nx.reshape(gx, x.shape))]
    if op == "transpose":                                                # :734-736
        return [(a[0], nx.transpose(g, _argsort(list(e.ints))))]
    if op == "reverse":                                                  # :787-789
        return [(a[0], nx.reverse(g, axes=list(e.ints)))]
    if op == "slice":                                                    # :752-759: zeros around (and between) the taken elements
        x = a[0]
        if len(a) > 1:
            # starts computed at run time (:761-768): the gradient, spread over the strides, is put
            # back at the same position of a tensor of zeros
            r = x.rank
            sd = e.ints[2 * r:3 * r]
            spread = nx.pad(g, 0.0, [(0, 0, k - 1) for k in sd]) if any(k != 1 for k in sd) else g
            zeros = nx.broadcast(E.constant(x.type, (), 0.0), x.shape)
            return [(x, nx.put_slice(zeros, list(a[1:]), spread))]
        r = x.rank
        st, ln, sd = e.ints[:r], e.ints[r:2 * r], e.ints[2 * r:3 * r]
        cfg = []
        for d, s, l, k, o in zip(x.shape, st, ln, sd, ans.shape):
            covered = s + (o - 1) * k + 1
            cfg.append((s, d - covered, k - 1))
        return [(x, nx.pad(g, 0.0, cfg))]
    if op == "pad":                                                      # :738-750
        x, v = a
        r = x.rank
        lo, hi, it = e.ints[:r], e.ints[r:2 * r], e.ints[2 * r:3 * r]
        inner = nx.pad(g, 0.0, [(-l, -h, 0) for l, h in zip(lo, hi)])
        gx = nx.slice(inner, [0] * r, list(inner.shape), [i + 1 for i in it])
        gv = nx.sum(g) - nx.sum(gx)
        return [(x, gx), (v, gv)]
    if op == "put_slice":                                                # :770-777
        x, piece, starts = a[0], a[1], list(a[2:])
        out = []
        if T.is_float(x.type):
            out.append((x, nx.as_type(nx.put_slice(g, starts, nx.broadcast(E.constant(g.type, (), 0.0), piece.shape)), x.type)))
        if T.is_float(piece.type):
            out.append((piece, nx.as_type(nx.slice(g, starts, list(piece.shape)), piece.type)))
        return out
    if op == "gather":                                                   # :970-988: the lookups scatter their gradients back
        x, idx = a
        axes = list(e.ints)
        depth = idx.shape[-1]
        num = 1
        for d in idx.shape[:-1]:
            num *= d
        rest = [d for i, d in enumerate(x.shape) if i not in axes]
        zeros = nx.broadcast(E.constant(x.type, (), 0.0), x.shape)
        return [(x, nx.indexed_add(zeros, nx.reshape(idx, (num, depth)), nx.reshape(g, (num, *rest)), axes=axes))]
    if op in ("indexed_add", "indexed_put"):                             # :779-795
        target, idx, upd = a
        axes = list(e.ints)
        looked_up = nx.gather(g, idx, axes=axes)                         # {n} ++ the axes that are not indexed
        if looked_up.shape != upd.shape:                                 # a slice narrower than the target starts at 0
            looked_up = nx.slice(looked_up, [0] * upd.rank, list(upd.shape))
        out = [(upd, looked_up)]
        if op == "indexed_add":
            out.append((target, g))
        else:
            out.append((target, nx.indexed_put(g, idx, nx.broadcast(E.constant(g.type, (), 0.0), upd.shape), axes=axes)))
        return out
    if op == "sort":                                                     # :962-968 (the sorted axis is the last one here)
        x = a[0]
        last = x.rank - 1
        order = nx.argsort(x, axis=last, direction="desc" if e.ints[0] else "asc", stable=True)
        back = nx.argsort(order, axis=last, direction="asc", stable=True)
        return [(x, nx.take_along_axis(g, back, axis=last))]
    if op == "concatenate":                                              # :946-960
        axis = e.ints[0]
        out, off = [], 0
        for x in a:
            out.append((x, nx.as_type(nx.slice_along_axis(g, off, x.shape[axis], axis=axis), x.type) if T.is_float(x.type) else None))
            off += x.shape[axis]
        return [(x, gx) for x, gx in out if gx is not None]
    if op == "window_sum":                                               # :893-927
        x = a[0]
        r = x.rank
        win, st, lo, hi, dil = (list(e.ints[i * r:(i + 1) * r]) for i in range(5))
        span = [(w - 1) * d + 1 for w, d in zip(win, dil)]
        spread = [(o - 1) * s + 1 for o, s in zip(ans.shape, st)]
        before = [sp - l - 1 for sp, l in zip(span, lo)]
        after = [n + sp - 1 - od - b for n, sp, od, b in zip(x.shape, span, spread, before)]
        gp = nx.pad(g, 0.0, [(b, f, s - 1) for b, f, s in zip(before, after, st)])
        return [(x, nx.window_sum(gp, win, strides=[1] * r, padding=[(0, 0)] * r, window_dilations=dil))]
    if op == "sum":                                                      # :791-793
        return [(a[0], _reduce_g(a[0], e.ints, g))]
    if op == "product":                                                  # :795-826
        # the product without x_i is ans / x_i; with exactly one zero among the factors only that factor
        # has a gradient (the product of the others), with more than one nobody has
        x = a[0]
        n = e.ints[1]
        axes = list(e.ints[2:2 + n]) or list(range(x.rank))
        unit = [1 if i in axes else d for i, d in enumerate(x.shape)]
        gb, ansb = nx.reshape(g, unit), nx.reshape(ans, unit)
        zero = nx.equal(x, 0.0)
        without = nx.select(zero, 1.0, x)
        rest = nx.product(without, axes=axes, keep_axes=True)
        zeros = nx.sum(nx.as_type(zero, "s32"), axes=axes, keep_axes=True)
        dx = gb * (ansb / without)
        dx = nx.select(nx.logical_and(zero, nx.equal(zeros, 1)), gb * rest, dx)
        dx = nx.select(nx.logical_and(zero, nx.greater(zeros, 1)), 0.0, dx)
        return [(x, nx.as_type(dx, x.type))]
    if op in ("reduce_max", "reduce_min"):                               # :828-844
        x = a[0]
        keep, n = e.ints[0], e.ints[1]
        axes = list(e.ints[2:2 + n]) or list(range(x.rank))
        unit = [1 if i in axes else d for i, d in enumerate(x.shape)]
        gb = nx.broadcast(nx.reshape(g, unit), x.shape)
        locs = nx.as_type(nx.equal(x, nx.reshape(ans, unit)), x.type)
        den = nx.sum(locs, axes=axes, keep_axes=True)
        return [(x, gb * locs / den)]
    if op == "dot":                                                      # :845-871
        x, y = a[0], a[1]
        c1, b1, c2, b2 = _dot_axes(e.ints)
        nbx, nby = len(b1), len(b2)
        gr = ans.rank
        contract_gx = list(range(x.rank - len(c1), gr))
        contract_gy = list(range(nby, x.rank - len(c1)))
        free_x = [i for i in range(x.rank) if i not in c1 and i not in range(nbx)]
        free_y = [i for i in range(y.rank) if i not in c2 and i not in range(nby)]
        transpose_x = [c1[i] for i in _argsort(c2)]
        transpose_y = [c2[i] for i in _argsort(c1)]
        gx = nx.transpose(nx.dot(g, contract_gx, list(range(nbx)), y, free_y, b2), _argsort(b1 + free_x + transpose_x))
        gy = nx.transpose(nx.dot(g, contract_gy, list(range(nby)), x, free_x, b1), _argsort(b2 + free_y + transpose_y))
        return [(x, nx.as_type(gx, x.type)), (y, nx.as_type(gy, y.type))]
    raise NotImplementedError(f"gradient of :{op} is not implemented")


def _total(gs, like):
    g = gs[0]
    for more in gs[1:]:
        g = g + more
    if g.type != like.type:
        g = nx.as_type(g, like.type)
    return nx.broadcast(g, like.shape) if g.shape != like.shape else g


def _backward(y, wrt):
    """Gradients of the scalar `y` with respect to the nodes in `wrt` (zeros for the ones `y`
    does not depend on).  Only nodes between `wrt` and `y` are visited, as in grad.ex:95-150."""
    order = E.topo_order([y])[0]
    needed = {w.data.id for w in wrt}
    for t in order:
        if t.data.op != "metadata" and any(a.data.id in needed for a in t.data.args):
            needed.add(t.data.id)
    pending = {y.data.id: [E.constant(y.type, (), 1.0)]}
    final = {}
    for t in reversed(order):
        gs = pending.pop(t.data.id, None)
        if not gs or t.data.id not in needed:
            continue
        g = _total(gs, t)
        final[t.data.id] = g
        for operand, contribution in _rule(t, g):
            if operand.data.id in needed:
                pending.setdefault(operand.data.id, []).append(contribution)
    return [final[w.data.id] if w.data.id in final else nx.broadcast(E.constant(w.type, (), 0.0), w.shape) for w in wrt]


def value_and_grad(fun, argnums=0):
    """``Nx.Defn.value_and_grad/2``: a function returning ``(fun(*args), gradient)``; the gradient is
    taken with respect to the argument(s) `argnums` (an index or a tuple of indices; containers of
    tensors are differentiated leaf by leaf).  Works inside a traced defn and at the top level."""
    from . import defn

    def traced(*args):
        nums = (argnums,) if isinstance(argnums, int) else tuple(argnums)
        leaves, specs = [], []
        for i in nums:
            flat = []
            specs.append(defn._flatten(args[i], flat))
            leaves.append([B.to_expr(t) for t in flat])
        # differentiate with respect to exactly the nodes the function sees
        args = list(args)
        for i, sp, lv in zip(nums, specs, leaves):
            args[i] = defn._unflatten(sp, iter(lv))
        y = fun(*args)
        if not isinstance(y, Tensor) or y.shape != ():
            raise ValueError(f"expected the function to return a scalar tensor, got {getattr(y, 'shape', type(y))}")
        if not T.is_float(y.type):
            raise ValueError("can only compute the gradient of a floating-point result")
        gs = _backward(B.to_expr(y), [t for lv in leaves for t in lv])
        it = iter(gs)
        grads = [defn._unflatten(sp, it) for sp in specs]
        return y, (grads[0] if isinstance(argnums, int) else tuple(grads))

    def wrapped(*args):
        if defn._traced(args):
            return traced(*args)
        return defn.jit(traced)(*args)
    return wrapped


def grad(fun, argnums=0):
    """``Nx.Defn.grad/2``."""
    vg = value_and_grad(fun, argnums)
    return lambda *args: vg(*args)[1]
