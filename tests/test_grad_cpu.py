"""Reverse-mode gradients (the mirror of Nx.Defn.Grad): the gradient graph, evaluated on the CPU by
the oracle in f64, against (1) the expected values of nx/test/nx/defn/grad_test.exs and (2) central
finite differences of the function itself, the check the reference's own `check_grads!` makes
(nx/test/support/grad_helpers.ex)."""
import numpy as np
import pytest

import nx_oracle as O
from helpers import assert_close, host_tensor, oracle_run
from nx_b200 import defn, nx
from nx_b200.grad import grad, value_and_grad


def run(fun, arrays, type="f64", build=True):
    host = [host_tensor(a, type) for a in arrays]
    blob, res = oracle_run(fun, host)
    if build:
        defn.Program(blob)                   # the kernels of the gradient graph compile (no GPU needed)
    return [np.asarray(r[0], dtype=np.float64) for r in res]


def finite_difference(fun, arrays, wrt, eps=1e-6):
    base = [np.asarray(a, dtype=np.float64) for a in arrays]
    out = np.zeros_like(base[wrt])
    it = np.nditer(base[wrt], flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        hi = [b.copy() for b in base]
        lo = [b.copy() for b in base]
        hi[wrt][i] += eps
        lo[wrt][i] -= eps
        out[i] = (run(fun, hi, build=False)[0] - run(fun, lo, build=False)[0]) / (2 * eps)
    return out


def check(fun, arrays, wrt=0, rtol=1e-5, atol=1e-7):
    got = run(lambda *xs: grad(fun, wrt)(*xs), arrays)[0]
    want = finite_difference(fun, arrays, wrt)
    assert_close(got, want, rtol, atol, "gradient vs finite differences")


# ---- expected values from the reference's tests ---------------------------------------------------

def test_reference_scalars():
    # grad_test.exs:233-270
    f = lambda t: nx.tanh(nx.tanh(nx.pow(t, 2) + nx.pow(t, 3)))
    assert_close(run(grad(f), [1.0])[0], 0.15662670135498047, 1e-6, 0)
    f = lambda t: nx.tanh(nx.tanh(nx.pow(t, 2) * nx.pow(t, 3)))
    assert_close(run(grad(f), [1.0])[0], 1.2343397629215758, 1e-6, 0)
    f = lambda t: nx.sum(nx.pow(t, 2) * nx.pow(t, 3))
    assert_close(run(grad(f), [[[1.0, 2.0], [3.0, 4.0]]])[0], [[5.0, 80.0], [405.0, 1280.0]], 1e-12, 0)
    f = lambda t: nx.tanh(t) / t                                                     # :275-292
    assert_close(run(grad(f), [1.0])[0], -0.3416198492050171, 1e-6, 0)


def test_reference_simple():
    # grad_test.exs:23-53
    assert_close(run(grad(lambda t: t), [1.0])[0], 1.0, 0, 0)
    assert_close(run(grad(lambda t: nx.tensor(1.0)), [1.0])[0], 0.0, 0, 0)
    assert_close(run(lambda t, a: grad(lambda t: nx.sum(a))(t), [[1.0, 2.0], [2.0, 3.0]])[0], [0.0, 0.0], 0, 0)


def test_reference_dot():
    # grad_test.exs:412-551
    lhs = lambda x, y: grad(lambda x: nx.sum(nx.dot(x, y)))(x)
    assert_close(run(lhs, [[[1.0], [2.0], [3.0]], [[1.0, 2, 3, 4, 5]]])[0], [[15.0], [15.0], [15.0]], 0, 0)
    assert_close(run(lhs, [[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], [1.0, 2.0]])[0], [[1.0, 2.0]] * 3, 0, 0)
    assert_close(run(lhs, [[1.0, 2.0], [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]])[0], [6.0, 15.0], 0, 0)
    rhs = lambda x, y: grad(lambda y: nx.sum(nx.dot(x, y)))(y)
    assert_close(run(rhs, [[[1.0], [2.0], [3.0]], [[1.0, 2, 3, 4, 5]]])[0], [[6.0] * 5], 0, 0)
    assert_close(run(rhs, [[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], [1.0, 2.0]])[0], [9.0, 12.0], 0, 0)
    assert_close(run(rhs, [[1.0, 2.0], [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]])[0], [[1.0] * 3, [2.0] * 3], 0, 0)
    both = grad(lambda x: nx.sum(nx.dot(nx.pow(x, 2), nx.pow(x, 3))))
    assert_close(run(both, [[1.0, 2.0, 3.0]])[0], [5.0, 80.0, 405.0], 0, 0)
    got = run(both, [np.arange(27.0).reshape(3, 3, 3)])[0]
    assert_close(got[0], [[0.0, 83430.0, 263952.0], [198207.0, 410616.0, 759375.0], [533952.0, 884142.0, 1410048.0]], 0, 0)
    assert_close(got[2, 2], [5121792.0, 6268050.0, 7817472.0], 0, 0)

    def two_layers(x, w1, b1, w2, b2, labels):
        return grad(lambda x: nx.sum((nx.dot(nx.dot(x, w1) + b1, w2) + b2) * labels))(x)
    shapes = [(5, 4), (4, 3), (3,), (3, 2), (2,), (5, 2)]
    args = [np.arange(float(np.prod(s))).reshape(s) for s in shapes]
    assert_close(run(two_layers, args)[0], [[13.0, 40.0, 67.0, 94.0], [59.0, 176.0, 293.0, 410.0], [105.0, 312.0, 519.0, 726.0],
                                            [151.0, 448.0, 745.0, 1042.0], [197.0, 584.0, 971.0, 1358.0]], 0, 0)
    bcast = lambda b1, w2, labels: grad(lambda b1: nx.sum(nx.dot(b1, w2) * labels))(b1)
    assert_close(run(bcast, [np.arange(3.0), np.arange(6.0).reshape(3, 2), np.arange(10.0).reshape(5, 2)])[0], [25.0, 115.0, 205.0], 0, 0)
    batched = lambda a, b: grad(lambda a: nx.sum(nx.dot(a, [1], [0], b, [2], [0])))(a)
    got = run(batched, [np.arange(24.0).reshape(3, 2, 4), np.arange(18.0).reshape(3, 3, 2)])[0]
    assert_close(got, [[[6.0] * 4, [9.0] * 4], [[24.0] * 4, [27.0] * 4], [[42.0] * 4, [45.0] * 4]], 0, 0)


def test_value_and_grad_and_containers():
    # grad_test.exs:60-70, 2029-2060
    f = lambda a, b: nx.tanh(a) + nx.pow(b, 2)
    val, (ga, gb) = (lambda r: (r[0], (r[1], r[2])))(run(lambda a, b: value_and_grad(lambda t: f(*t))((a, b)), [1.0, 2.0]))
    assert_close(val, np.tanh(1.0) + 4.0, 1e-12, 0)
    assert_close(ga, 1 - np.tanh(1.0) ** 2, 1e-12, 0)
    assert_close(gb, 4.0, 1e-12, 0)
    ga2, gb2 = run(lambda a, b: grad(f, (0, 1))(a, b), [1.0, 2.0])
    assert_close([ga2, gb2], [ga, gb], 0, 0)
    with pytest.raises(ValueError, match="scalar"):
        run(grad(lambda t: t * 2.0), [[1.0, 2.0]])


def test_stop_grad_through_logsumexp():
    # the max inside logsumexp is wrapped in stop_grad (nx.ex:18407-18414): the gradient is softmax
    x = np.array([[0.5, -1.0, 2.0], [3.0, 3.0, -2.0]])
    got = run(grad(lambda t: nx.sum(nx.logsumexp(t, axes=[1]))), [x])[0]
    sm = np.exp(x) / np.exp(x).sum(1, keepdims=True)
    assert_close(got, sm, 1e-12, 0)


# ---- finite differences ----------------------------------------------------------------------------

RNG = np.random.default_rng(7)
A23 = RNG.uniform(0.5, 2.0, (2, 3))
B3 = RNG.uniform(0.5, 2.0, (3,))

UNARY = ["exp", "expm1", "log", "log1p", "sigmoid", "tanh", "sqrt", "rsqrt", "cbrt", "sin", "cos", "tan", "sinh", "cosh",
         "atan", "erf", "erfc", "negate", "abs"]


@pytest.mark.parametrize("name", UNARY)
def test_unary_rules(name):
    op = getattr(nx, name)
    check(lambda t: nx.sum(op(t) * nx.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], "f64")), [A23 * (-1 if name == "abs" else 1)])


BINARY = {
    "add broadcast": lambda a, b: nx.sum(nx.exp(a + b)),
    "subtract": lambda a, b: nx.sum(nx.exp(a - b) * a),
    "multiply": lambda a, b: nx.sum(nx.sin(a * b)),
    "divide": lambda a, b: nx.sum(a / (b * b)),
    "pow": lambda a, b: nx.sum(nx.pow(a, b)),
    "max": lambda a, b: nx.sum(nx.max(a, b * 0.9) * a),
    "min": lambda a, b: nx.sum(nx.min(a, b * 0.9) * b),
    "same operand": lambda a, b: nx.sum((a + a) * (a * a) + b),
}


@pytest.mark.parametrize("name", list(BINARY))
@pytest.mark.parametrize("wrt", [0, 1])
def test_binary_rules(name, wrt):
    check(BINARY[name], [A23, B3], wrt)


def test_max_splits_ties():
    # grad.ex:1057-1075: equal operands share the gradient
    got = run(lambda a, b: grad(lambda a, b: nx.sum(nx.max(a, b)), (0, 1))(a, b), [[1.0, 2.0, 3.0], [1.0, 5.0, 0.0]])
    assert_close(got[0], [0.5, 0.0, 1.0], 0, 0)
    assert_close(got[1], [0.5, 1.0, 0.0], 0, 0)


SHAPES = {
    "reshape transpose": lambda t: nx.sum(nx.transpose(nx.reshape(t, (3, 2, 2)), [2, 0, 1]) * nx.iota((2, 3, 2), type="f64")),
    "broadcast axes": lambda t: nx.sum(nx.broadcast(nx.slice(t, [0, 0], [2, 1]), (2, 5, 4), axes=[0, 2]) * nx.iota((2, 5, 4), type="f64")),
    "broadcast unit": lambda t: nx.sum(nx.broadcast(nx.slice(t, [0, 0], [1, 6]), (4, 6)) * nx.iota((4, 6), type="f64")),
    "strided slice": lambda t: nx.sum(nx.exp(nx.slice(t, [0, 1], [2, 5], [1, 2]))),
    "concatenate": lambda t: nx.sum(nx.concatenate([nx.exp(t), t * 2.0, nx.sin(t)], axis=1) * nx.iota((2, 18), type="f64")),
    "stack": lambda t: nx.sum(nx.stack([nx.exp(t), nx.cos(t)], axis=1) * nx.iota((2, 2, 6), type="f64")),
    "pad interior": lambda t: nx.sum(nx.pad(t, 3.0, [(1, 2, 1), (-1, 1, 2)]) * nx.iota((6, 16), type="f64")),
    "pad value": lambda t: nx.sum(nx.pad(nx.iota((2, 2), type="f64"), nx.sum(t), [(1, 1, 0), (0, 2, 1)]) * nx.iota((4, 5), type="f64")),
    "reverse": lambda t: nx.sum(nx.reverse(t, axes=[1]) * nx.iota((2, 6), type="f64")),
    "sum axes": lambda t: nx.sum(nx.exp(nx.sum(t, axes=[1])) ),
    "sum keep": lambda t: nx.sum(t / nx.sum(t, axes=[0], keep_axes=True) * nx.iota((2, 6), type="f64")),
    "mean": lambda t: nx.sum(nx.pow(nx.mean(t, axes=[1]), 3)),
    "reduce_max": lambda t: nx.sum(nx.reduce_max(t, axes=[1]) * nx.tensor([2.0, 3.0], "f64")),
    "reduce_min keep": lambda t: nx.sum(t - nx.reduce_min(t, axes=[0], keep_axes=True)),
    "select clip": lambda t: nx.sum(nx.select(nx.greater(t, 1.2), nx.exp(t), nx.clip(t, 0.8, 1.0) * 3.0)),
    "squeeze new_axis": lambda t: nx.sum(nx.squeeze(nx.new_axis(t, 1), axes=[1]) * t),
    "window_sum": lambda t: nx.sum(nx.window_sum(t, (2, 3), strides=[1, 2], padding=[(1, 0), (0, 2)], window_dilations=[1, 2])
                                   * nx.iota((2, 2), type="f64")),
    "window_mean": lambda t: nx.sum(nx.exp(nx.window_mean(t, (1, 2), strides=[1, 2]))),
}


@pytest.mark.parametrize("name", list(SHAPES))
def test_shape_and_reduction_rules(name):
    check(SHAPES[name], [RNG.uniform(0.5, 2.0, (2, 6))])


def test_as_type_rule():
    # grad.ex:1088: the gradient is cast back to the operand's type
    x = RNG.uniform(0.5, 2.0, (2, 6))
    got = run(grad(lambda t: nx.sum(nx.as_type(nx.as_type(t, "f32") * 2.0, "f64") * t)), [x])[0]
    assert_close(got, 4.0 * x.astype(np.float32).astype(np.float64), 1e-12, 0)     # both terms pass through f32


def test_reduce_max_splits_ties():
    got = run(grad(lambda t: nx.sum(nx.reduce_max(t, axes=[1]))), [[[1.0, 3.0, 3.0], [2.0, 0.0, 1.0]]])[0]
    assert_close(got, [[0.0, 0.5, 0.5], [1.0, 0.0, 0.0]], 0, 0)


def test_dot_rules_general_axes():
    a = RNG.uniform(-1, 1, (2, 3, 4))
    b = RNG.uniform(-1, 1, (2, 4, 5, 3))
    f = lambda x, y: nx.sum(nx.dot(x, [2, 1], [0], y, [1, 3], [0]) * nx.iota((2, 5), type="f64"))
    check(f, [a, b], 0)
    check(f, [a, b], 1)
    g = lambda x, y: nx.sum(nx.sin(nx.dot(x, [0], [], y, [1], [])))
    check(g, [RNG.uniform(-1, 1, (3, 2)), RNG.uniform(-1, 1, (4, 3, 2))], 0)
    check(g, [RNG.uniform(-1, 1, (3, 2)), RNG.uniform(-1, 1, (4, 3, 2))], 1)


def test_conv_through_its_lowering():
    # grad_test.exs:553-583 checks conv gradients of both operands; here against finite differences
    x = RNG.uniform(-1, 1, (1, 2, 4, 4))
    w = RNG.uniform(-1, 1, (3, 2, 2, 2))
    f = lambda x, w: nx.sum(nx.conv(x, w, strides=[2, 1], padding=[(1, 0), (0, 1)], kernel_dilation=[1, 2]) * nx.iota((1, 3, 2, 3), type="f64"))
    check(f, [x, w], 0)
    check(f, [x, w], 1)


def test_mlp_softmax_cross_entropy():
    x = RNG.uniform(-1, 1, (4, 5))
    w1 = RNG.uniform(-1, 1, (5, 6))
    b1 = RNG.uniform(-1, 1, (6,))
    w2 = RNG.uniform(-1, 1, (6, 3))
    y = np.eye(3)[[0, 2, 1, 1]]

    def loss(w1, b1, w2, x, y):
        h = nx.max(nx.dot(x, w1) + b1, 0.0)
        logits = nx.dot(h, w2)
        logp = logits - nx.logsumexp(logits, axes=[1], keep_axes=True)
        return nx.negate(nx.mean(nx.sum(logp * y, axes=[1])))
    for wrt in range(3):
        check(loss, [w1, b1, w2, x, y], wrt)


def test_grad_of_grad():
    # grad_test.exs:2015-2027
    f = lambda t: nx.sum(nx.sin(t) * t)
    g2 = grad(lambda t: nx.sum(grad(f)(t)))
    x = np.array([0.3, 1.1])
    assert_close(run(g2, [x])[0], 2 * np.cos(x) - x * np.sin(x), 1e-12, 0)


def test_unsupported_op_raises():
    with pytest.raises(NotImplementedError, match="gradient of :window_max"):
        run(grad(lambda t: nx.sum(nx.window_max(t, (2,)))), [[3.0, 1.0, 2.0]])


def test_stored_row_maximum_is_not_reloaded_by_its_own_kernel():
    """The softmax-cross-entropy gradient needs the row maximum (wrapped in stop_grad) both inside the
    row kernel that computes it and in a later kernel: the row kernel must take it from its registers
    (three passes: max, sum of exponentials, weighted sum), not from the buffer it has yet to write."""
    def loss(w, x, y):
        logits = nx.dot(x, w)
        return nx.negate(nx.mean(nx.sum((logits - nx.logsumexp(logits, axes=[1], keep_axes=True)) * y, axes=[1])))
    host = [host_tensor(np.zeros(s), "f32") for s in [(8, 4), (16, 8), (16, 4)]]
    blob, _ = defn.build_program(lambda w, x, y: value_and_grad(loss)(w, x, y), host)
    prog = defn.Program(blob)
    rows = [l for l in prog.describe().splitlines() if "reduce_max" in l]
    assert len(rows) == 1 and "phases=3" in rows[0], prog.describe()
    src = [s for s in prog.kernel_sources() if "OpMax" in s][0]
    body = src[src.index('extern "C"'):]
    stored = [tok.split("(")[1].split(" ")[0] for tok in body.split("st1<float>")[1:]]
    for p in stored:
        assert f"ld1<float>({p} " not in body and f">({p} +" not in body.replace("st1<float>(" + p, ""), body


# ---- lookups and scatters (grad.ex:761-795, :962-988) -------------------------------------------------

def test_gather_take_and_embedding_lookup():
    table = np.arange(12.0).reshape(4, 3) / 7.0
    ids = np.array([2, 0, 2, 3])
    w = np.linspace(-1, 1, 12).reshape(4, 3)

    def loss(table):
        return nx.sum(nx.take(table, nx.tensor(ids, "s32"), axis=0) * nx.tensor(w, "f64"))

    got = run(grad(loss), [table])[0]
    want = np.zeros_like(table)
    np.add.at(want, ids, w)                                             # repeated ids accumulate
    assert_close(got, want, 1e-12, 0, "gradient of an embedding lookup")
    check(loss, [table])
    # general gather over two axes, and take_along_axis
    idx = np.array([[0, 1], [3, 2], [3, 2], [1, 0]])
    check(lambda t: nx.sum(nx.pow(nx.gather(nx.reshape(t, (4, 3, 1)), nx.tensor(idx, "s32"), axes=[0, 1]), 2)), [table])
    along = np.array([[2, 0], [1, 1], [0, 2], [2, 2]])
    check(lambda t: nx.sum(nx.sin(nx.take_along_axis(t, nx.tensor(along, "s32"), axis=1))), [table])


def test_put_slice_and_dynamic_slice():
    x = np.arange(20.0).reshape(4, 5) / 9.0
    piece = np.array([[1.5, -2.0], [0.5, 3.0]])
    f = lambda x, p: nx.sum(nx.pow(nx.put_slice(x, [1, 2], p), 2) * nx.tensor(np.arange(20.0).reshape(4, 5), "f64"))
    check(f, [x, piece], wrt=0)
    check(f, [x, piece], wrt=1)
    # a slice whose start is a tensor: the gradient is put back at that position
    start = nx.tensor(2, "s32")
    g = lambda x: nx.sum(nx.pow(nx.slice(x, [start, 1], [2, 3]), 3))
    check(g, [x])
    g2 = lambda x: nx.sum(nx.exp(nx.slice(x, [nx.tensor(0, "s32"), nx.tensor(0, "s32")], [3, 5], [2, 2])))
    check(g2, [x])


def test_indexed_add_and_put():
    target = np.arange(12.0).reshape(3, 4) / 5.0
    idx = np.array([[0, 1], [2, 3], [0, 1], [1, 0]])
    upd = np.array([0.5, -1.0, 2.0, 0.25])
    w = np.arange(12.0).reshape(3, 4)
    f = lambda t, u: nx.sum(nx.pow(nx.indexed_add(t, nx.tensor(idx, "s32"), u), 2) * nx.tensor(w, "f64"))
    check(f, [target, upd], wrt=0)
    check(f, [target, upd], wrt=1)
    # indexed_put (distinct positions): the target loses the gradient where it was overwritten
    idx2 = np.array([[0, 1], [2, 3], [1, 0]])
    h = lambda t, u: nx.sum(nx.pow(nx.indexed_put(t, nx.tensor(idx2, "s32"), u), 2) * nx.tensor(w, "f64"))
    check(h, [target, upd[:3]], wrt=0)
    check(h, [target, upd[:3]], wrt=1)
    # rows on one axis
    rows = np.array([[2], [0]])
    k = lambda t, u: nx.sum(nx.sin(nx.indexed_add(t, nx.tensor(rows, "s32"), u)))
    check(k, [target, np.ones((2, 4)) * 0.3], wrt=1)


def test_sort_gradient_follows_the_permutation():
    x = np.array([[0.3, -1.0, 2.0, 0.1], [5.0, 4.0, -3.0, 0.0]])
    w = np.array([1.0, 10.0, 100.0, 1000.0])
    f = lambda t: nx.sum(nx.sort(t, axis=1) * nx.tensor(w, "f64"))
    got = run(grad(f), [x])[0]
    want = np.zeros_like(x)
    for r in range(2):
        want[r, np.argsort(x[r])] = w
    assert_close(got, want, 0, 0, "gradient of sort")
    check(lambda t: nx.sum(nx.pow(nx.sort(t, axis=0, direction="desc"), 2) * nx.tensor(np.arange(8.0).reshape(2, 4), "f64")), [x])


# ---- rules added after random compositions were checked against finite differences -----------------

def test_reference_atan2_remainder_and_erf_inv():
    # grad_test.exs:318-323, 395-400
    assert_close(run(grad(lambda t: nx.remainder(nx.tanh(t), t)), [1.0])[0], 0.41997434161402614, 1e-12, 0)
    assert_close(run(grad(lambda t: nx.atan2(nx.tanh(t), t)), [1.0])[0], -0.21621156120382867, 1e-12, 0)
    # grad_test.exs:2225-2242: the curve is too sharp near 1 for finite differences
    for x, want in [(0.9, 3.43), (0.98, 13.26), (0.99, 24.45), (0.995, 45.56), (0.999, 198.94)]:
        assert abs(run(grad(nx.erf_inv), [x])[0] - want) < 0.01


def test_reference_product():
    # grad_test.exs:4222-4290
    total = lambda **o: grad(lambda t: nx.sum(nx.product(t, **o)))
    a = [[[[1.0, 2, 3, 4], [2, 1, 3, -1]]]]
    assert_close(run(total(), [a])[0], [[[[-144.0, -72, -48, -36], [-72, -144, -48, 144]]]], 1e-12, 0)
    b = [[[[1.0, 2, 3, 4], [2, 1, 3, -1], [3, 2, 3, 0]]]]
    assert_close(run(total(), [b])[0], [[[[0.0] * 4, [0.0] * 4, [0.0, 0, 0, -2592]]]], 1e-12, 0)
    c = [[[[1.0, 2, 3, 4], [2, 1, 3, -1], [3, 2, 3, 0], [0, 2, 3, 0]]]]
    assert_close(run(total(axes=[3]), [c])[0], [[[[24.0, 12, 8, 6], [-3, -6, -2, 6], [0, 0, 0, 18], [0, 0, 0, 0]]]], 1e-12, 0)
    assert_close(run(total(keep_axes=True), [a])[0], [[[[-144.0, -72, -48, -36], [-72, -144, -48, 144]]]], 1e-12, 0)
    assert_close(run(total(axes=[3], keep_axes=True), [a])[0], [[[[24.0, 12, 8, 6], [-3, -6, -2, 6]]]], 1e-12, 0)
    composed = grad(lambda t: nx.sum(nx.sin(nx.product(nx.cos(t)))))
    assert_close(run(composed, [a])[0], [[[[0.0272486, -0.03822973, -0.00249401, 0.02025739],
                                           [-0.03822973, 0.0272486, -0.00249401, -0.0272486]]]], 1e-5, 1e-8)


@pytest.mark.parametrize("name", ["asin", "acos", "atanh", "asinh", "acosh", "erf_inv", "atan2_l", "atan2_r", "rem_l", "rem_r", "product"])
def test_added_rules_against_finite_differences(name):
    rng = np.random.default_rng(11)
    inside = rng.uniform(-0.8, 0.8, (3, 4))
    wide = rng.standard_normal((3, 4)) * 2.0
    other = rng.standard_normal((4,)) + 3.0
    w = rng.standard_normal((3, 4))
    if name in ("asin", "acos", "atanh", "erf_inv"):
        check(lambda x: nx.sum(getattr(nx, name)(x) * nx.tensor(w, "f64")), [inside], rtol=1e-5, atol=1e-6)
    elif name == "asinh":
        check(lambda x: nx.sum(nx.asinh(x) * nx.tensor(w, "f64")), [wide])
    elif name == "acosh":
        check(lambda x: nx.sum(nx.acosh(x) * nx.tensor(w, "f64")), [np.abs(wide) + 1.5])
    elif name.startswith("atan2"):
        check(lambda x, y: nx.sum(nx.atan2(x, y) * nx.tensor(w, "f64")), [wide, other], wrt=0 if name.endswith("l") else 1)
    elif name.startswith("rem"):
        # positive operands: the reference's rule for the divisor is -floor(x / y) (grad.ex:1020-1025), which is
        # the derivative of the truncating remainder only where x / y is positive
        check(lambda x, y: nx.sum(nx.remainder(x, y) * nx.tensor(w, "f64")), [np.abs(wide) * 3.0 + 0.1, other],
              wrt=0 if name.endswith("l") else 1)
    else:
        check(lambda x: nx.sum(nx.product(x, axes=[1]) * nx.tensor(w[:, 0], "f64")), [wide])
