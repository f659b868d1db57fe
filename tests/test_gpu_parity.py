"""Parity of the CUDA path against the CPU oracle on seeded random inputs.

Tolerances (the ones the north star states): bit-exact for integer and index
outputs; f32 within rtol 1e-5 (plus atol 1e-6 for values that cancel to ~0);
bf16 within rtol 2e-2 / atol 1e-2.
"""
import numpy as np
import pytest

import nx_oracle as O
from helpers import assert_close
from nx_b200 import backend, defn, nx, types as T

pytestmark = pytest.mark.gpu

F32_TOL = dict(rtol=1e-5, atol=1e-6)
BF16_TOL = dict(rtol=2e-2, atol=1e-2)


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def run_both(fun, arrays, types):
    """arrays: numpy arrays (f32 for bf16 inputs); returns [(gpu, oracle, type)]."""
    host = []
    for a, t in zip(arrays, types):
        backend.set_default_backend(None)
        host.append(nx.tensor(a, t))
        backend.set_default_backend("b200", 0)
    dev = [backend.backend_transfer(h) for h in host]
    out = defn.jit(fun)(*dev)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    blob, _ = defn.build_program(fun, host)
    ref = O.run_program(blob, [h.data.raw for h in host], "xla_like")
    assert len(ref) == len(outs)
    return [(nx.to_numpy(g), r[0], r[1]) for g, r in zip(outs, ref)]


def check(results, what=""):
    for i, (g, r, t) in enumerate(results):
        assert g.shape == r.shape
        if t[0] in ("s", "u"):
            assert np.array_equal(g, r), f"{what} output {i}: integer mismatch"
        elif t == ("bf", 16):
            assert_close(g, r, what=f"{what} output {i}", **BF16_TOL)
        else:
            assert_close(g, r, what=f"{what} output {i}", **F32_TOL)


def fused_rows(x):
    m = nx.reduce_max(x, axes=[1], keep_axes=True)
    e = nx.exp(x - m)
    s = nx.sum(e, axes=[1], keep_axes=True)
    return (nx.squeeze(m, [1]), e, nx.squeeze(s, [1]), nx.logsumexp(x, axes=[1]), e / s,
            nx.argmax(x, axis=1), nx.tanh(x * 0.5 + 0.1) * nx.sigmoid(x))


@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (7, 127), (4, 128), (5, 129), (16, 1000), (8, 4096),
                                   (3, 32768), (2, 40000), (64, 10)])
def test_fused_row_program_f32(shape):
    """The bandwidth-bound configuration (row max, exp, sum, logsumexp, softmax,
    argmax, tanh*sigmoid chain) at sizes around every tile and vector boundary."""
    rng = np.random.default_rng(1)
    x = rng.normal(0, 2, shape).astype(np.float32)
    check(run_both(fused_rows, [x], ["f32"]), f"rows {shape}")


def test_fused_row_program_with_infinite_and_nan_rows():
    """Rows whose maximum is +inf, -inf or NaN: the planner takes logsumexp's sum from the softmax's sum
    where the maximum is finite and from the sign of the maximum where it is not; the oracle evaluates
    the graph as written (nx/lib/nx.ex:18400-18433)."""
    rng = np.random.default_rng(3)
    x = rng.normal(0, 2, (9, 700)).astype(np.float32)
    x[1] = -np.inf                         # every element -inf: maximum -inf, sum(exp(x - 0)) = 0
    x[2, 17] = np.inf                      # one +inf
    x[3, 5] = x[3, 600] = np.inf           # several +inf
    x[4, 9] = np.nan                       # NaN: the maximum is NaN, not infinite
    x[5, 9] = np.nan
    x[5, 10] = np.inf                      # NaN and +inf
    x[6, :350] = -np.inf                   # -inf among finite values: finite maximum
    x[7, 3] = 88.0                         # exp(x) overflows without the shift
    x[8] = 0.0
    results = run_both(fused_rows, [x], ["f32"])
    for i, (g, r, t) in enumerate(results):
        assert np.array_equal(np.isnan(g), np.isnan(r)), f"output {i}: NaN pattern"
        assert np.array_equal(np.isinf(g), np.isinf(r)) and np.array_equal(np.sign(g[np.isinf(g)]), np.sign(r[np.isinf(r)])), f"output {i}: infinities"
        fin = np.isfinite(r)
        if t[0] in ("s", "u"):
            assert np.array_equal(g, r), f"output {i}"
        else:
            assert_close(g[fin], r[fin], what=f"output {i}", **F32_TOL)


def test_fused_row_program_is_one_launch():
    prog = defn.compile(fused_rows, [defn.template((64, 1024), "f32")]).program
    assert prog.launch_count() == 1, prog.describe()


def test_argmax_ties_and_nan_rows():
    x = np.zeros((6, 300), dtype=np.float32)
    x[1, 7] = x[1, 200] = 3.0            # tie: lowest index
    x[2, 5] = np.nan                      # one NaN beats numbers
    x[3, 5] = x[3, 250] = np.nan          # several NaNs: last one (BinaryBackend scan order)
    x[4] = -np.inf
    x[5, 299] = np.inf
    t = nx.tensor(x)
    lo = nx.to_numpy(nx.argmax(t, axis=1))
    hi = nx.to_numpy(nx.argmax(t, axis=1, tie_break="high"))
    assert lo.tolist() == [0, 7, 5, 250, 0, 299]
    assert hi.tolist() == [299, 200, 5, 250, 299, 299]
    assert nx.to_numpy(nx.argmin(t, axis=1)).tolist() == [0, 0, 5, 250, 0, 0]


UNARY = ["exp", "expm1", "log", "log1p", "sigmoid", "cos", "sin", "tan", "cosh", "sinh", "tanh", "acos", "asin",
         "atan", "acosh", "asinh", "atanh", "sqrt", "rsqrt", "cbrt", "erf", "erfc", "erf_inv"]


@pytest.mark.parametrize("op", UNARY)
def test_unary_math_f32(op):
    rng = np.random.default_rng(7)
    x = rng.uniform(-3, 3, (33, 77)).astype(np.float32)
    if op in ("log", "sqrt", "rsqrt", "log1p"):
        x = np.abs(x) + 0.01
    if op in ("acos", "asin", "atanh", "erf_inv"):
        x = np.clip(x / 3.1, -0.99, 0.99)
    if op == "acosh":
        x = np.abs(x) + 1.0
    f = getattr(nx, op)
    check(run_both(lambda t: f(t), [x], ["f32"]), op)


@pytest.mark.parametrize("op,lo,hi", [("exp", -110.0, 89.5), ("exp", -1e-3, 1e-3), ("tanh", -0.2, 0.2), ("tanh", -1e-4, 1e-4),
                                      ("tanh", -12.0, 12.0), ("sigmoid", -100.0, 100.0), ("sigmoid", -1e-3, 1e-3)])
def test_hand_written_math_over_wide_ranges(op, lo, hi):
    """exp / tanh / sigmoid are this library's own routines: sweep the ends of their ranges."""
    x = np.linspace(lo, hi, 200001).astype(np.float32)
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, np.nan], dtype=np.float32)])
    f = getattr(nx, op)
    for g, r, t in run_both(lambda t: f(t), [x], ["f32"]):
        # results below the smallest normal number are flushed to zero on the device
        assert_close(g, r, rtol=1e-5, atol=1.2e-38, what=op)


@pytest.mark.parametrize("op", ["exp", "tanh", "sigmoid", "rsqrt", "cos", "sin", "erf", "negate", "abs"])
def test_unary_bf16(op):
    rng = np.random.default_rng(8)
    x = np.abs(rng.normal(0, 1, (17, 256)).astype(np.float32)) + 0.05
    f = getattr(nx, op)
    check(run_both(lambda t: f(t), [x], ["bf16"]), op)


BINARY = ["add", "subtract", "multiply", "divide", "pow", "remainder", "atan2", "min", "max"]


@pytest.mark.parametrize("op", BINARY)
@pytest.mark.parametrize("types", [("f32", "f32"), ("bf16", "bf16"), ("f32", "bf16"), ("s32", "f32")])
def test_binary_float(op, types):
    rng = np.random.default_rng(9)
    a = rng.uniform(0.5, 3, (9, 1, 64)).astype(np.float32)
    b = rng.uniform(0.5, 3, (5, 64)).astype(np.float32)
    if types[0].startswith("s"):
        a = np.round(a * 3)
    f = getattr(nx, op)
    check(run_both(lambda x, y: f(x, y), [a, b], list(types)), f"{op} {types}")


INT_BINARY = ["add", "subtract", "multiply", "quotient", "remainder", "min", "max", "bitwise_and", "bitwise_or",
              "bitwise_xor", "left_shift", "right_shift", "pow"]


@pytest.mark.parametrize("op", INT_BINARY)
@pytest.mark.parametrize("types", [("s32", "s32"), ("s8", "s8"), ("u8", "s8"), ("u8", "u8"), ("s64", "s32"), ("u16", "u32")])
def test_binary_integer_exact(op, types):
    rng = np.random.default_rng(10)
    a = rng.integers(1, 100, (13, 37))
    b = rng.integers(1, 6, (37,))
    if op in ("left_shift", "right_shift", "pow"):
        b = rng.integers(0, 4, (37,))
    f = getattr(nx, op)
    check(run_both(lambda x, y: f(x, y), [a, b], list(types)), f"{op} {types}")


@pytest.mark.parametrize("op", ["equal", "not_equal", "greater", "less", "greater_equal", "less_equal",
                                "logical_and", "logical_or", "logical_xor"])
def test_comparisons(op):
    rng = np.random.default_rng(11)
    a = rng.integers(-2, 3, (40, 9)).astype(np.float32)
    b = rng.integers(-2, 3, (9,))
    a[0, 0] = np.nan
    f = getattr(nx, op)
    check(run_both(lambda x, y: f(x, y), [a, b], ["f32", "s32"]), op)


@pytest.mark.parametrize("src,dst", [("f32", "s32"), ("f32", "u8"), ("f32", "bf16"), ("bf16", "f32"), ("s32", "f32"),
                                     ("s32", "s8"), ("u8", "f32"), ("f32", "f64"), ("f64", "f32"), ("f32", "f16"),
                                     ("s64", "bf16")])
def test_as_type(src, dst):
    rng = np.random.default_rng(12)
    x = rng.uniform(-200, 200, (1000,)).astype(np.float32)
    if src[0] in "su":
        x = np.round(x)
    if src[0] == "u":
        x = np.abs(x)
    check(run_both(lambda t: nx.as_type(t, dst), [x], [src]), f"{src}->{dst}")


def test_as_type_non_finite_to_int():
    x = np.array([np.inf, np.nan, -np.inf, 1e20, -1e20, 3.99, -3.99], dtype=np.float32)
    t = nx.tensor(x)
    assert nx.to_numpy(nx.as_type(t, "s16")).tolist() == [32767, 0, -32768, 32767, -32768, 3, -3]
    assert nx.to_numpy(nx.as_type(t, "u8")).tolist() == [255, 0, 0, 255, 0, 3, 0]
    assert nx.to_numpy(nx.as_type(t, "s64")).tolist()[:3] == [2**63 - 1, 0, -2**63]


@pytest.mark.parametrize("op", ["sum", "product", "reduce_max", "reduce_min"])
@pytest.mark.parametrize("axes,keep", [([2], False), ([1, 2], True), ([0], False), ([0, 2], True), (None, False), ([1], False)])
def test_reductions_all_axes(op, axes, keep):
    rng = np.random.default_rng(13)
    x = rng.uniform(0.9, 1.1, (6, 10, 36)).astype(np.float32)
    f = getattr(nx, op)
    check(run_both(lambda t: f(t, axes=axes, keep_axes=keep), [x], ["f32"]), f"{op} {axes}")
    xi = rng.integers(-3, 4, (6, 10, 36))
    if op != "product":
        check(run_both(lambda t: f(t, axes=axes, keep_axes=keep), [xi], ["s8"]), f"{op} {axes} s8")


def test_all_any():
    rng = np.random.default_rng(14)
    x = rng.integers(0, 2, (50, 70))
    check(run_both(lambda t: (nx.all(t, axes=[1]), nx.any(t, axes=[1]), nx.all(t), nx.any(t, axes=[0])), [x], ["u8"]))


def test_shape_ops_fuse_into_consumers():
    rng = np.random.default_rng(15)
    x = rng.normal(0, 1, (4, 6, 8)).astype(np.float32)
    b = rng.normal(0, 1, (6,)).astype(np.float32)

    def f(x, b):
        t = nx.transpose(x, [2, 0, 1])                     # {8,4,6}
        y = t + nx.broadcast(b, (8, 4, 6), axes=[2])
        s = nx.slice(y, [1, 0, 2], [6, 4, 3], [2, 1, 1])   # {3,4,3}
        r = nx.reshape(s, (9, 4))
        i = nx.iota((9, 4), axis=0)
        return r * 2.0, nx.select(nx.greater(i, 3), r, 0.0), nx.squeeze(nx.new_axis(r, 0), [0]) - 1

    check(run_both(f, [x, b], ["f32", "f32"]), "shape ops")


def test_outputs_that_are_inputs_or_constants():
    x = np.arange(12, dtype=np.float32).reshape(3, 4)

    def f(t):
        return t, nx.reshape(t, (4, 3)), nx.broadcast(nx.as_type(2, "f32"), (2, 2)), nx.iota((2, 3), axis=1), t

    check(run_both(f, [x], ["f32"]), "leaf outputs")


def test_mlp_small_config():
    """relu(x.W1+b1).W2+b2 -> softmax -> argmax on {64,784}x{784,128}x{128,10}
    (the CPU-sized configuration), f32 logits and exact argmax."""
    rng = np.random.default_rng(0)
    x = rng.uniform(0, 1, (64, 784)).astype(np.float32)
    w1 = rng.normal(0, 0.05, (784, 128)).astype(np.float32)
    b1 = rng.normal(0, 0.05, (128,)).astype(np.float32)
    w2 = rng.normal(0, 0.05, (128, 10)).astype(np.float32)
    b2 = rng.normal(0, 0.05, (10,)).astype(np.float32)

    def mlp(x, w1, b1, w2, b2):
        h = nx.max(nx.dot(x, w1) + b1, 0.0)
        logits = nx.dot(h, w2) + b2
        m = nx.reduce_max(logits, axes=[1], keep_axes=True)
        e = nx.exp(logits - m)
        p = e / nx.sum(e, axes=[1], keep_axes=True)
        return logits, p, nx.argmax(p, axis=1)

    res = run_both(mlp, [x, w1, b1, w2, b2], ["f32"] * 5)
    # dot products of 784 terms: compare with an absolute floor scaled to the logits' size
    assert_close(res[0][0], res[0][1], rtol=1e-5, atol=2e-6, what="logits")
    assert_close(res[1][0], res[1][1], rtol=1e-5, atol=1e-6, what="softmax")
    assert np.array_equal(res[2][0], res[2][1])
    # and against the BinaryBackend-mode oracle (f64 scalar math), the oracle of this config
    backend.set_default_backend(None)
    host = [nx.tensor(a, "f32") for a in (x, w1, b1, w2, b2)]
    backend.set_default_backend("b200", 0)
    blob, _ = defn.build_program(mlp, host)
    bb = O.run_program(blob, [h.data.raw for h in host], "binary_backend")
    assert_close(res[0][0], bb[0][0], rtol=1e-5, atol=2e-6, what="logits vs binary_backend")
    assert np.array_equal(res[2][0], bb[2][0])


def test_dot_integer_exact_and_wrapping():
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, (33, 300))
    b = rng.integers(-127, 128, (300, 17))
    check(run_both(lambda x, y: nx.dot(nx.as_type(x, "s32"), nx.as_type(y, "s32")), [a, b], ["s8", "s8"]), "s8->s32 dot")
    check(run_both(lambda x, y: nx.dot(x, y), [a, b], ["s8", "s8"]), "s8 dot wraps to s8")
    check(run_both(lambda x, y: nx.dot(x, [1], y, [0]), [a, b], ["s32", "s32"]), "s32 dot")


def test_dot_layouts():
    rng = np.random.default_rng(4)
    a = rng.normal(0, 1, (3, 20, 12)).astype(np.float32)
    b = rng.normal(0, 1, (3, 12, 7)).astype(np.float32)
    c = rng.normal(0, 1, (3, 7, 12)).astype(np.float32)
    tol = dict(rtol=1e-5, atol=1e-5)
    for fun, arrs in [
        (lambda x, y: nx.dot(x, [2], [0], y, [1], [0]), [a, b]),
        (lambda x, y: nx.dot(x, [2], [0], y, [2], [0]), [a, c]),
        (lambda x, y: nx.dot(x, [1], [0], y, [2], [0]), [np.ascontiguousarray(a.transpose(0, 2, 1)), c]),
        (lambda x, y: nx.dot(nx.transpose(x, [0, 2, 1]), [2], [0], y, [1], [0]), [a, rng.normal(0, 1, (3, 20, 5)).astype(np.float32)]),
        (lambda x, y: nx.dot(x, [0, 2], [], y, [0, 1], []), [a, rng.normal(0, 1, (3, 12, 9)).astype(np.float32)]),
    ]:
        for g, r, t in run_both(fun, arrs, ["f32", "f32"]):
            assert_close(g, r, what="dot layout", **tol)


# ---- indexed reads and writes: gather / take / put_slice / slice with tensor starts ---------------
def test_embedding_lookup_feeds_a_fused_row_kernel():
    """Nx.take on a bf16 table by token ids (an embedding lookup), alone and with an RMS norm
    computed from the looked-up rows in the same kernel."""
    rng = np.random.default_rng(11)
    table = rng.normal(0, 1, (1000, 256)).astype(np.float32)
    ids = rng.integers(0, 1000, (4, 37))
    ids[0, :3] = [-5, 1000, 999]                      # out of range: clamped like XLA's gather

    def rms(t):
        return t * nx.rsqrt(nx.mean(t * t, axes=[-1], keep_axes=True) + 1e-5)

    res = run_both(lambda w, i: (nx.take(w, i), rms(nx.take(w, i))), [table, ids], ["bf16", "s64"])
    assert res[0][0].shape == (4, 37, 256)
    assert np.array_equal(res[0][0], res[0][1]), "a lookup copies values"
    check(res[1:], "rms norm of embeddings")
    for it in ("s32", "u8", "u32"):
        small = rng.integers(0, 200, (9,))
        r = run_both(lambda w, i: nx.take(w, i, axis=1), [table[:50], small], ["f32", it])
        assert np.array_equal(r[0][0], r[0][1]), it


def test_gather_general_axes():
    rng = np.random.default_rng(12)
    t = rng.normal(0, 1, (5, 6, 7, 8)).astype(np.float32)
    idx = np.stack([rng.integers(-1, 7, (3, 4)), rng.integers(0, 9, (3, 4))], axis=-1)      # axes 1 and 3
    for g, r, _ in run_both(lambda a, i: nx.gather(a, i, axes=[1, 3]), [t, idx], ["f32", "s32"]):
        assert g.shape == (3, 4, 5, 7) and np.array_equal(g, r)
    full = np.stack([rng.integers(0, d, (11,)) for d in t.shape], axis=-1)
    for g, r, _ in run_both(lambda a, i: nx.gather(a * 2.0, i), [t, full], ["f32", "s64"]):          # table computed in the program
        assert g.shape == (11,) and np.array_equal(g, r)


@pytest.mark.parametrize("pos", [0, 5, 60, 63, 200])
def test_kv_cache_update_and_window_read(pos):
    """put_slice of one position into a {B,H,S,D} cache at a position held in a tensor, then a
    dynamic slice reading a window back; positions beyond the end are clamped."""
    rng = np.random.default_rng(13)
    cache = rng.normal(0, 1, (2, 3, 64, 16)).astype(np.float32)
    new = rng.normal(0, 1, (2, 3, 1, 16)).astype(np.float32)

    def f(c, n, p):
        c2 = nx.put_slice(c, [0, 0, p, 0], n)
        return c2, nx.slice(c2, [0, 0, p, 0], [2, 3, 4, 16]) * 2.0

    res = run_both(f, [cache, new, np.array(pos)], ["bf16", "bf16", "s32"])
    assert np.array_equal(res[0][0], res[0][1])
    p = min(pos, 63)
    assert np.array_equal(res[0][0][:, :, p], res[0][1][:, :, p])
    check(res[1:], "window")
    mixed = run_both(lambda c, n, p: nx.put_slice(c, [0, 0, p, 0], n), [cache, new, np.array(pos)], ["f32", "bf16", "s64"])
    assert mixed[0][2] == ("f", 32) and np.array_equal(mixed[0][0], mixed[0][1])


def test_repeated_runs_replay_a_graph_and_still_read_current_data():
    """From its third run on the same buffers a small program is replayed as a captured CUDA graph
    (the first run executes step by step, the second captures): the replay must read what the
    buffers hold now.  A second program refills the replayed program's input between runs."""
    rng = np.random.default_rng(21)
    w = nx.tensor(rng.normal(0, 1, (64, 32)).astype(np.float32))
    fill = defn.compile(lambda t: t * 1.0 + 0.0 * nx.sum(t), [defn.template((16, 64), "f32")]).program
    mlp = defn.compile(lambda t, m: nx.tanh(nx.dot(t, m)) + nx.sum(t, axes=[1], keep_axes=True),
                       [defn.template((16, 64), "f32"), defn.template((64, 32), "f32")]).program
    x_dev = fill.run([nx.tensor(np.zeros((16, 64), np.float32))], 0)       # the buffer both programs share
    outs = None
    for i in range(6):
        x = rng.normal(0, 1, (16, 64)).astype(np.float32)
        fill.run_into([nx.tensor(x)], x_dev, 0)
        outs = mlp.run([x_dev[0], w], 0) if outs is None else mlp.run_into([x_dev[0], w], outs, 0)
        want = np.tanh(x.astype(np.float64) @ nx.to_numpy(w).astype(np.float64)) + x.sum(axis=1, keepdims=True)
        assert_close(nx.to_numpy(outs[0]), want, rtol=1e-5, atol=1e-5, what=f"run {i}")


def test_pad_and_reverse_fuse_into_consumers():
    rng = np.random.default_rng(31)
    x = rng.normal(0, 1, (5, 7, 9)).astype(np.float32)
    for cfg in ([(1, 2, 0), (0, 0, 0), (3, 1, 0)], [(0, 1, 2), (2, 0, 1), (-1, -2, 0)], [(-2, 3, 1), (0, -1, 0), (1, 1, 3)]):
        check(run_both(lambda t: nx.exp(nx.pad(t, -1.5, cfg)) * 2.0, [x], ["f32"]), f"pad {cfg}")
    check(run_both(lambda t: nx.sum(nx.pad(t, 0.0, [(0, 0, 0), (1, 1, 0), (0, 7, 0)]), axes=[2]), [x], ["bf16"]), "pad + row sum bf16")
    for axes in (None, [0], [2], [0, 2], [1]):
        res = run_both(lambda t: (nx.reverse(t, axes=axes), nx.reverse(t, axes=axes) + t), [x], ["f32"])
        assert np.array_equal(res[0][0], res[0][1])
        check(res[1:], f"reverse {axes}")
    idx = rng.integers(0, 9, (5, 7, 4))
    res = run_both(lambda t, i: nx.take_along_axis(t, i, axis=2), [x, idx], ["f32", "s32"])
    assert np.array_equal(res[0][0], np.take_along_axis(x, idx, axis=2)) and np.array_equal(res[0][0], res[0][1])


def test_window_reductions_pooling_shapes():
    """2x2 / 3x3 pooling over {N,C,H,W} as a CNN uses it, with strides, :same padding and dilation."""
    rng = np.random.default_rng(41)
    x = rng.normal(0, 1, (2, 3, 17, 20)).astype(np.float32)
    for fn in (nx.window_max, nx.window_sum, nx.window_min, nx.window_mean):
        check(run_both(lambda t: fn(t, (1, 1, 2, 2), strides=[1, 1, 2, 2]), [x], ["f32"]), "2x2 stride 2")
        check(run_both(lambda t: fn(t, (1, 1, 3, 3), strides=[1, 1, 2, 1], padding="same"), [x], ["f32"]), "3x3 same")
        check(run_both(lambda t: fn(t, (1, 1, 2, 3), padding=[(0, 0), (0, 0), (1, 2), (3, 0)], window_dilations=[1, 1, 2, 2]), [x], ["f32"]), "dilated")
    xi = rng.integers(-50, 50, (4, 9, 11))
    for fn in (nx.window_max, nx.window_sum, nx.window_product):
        check(run_both(lambda t: fn(t, (2, 3, 1), strides=[1, 2, 3], padding=[(0, 1), (2, 0), (1, 1)]), [xi], ["s32"]), "integers")
    check(run_both(lambda t: nx.exp(nx.window_max(t, (1, 1, 2, 2), strides=[1, 1, 2, 2])) + 1.0, [x], ["bf16"]), "bf16 pooled then exp")


def test_conv_on_the_device():
    """Nx.conv (lowered to pad / strided slices / dot): f32 and bf16 images, strides, padding, dilation, groups."""
    rng = np.random.default_rng(51)
    x = rng.normal(0, 1, (2, 8, 14, 12)).astype(np.float32)
    w = rng.normal(0, 0.3, (16, 8, 3, 3)).astype(np.float32)
    for opts in (dict(), dict(strides=[2, 1], padding="same"), dict(padding=[(1, 0), (-1, 2)], kernel_dilation=[2, 1]),
                 dict(padding="same", input_dilation=[1, 2])):
        check(run_both(lambda a, b: nx.conv(a, b, **opts), [x, w], ["f32", "f32"]), f"conv {opts}")
    wg = rng.normal(0, 0.3, (16, 2, 3, 3)).astype(np.float32)
    check(run_both(lambda a, b: nx.conv(a, b, feature_group_size=4, padding="same"), [x, wg], ["f32", "f32"]), "grouped conv")
    res = run_both(lambda a, b: nx.max(nx.conv(a, b, padding="same"), 0.0), [x, w], ["bf16", "bf16"])
    assert res[0][2] == ("bf", 16)
    check(res, "bf16 conv + relu")


def test_sort_argsort_top_k():
    """Bitonic rows in shared memory: every element type, both directions, ties (stable), NaN / -0.0,
    lengths around the powers of two, another axis, and top_k as a sampling step would use it."""
    rng = np.random.default_rng(61)
    for length in (1, 2, 31, 32, 33, 1000, 4096, 5000, 16384):
        x = rng.normal(0, 1, (3, length)).astype(np.float32)
        x[0, : length // 3] = x[0, 0]                                        # ties
        if length > 4:
            x[1, 1], x[1, 3], x[2, 0], x[2, 2] = np.nan, np.inf, -0.0, 0.0
        for d in ("asc", "desc"):
            res = run_both(lambda t: (nx.sort(t, axis=1, direction=d), nx.argsort(t, axis=1, direction=d)), [x], ["f32"])
            assert np.array_equal(res[0][0], res[0][1], equal_nan=True), (length, d)
            assert np.array_equal(res[1][0], res[1][1]), (length, d, "argsort")
    for ty in ("s8", "u8", "s16", "u32", "s64", "u64", "f64", "bf16", "f16"):
        a = rng.integers(-100, 100, (5, 77)) if ty[0] == "s" else rng.integers(0, 200, (5, 77)) if ty[0] == "u" else rng.normal(0, 3, (5, 77))
        res = run_both(lambda t: (nx.sort(t, axis=1, direction="desc"), nx.argsort(t, axis=1)), [a], [ty])
        assert np.array_equal(res[0][0], res[0][1]) and np.array_equal(res[1][0], res[1][1]), ty
    y = rng.normal(0, 1, (4, 50, 6)).astype(np.float32)
    res = run_both(lambda t: (nx.sort(t, axis=1), nx.argsort(t, axis=0, direction="desc", type="s64")), [y], ["f32"])
    assert np.array_equal(res[0][0], np.sort(y, axis=1)) and np.array_equal(res[1][0], res[1][1]) and res[1][2] == ("s", 64)
    logits = rng.normal(0, 1, (8, 8000)).astype(np.float32)
    res = run_both(lambda t: nx.top_k(nx.exp(t) / nx.sum(nx.exp(t), axes=[1], keep_axes=True), k=40), [logits], ["f32"])
    assert np.array_equal(res[1][0], np.argsort(-logits, axis=1, kind="stable")[:, :40])
    check(res[:1], "top-k probabilities")
