"""while / cond orchestrated by the host over compiled programs (the scenarios of
exla/test/exla/defn/expr_test.exs "while" and "cond"), ending with a greedy autoregressive
decode loop over a KV cache that exercises take, put_slice and slice with tensor indices."""
import numpy as np
import pytest

from nx_b200 import backend, defn, nx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def test_while_counts_and_accumulates():
    # while {i, acc} = {0, 1.0}, i < 10 do {i + 1, acc * 2} end
    i, acc = defn.while_loop(lambda i, a: nx.less(i, 10), lambda i, a: (i + 1, a * 2.0), (nx.tensor(0), nx.tensor(1.0)))
    assert nx.to_number(i) == 10 and nx.to_number(acc) == 1024.0
    # a loop whose condition is false at once returns the initial state
    (x,) = defn.while_loop(lambda x: nx.greater(nx.sum(x), 100.0), lambda x: (x * 2.0,), (nx.tensor([1.0, 2.0]),))
    assert np.array_equal(nx.to_numpy(x), [1.0, 2.0])
    # tensors in the state: factorial-like product over an iota
    n, fact = defn.while_loop(lambda n, f: nx.greater(n, 1), lambda n, f: (n - 1, f * nx.as_type(n, "f32")),
                              (nx.tensor(6), nx.tensor([1.0, 2.0])))
    assert np.array_equal(nx.to_numpy(fact), [720.0, 1440.0])


def test_while_rejects_a_body_that_changes_the_state_template():
    with pytest.raises(ValueError, match="same shape, type"):
        defn.while_loop(lambda i: nx.less(i, 3), lambda i: (nx.as_type(i, "f32") + 1.0,), (nx.tensor(0),))
    with pytest.raises(ValueError, match="scalar"):
        defn.while_loop(lambda x: nx.less(x, 3.0), lambda x: (x + 1.0,), (nx.tensor([0.0, 1.0]),))
    with pytest.raises(RuntimeError, match="did not finish"):
        defn.while_loop(lambda i: nx.greater_equal(i, 0), lambda i: (i + 1,), (nx.tensor(0),), max_iterations=5)


def test_while_inside_a_jitted_defn():
    """The loop is cut out of the traced graph: a program before it (initial state + captured
    values), the loop over condition/body programs, a program after it."""
    def f(x, n):
        y = x * 2.0                                                     # computed before the loop, used inside it
        i, acc = defn.while_loop(lambda i, a: nx.less(i, n), lambda i, a: (i + 1, a + y), (nx.tensor(0), x))
        return acc + 1.0, i                                             # the loop's result is used afterwards

    jf = defn.jit(f)
    a, i = jf(nx.tensor([1.0, 2.0, 3.0, 4.0]), nx.tensor(5))
    assert np.array_equal(nx.to_numpy(a), [12.0, 23.0, 34.0, 45.0]) and nx.to_number(i) == 5
    a, i = jf(nx.tensor([1.0, 2.0, 3.0, 4.0]), nx.tensor(0))           # same executable, zero iterations
    assert np.array_equal(nx.to_numpy(a), [2.0, 3.0, 4.0, 5.0]) and nx.to_number(i) == 0

    def two_loops(x):
        (a,) = defn.while_loop(lambda a: nx.less(nx.sum(a), 100.0), lambda a: (a * 2.0,), (x,))
        # the second loop starts from the first one's result and nests a third
        def body(j, b):
            (c,) = defn.while_loop(lambda c: nx.less(nx.reduce_max(c), 1000.0), lambda c: (c * 10.0,), (b,))
            return j + 1, c / 1000.0
        j, b = defn.while_loop(lambda j, b: nx.less(j, 3), body, (nx.tensor(0), a))
        return a, b, j

    a, b, j = defn.jit(two_loops)(nx.tensor([1.0, 2.0]))
    ra = np.array([1.0, 2.0])
    while ra.sum() < 100.0:
        ra = ra * 2.0
    rb = ra.copy()
    for _ in range(3):
        c = rb.copy()
        while c.max() < 1000.0:
            c = c * 10.0
        rb = c / 1000.0
    np.testing.assert_allclose(nx.to_numpy(a), ra)
    np.testing.assert_allclose(nx.to_numpy(b), rb, rtol=1e-6)
    assert nx.to_number(j) == 3


def test_cond_eager_and_inside_a_defn():
    x = nx.tensor([1.0, 2.0, 3.0])
    f = lambda t, p: defn.cond(p, lambda v: v * 2.0, lambda v: v + 1.0, t)
    assert np.array_equal(nx.to_numpy(f(x, nx.tensor(1, "u8"))), [2.0, 4.0, 6.0])
    assert np.array_equal(nx.to_numpy(f(x, nx.tensor(0, "u8"))), [2.0, 3.0, 4.0])
    jf = defn.jit(lambda t: defn.cond(nx.greater(nx.sum(t), 5.0), lambda v: (v * 2.0, nx.sum(v)), lambda v: (v + 1.0, nx.reduce_max(v)), t))
    a, b = jf(x)
    assert np.array_equal(nx.to_numpy(a), [2.0, 4.0, 6.0]) and nx.to_number(b) == 6.0
    a, b = jf(nx.tensor([1.0, 1.0, 1.0]))
    assert np.array_equal(nx.to_numpy(a), [2.0, 2.0, 2.0]) and nx.to_number(b) == 1.0


def test_greedy_decode_loop_over_a_kv_cache():
    T, V, H = 24, 50, 32
    rng = np.random.default_rng(4)
    E = rng.normal(0, 1, (V, H)).astype(np.float32)
    Wq, Wk, Wv = (rng.normal(0, H ** -0.5, (H, H)).astype(np.float32) for _ in range(3))
    Wo = rng.normal(0, 1, (H, V)).astype(np.float32)

    # reference: the same loop in float64 numpy (argmax margins of this seed are > 0.05)
    tokens = np.zeros(T, np.int32)
    tokens[0] = 7
    kc, vc = np.zeros((T, H)), np.zeros((T, H))
    for pos in range(T - 1):
        x = E[tokens[pos]].astype(np.float64)[None]
        q, k, v = x @ Wq, x @ Wk, x @ Wv
        kc[pos], vc[pos] = k[0], v[0]
        s = (q @ kc.T) * H ** -0.5
        s[0, pos + 1:] = -np.inf
        p = np.exp(s - s.max())
        p /= p.sum()
        tokens[pos + 1] = ((x + p @ vc) @ Wo)[0].argmax()

    e, wq, wk, wv, wo = (nx.tensor(a) for a in (E, Wq, Wk, Wv, Wo))

    def step(toks, pos, kcache, vcache):
        tok = nx.slice(toks, [pos], [1])                                   # the current token, by a tensor index
        x = nx.take(e, tok)                                                # {1, H} embedding lookup
        q, k, v = nx.dot(x, wq), nx.dot(x, wk), nx.dot(x, wv)
        kcache = nx.put_slice(kcache, [pos, 0], k)
        vcache = nx.put_slice(vcache, [pos, 0], v)
        s = nx.dot(q, [1], kcache, [1]) * (H ** -0.5)                      # {1, T}
        s = nx.select(nx.less_equal(nx.iota((1, T), axis=1), pos), s, -float("inf"))
        p = nx.exp(s - nx.reduce_max(s, axes=[1], keep_axes=True))
        p = p / nx.sum(p, axes=[1], keep_axes=True)
        logits = nx.dot(x + nx.dot(p, vcache), wo)
        nxt = nx.as_type(nx.argmax(logits, axis=1), "s32")                 # {1}
        return nx.put_slice(toks, [pos + 1], nxt), pos + 1, kcache, vcache

    init = (nx.tensor(np.array([7] + [0] * (T - 1), np.int32)), nx.tensor(0), nx.tensor(np.zeros((T, H), np.float32)),
            nx.tensor(np.zeros((T, H), np.float32)))
    before = dict(defn.loop_stats)
    toks, pos, kcache, vcache = defn.while_loop(lambda t, p, k, v: nx.less(p, T - 1), step, init)
    assert nx.to_number(pos) == T - 1
    # the loop runs on the device several tokens at a time: fewer than one look at the condition per 8 tokens
    syncs = defn.loop_stats["host_syncs"] - before["host_syncs"]
    assert syncs <= (T - 1 + 7) // 8, (syncs, T)
    assert np.array_equal(nx.to_numpy(toks), tokens)
    np.testing.assert_allclose(nx.to_numpy(kcache), kc, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(nx.to_numpy(vcache), vc, rtol=1e-4, atol=1e-5)
