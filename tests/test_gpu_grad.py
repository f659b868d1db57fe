"""Gradients on the device: the gradient graph of a small classifier runs as fused kernels and
matches the oracle's evaluation of the same graph; a training loop with donated parameters learns."""
import numpy as np
import pytest

import nx_oracle as O
from helpers import assert_close
from nx_b200 import backend, defn, nx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def loss_fn(params, x, y):
    h = nx.max(nx.dot(x, params["w1"]) + params["b1"], 0.0)
    logits = nx.dot(h, params["w2"]) + params["b2"]
    logp = logits - nx.logsumexp(logits, axes=[1], keep_axes=True)
    return nx.negate(nx.mean(nx.sum(logp * y, axes=[1])))


def make(rng, n=256, d=784, hidden=128, classes=10):
    labels = rng.integers(0, classes, n)
    centres = rng.normal(0, 1, (classes, d)).astype(np.float32)
    x = (centres[labels] + rng.normal(0, 1.0, (n, d))).astype(np.float32)
    y = np.eye(classes, dtype=np.float32)[labels]
    params = {"w1": rng.normal(0, 0.05, (d, hidden)).astype(np.float32), "b1": np.zeros(hidden, np.float32),
              "w2": rng.normal(0, 0.05, (hidden, classes)).astype(np.float32), "b2": np.zeros(classes, np.float32)}
    return params, x, y


def host(a):
    backend.set_default_backend(None)
    try:
        return nx.tensor(a, "f32")
    finally:
        backend.set_default_backend("b200", 0)


def test_value_and_grad_matches_the_oracle():
    params, x, y = make(np.random.default_rng(0), n=64)
    step = lambda p, x, y: defn.value_and_grad(lambda p: loss_fn(p, x, y))(p)
    hp, hx, hy = {k: host(v) for k, v in params.items()}, host(x), host(y)
    blob, _ = defn.build_program(step, [hp, hx, hy])
    flat = [hp[k] for k in sorted(hp)] + [hx, hy]
    ref = O.run_program(blob, [h.data.raw for h in flat], "xla_like")
    dev = lambda t: backend.backend_transfer(t)
    loss, grads = defn.jit(step)({k: dev(v) for k, v in hp.items()}, dev(hx), dev(hy))
    assert_close(nx.to_numpy(loss), ref[0][0], rtol=1e-5, atol=1e-6, what="loss")
    for i, k in enumerate(sorted(grads)):
        assert grads[k].shape == params[k].shape
        # sums of 64..784 products: absolute floor scaled to the gradients' size
        assert_close(nx.to_numpy(grads[k]), ref[1 + i][0], rtol=1e-4, atol=2e-6, what=f"d loss / d {k}")
    # and against the closed form in f64
    p64 = {k: v.astype(np.float64) for k, v in params.items()}
    h = np.maximum(x @ p64["w1"] + p64["b1"], 0)
    logits = h @ p64["w2"] + p64["b2"]
    sm = np.exp(logits - logits.max(1, keepdims=True))
    sm /= sm.sum(1, keepdims=True)
    dlogits = (sm - y) / len(x)
    assert_close(nx.to_numpy(grads["w2"]), h.T @ dlogits, rtol=1e-3, atol=1e-6, what="closed form w2")
    dh = dlogits @ p64["w2"].T * (h > 0)
    assert_close(nx.to_numpy(grads["w1"]), x.T.astype(np.float64) @ dh, rtol=1e-3, atol=1e-6, what="closed form w1")


def test_training_loop_with_donated_parameters_learns():
    params, x, y = make(np.random.default_rng(1))

    def sgd(p, x, y):
        loss, g = defn.value_and_grad(lambda p: loss_fn(p, x, y))(p)
        return {k: p[k] - 0.1 * g[k] for k in p}, loss
    step = defn.jit(sgd)
    p = {k: nx.tensor(v) for k, v in params.items()}
    dx, dy = nx.tensor(x), nx.tensor(y)
    losses = []
    for _ in range(30):
        p, loss = step({k: nx.donatable(v) for k, v in p.items()}, dx, dy)
        losses.append(float(nx.to_number(loss)))
    assert losses[0] > 2.0 and losses[-1] < 0.25 * losses[0], losses
    assert all(b <= a * 1.05 for a, b in zip(losses, losses[1:])), losses


def test_scatter_matches_the_oracle_with_repeated_positions():
    """indexed_add / indexed_put at sizes where many updates land on the same element: integer sums are
    exact whatever the order of the atomic adds; float sums agree up to their rounding order."""
    rng = np.random.default_rng(5)
    n, rows, cols = 20000, 300, 64
    idx = np.stack([rng.integers(0, rows, n), rng.integers(0, cols, n)], axis=1).astype(np.int32)
    idx[:50, 0] = rows + 5                                            # outside the target: dropped
    idx[50:60, 1] = -1
    for type, tol in (("s32", None), ("f32", 1e-5), ("s8", None), ("u16", None), ("s64", None), ("bf16", None)):
        kind = np.float32 if type in ("f32", "bf16") else np.int64
        target = rng.integers(-3, 4, (rows, cols)).astype(kind)
        upd = rng.integers(-2, 3, n).astype(kind)                      # small integers: exact in every type
        if type == "u16":
            target, upd = np.abs(target), np.abs(upd)
        if type == "f32":
            upd = upd + rng.normal(0, 0.1, n).astype(np.float32)
        fun = lambda t, i, u: nx.indexed_add(t, i, u)
        args = [(target, type), (idx, "s32"), (upd, type)]
        backend.set_default_backend(None)
        hargs = [nx.tensor(a, t) for a, t in args]
        backend.set_default_backend("b200", 0)
        blob, _ = defn.build_program(fun, hargs)
        (want, _, _), = O.run_program(blob, [h.data.raw for h in hargs], "xla_like")
        got = nx.to_numpy(defn.jit(fun)(*[backend.backend_transfer(h) for h in hargs]))
        if tol is None:
            assert np.array_equal(got, want), f"indexed_add {type}"
        else:
            assert_close(got, want, rtol=tol, atol=1e-5, what=f"indexed_add {type}")
    # rows of a table (one indexed axis), distinct positions so that indexed_put is deterministic
    table = rng.normal(0, 1, (512, 96)).astype(np.float32)
    pos = rng.permutation(512)[:100].astype(np.int64).reshape(100, 1)
    new = rng.normal(0, 1, (100, 96)).astype(np.float32)
    got = nx.to_numpy(defn.jit(lambda t, i, u: nx.indexed_put(t, i, u))(nx.tensor(table), nx.tensor(pos), nx.tensor(new)))
    want = table.copy()
    want[pos[:, 0]] = new
    assert np.array_equal(got, want)


def test_embedding_table_learns():
    """A lookup table trained by gradient descent: the gradient of `take` is a scatter-add into the table
    (nx/lib/nx/defn/grad.ex:970-988).  Checked against the oracle's evaluation of the same gradient graph
    and by the loss going down."""
    rng = np.random.default_rng(9)
    vocab, dim, n, classes = 50, 16, 400, 5
    ids = rng.integers(0, vocab, n).astype(np.int32)
    labels = (ids * 7 + 3) % classes                                  # a function of the id: learnable by the table alone
    y = np.eye(classes, dtype=np.float32)[labels]
    table = rng.normal(0, 0.1, (vocab, dim)).astype(np.float32)
    w = rng.normal(0, 0.3, (dim, classes)).astype(np.float32)

    def loss(table, w, ids, y):
        h = nx.take(table, ids, axis=0)
        logits = nx.dot(nx.tanh(h), w)
        logp = logits - nx.logsumexp(logits, axes=[1], keep_axes=True)
        return nx.negate(nx.mean(nx.sum(logp * y, axes=[1])))

    step = lambda table, w, ids, y: defn.value_and_grad(lambda tw: loss(tw[0], tw[1], ids, y))((table, w))
    backend.set_default_backend(None)
    hargs = [nx.tensor(table), nx.tensor(w), nx.tensor(ids), nx.tensor(y)]
    backend.set_default_backend("b200", 0)
    blob, _ = defn.build_program(step, hargs)
    ref = O.run_program(blob, [h.data.raw for h in hargs], "xla_like")
    dev = [backend.backend_transfer(h) for h in hargs]
    l0, (g_table, g_w) = defn.jit(step)(*dev)
    assert_close(nx.to_numpy(l0), ref[0][0], rtol=1e-5, atol=1e-6, what="loss")
    assert_close(nx.to_numpy(g_table), ref[1][0], rtol=1e-4, atol=1e-6, what="d loss / d table")
    assert_close(nx.to_numpy(g_w), ref[2][0], rtol=1e-4, atol=1e-6, what="d loss / d w")
    unused = np.setdiff1d(np.arange(vocab), ids)
    assert np.all(nx.to_numpy(g_table)[unused] == 0)                  # rows never looked up get no gradient

    def sgd(table, w, ids, y):
        l, (gt, gw) = step(table, w, ids, y)
        return table - 2.0 * gt, w - 2.0 * gw, l
    train = defn.jit(sgd)
    t, ww = dev[0], dev[1]
    losses = []
    for _ in range(60):
        t, ww, l = train(nx.donatable(t), nx.donatable(ww), dev[2], dev[3])
        losses.append(float(nx.to_number(l)))
    assert losses[-1] < 0.5 * losses[0], losses
