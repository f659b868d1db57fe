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
