"""Nx.cumulative_sum / product / min / max, lowered by the front-end to running windows inside blocks, a
reduction per block and the same scan over the blocks' totals: the doctests of nx/lib/nx.ex:11742-11863 and
random rows of every length class against numpy, through the oracle; the programs compile (no GPU needed).
The lowering has not been run on a GPU."""
import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import defn, nx
from nx_b200.grad import grad


def run(fun, x, type, build=True):
    h = host_tensor(x, type)
    blob, _ = defn.build_program(fun, [h])
    launches = defn.Program(blob).launch_count() if build else None
    with np.errstate(all="ignore"):
        value, out_type, _ = O.run_program(blob, [h.data.raw], "xla_like")[0]
    return np.asarray(value), out_type, launches


def test_reference_doctests():
    square = np.arange(9).reshape(3, 3)
    got, type_, _ = run(lambda t: nx.cumulative_sum(t), [1, 2, 3, 4], "s32")
    assert got.tolist() == [1, 3, 6, 10] and type_ == ("s", 32)
    assert run(lambda t: nx.cumulative_sum(t, axis=0), square, "s32")[0].tolist() == [[0, 1, 2], [3, 5, 7], [9, 12, 15]]
    assert run(lambda t: nx.cumulative_sum(t, axis=1), square, "s32")[0].tolist() == [[0, 1, 3], [3, 7, 12], [6, 13, 21]]
    assert run(lambda t: nx.cumulative_sum(t, axis=0, reverse=True), square, "s32")[0].tolist() == [[9, 12, 15], [9, 11, 13], [6, 7, 8]]
    assert run(lambda t: nx.cumulative_sum(t, axis=1, reverse=True), square, "s32")[0].tolist() == [[3, 3, 2], [12, 9, 5], [21, 15, 8]]
    assert run(lambda t: nx.cumulative_product(t), [1, 2, 3, 4], "s32")[0].tolist() == [1, 2, 6, 24]
    assert run(lambda t: nx.cumulative_product(t, axis=0), square, "s32")[0].tolist() == [[0, 1, 2], [0, 4, 10], [0, 28, 80]]
    assert run(lambda t: nx.cumulative_product(t, axis=1), square, "s32")[0].tolist() == [[0, 0, 0], [3, 12, 60], [6, 42, 336]]
    assert run(lambda t: nx.cumulative_product(t, axis=0, reverse=True), square, "s32")[0].tolist() == [[0, 28, 80], [18, 28, 40], [6, 7, 8]]
    assert run(lambda t: nx.cumulative_product(t, axis=1, reverse=True), square, "s32")[0].tolist() == [[0, 2, 2], [60, 20, 5], [336, 56, 8]]


@pytest.mark.parametrize("n", [1, 2, 31, 32, 33, 64, 65, 1000, 1024, 1025, 32000, 50257])
def test_rows_of_every_length_class_against_numpy(n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal((2, n)).astype(np.float32)
    got, type_, launches = run(lambda t: nx.cumulative_sum(t, axis=1), x, "f32")
    assert type_ == ("f", 32) and launches <= 4
    np.testing.assert_allclose(got, np.cumsum(x.astype(np.float64), axis=1), rtol=1e-4, atol=1e-3)
    build = n in (33, 1025)                              # the other operations share the program's shape
    got, _, _ = run(lambda t: nx.cumulative_max(t, axis=1, reverse=True), x, "f32", build)
    np.testing.assert_array_equal(got, np.maximum.accumulate(x[:, ::-1], axis=1)[:, ::-1])
    got, _, _ = run(lambda t: nx.cumulative_min(t, axis=1), x, "f32", build)
    np.testing.assert_array_equal(got, np.minimum.accumulate(x, axis=1))
    got, _, _ = run(lambda t: nx.cumulative_product(t, axis=1), 1 + x * 0.01, "f32", build)
    np.testing.assert_allclose(got, np.cumprod(1 + x.astype(np.float64) * 0.01, axis=1), rtol=1e-3)
    # integers wrap exactly as a running sum at their own width does; the scanned axis need not be the last
    xi = rng.integers(-100, 100, (n, 3)).astype(np.int8)
    got, type_, _ = run(lambda t: nx.cumulative_sum(t, axis=0), xi, "s8", build)
    assert type_ == ("s", 8)
    np.testing.assert_array_equal(got, np.cumsum(xi, axis=0, dtype=np.int8))


def test_the_running_sum_is_differentiable():
    x = np.random.default_rng(0).standard_normal(70)
    w = np.cos(np.arange(70) * 0.3)
    got, _, _ = run(grad(lambda t: nx.sum(nx.cumulative_sum(t) * nx.tensor(w, "f64"))), x, "f64", build=False)
    np.testing.assert_allclose(got, np.cumsum(w[::-1])[::-1], rtol=1e-12)


def test_nucleus_sampling_step_over_a_vocabulary():
    """The decoding step a serving loop runs after the block: the 50 best of 50,257 logits, their softmax,
    the running sum that cuts the nucleus at p = 0.9, and the choice given a uniform draw — one traced
    function, checked against numpy."""
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal((4, 50257)) * 3.0).astype(np.float32)
    draw = rng.uniform(0, 1, (4, 1)).astype(np.float32)

    def step(l, u):
        values, tokens = nx.top_k(l, k=50)
        e = nx.exp(values - nx.reduce_max(values, axes=[1], keep_axes=True))
        p = e / nx.sum(e, axes=[1], keep_axes=True)
        running = nx.cumulative_sum(p, axis=1)
        inside = nx.less(running - p, 0.9)                           # the nucleus: everything before 0.9 is reached
        kept = nx.select(inside, p, 0.0)
        total = nx.reduce_max(nx.select(inside, running, 0.0), axes=[1], keep_axes=True)
        kept_running = nx.select(inside, running, total)              # the running sum of `kept`, without a second scan
        threshold = u * total
        pick = nx.argmax(nx.greater_equal(kept_running, threshold), axis=1, keep_axis=True)      # first position reaching the draw
        return nx.squeeze(nx.take_along_axis(tokens, pick, axis=1), [1]), kept

    hosts = [host_tensor(logits, "f32"), host_tensor(draw, "f32")]
    blob, _ = defn.build_program(step, hosts)
    assert defn.Program(blob).launch_count() >= 1
    (token, token_type, _), (kept, _, _) = O.run_program(blob, [h.data.raw for h in hosts], "xla_like")

    order = np.argsort(-logits, axis=1, kind="stable")[:, :50]
    values = np.take_along_axis(logits, order, axis=1).astype(np.float64)
    p = np.exp(values - values.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    running = np.cumsum(p, axis=1)
    want_kept = np.where(running - p < 0.9, p, 0.0)
    kept_running = np.cumsum(want_kept, axis=1)
    pick = np.argmax(kept_running >= draw * kept_running[:, -1:], axis=1)
    np.testing.assert_allclose(np.asarray(kept), want_kept, rtol=1e-4, atol=1e-6)
    assert token_type == ("s", 32)
    np.testing.assert_array_equal(np.asarray(token), order[np.arange(4), pick])
