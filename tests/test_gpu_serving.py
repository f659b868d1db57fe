"""Nx.Serving mirror on the GPU: a jitted defn behind the batching server, one partition per
visible GPU (exla/test/exla/serving_test.exs runs the same scenario on EXLA's devices)."""
import threading

import numpy as np
import pytest

from nx_b200 import backend, nif, nx, serving as S

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def softmax_rows(x):
    e = nx.exp(x - nx.reduce_max(x, axes=[-1], keep_axes=True))
    return e / nx.sum(e, axes=[-1], keep_axes=True)


def expected(x):
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def test_run_inline():
    x = np.random.default_rng(0).normal(0, 1, (5, 33)).astype(np.float32)
    out = nx.to_numpy(S.Serving.jit(softmax_rows).batch_size(4).run(S.Batch.concatenate([x])))
    np.testing.assert_allclose(out, expected(x), rtol=1e-5, atol=1e-7)


def test_batched_run_over_all_partitions():
    rng = np.random.default_rng(1)
    s = S.Serving.jit(softmax_rows)
    srv = s.start("softmax", batch_size=8, batch_timeout_ms=20, partitions=True)
    try:
        assert len(srv.workers) == max(1, nif.device_count())
        inputs = [rng.normal(0, 1, (n, 64)).astype(np.float32) for n in (3, 8, 13, 1, 6)]
        outs = [None] * len(inputs)

        def call(i):
            outs[i] = nx.to_numpy(S.batched_run("softmax", S.Batch.concatenate([inputs[i]])))
        ts = [threading.Thread(target=call, args=(i,)) for i in range(len(inputs))]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=120)
        for x, o in zip(inputs, outs):
            assert o is not None and o.shape == x.shape
            np.testing.assert_allclose(o, expected(x), rtol=1e-5, atol=1e-7)
        assert sum(n for _, n, _ in srv.executed) == 31
        assert all(n + pad == 8 for _, n, pad in srv.executed)                  # every execution saw the compiled shape
    finally:
        S.stop("softmax")
