"""The batching server (nx_b200.serving), the mirror of Nx.Serving / Nx.Batch: stacking of
concurrent callers, splitting, padding, timeouts and partitions, with a numpy function
standing in for the compiled program (scenarios of nx/test/nx/serving_test.exs)."""
import threading
import time

import numpy as np
import pytest

from nx_b200 import serving as S


def double(opts):
    calls = opts.setdefault("calls", [])

    def run(batch):
        calls.append(batch.shape)
        return batch * 2
    return run


def test_batch_stack_concatenate_split_pad_merge():
    b = S.Batch.stack([np.array([1, 2, 3]), np.array([4, 5, 6])])
    assert b.size == 2
    S.Batch.concatenate([np.array([[7, 8, 9]])], b)
    assert b.size == 3
    left, right = b.split(2)
    assert (left.size, right.size) == (2, 1)
    assert np.array_equal(left.materialise(), [[1, 2, 3], [4, 5, 6]])
    assert np.array_equal(right.pad(2).materialise(), [[7, 8, 9], [0, 0, 0], [0, 0, 0]])
    m = S.Batch.merge([left, right])
    assert m.size == 3 and np.array_equal(m.materialise()[:3], [[1, 2, 3], [4, 5, 6], [7, 8, 9]])
    with pytest.raises(ValueError):
        S.Batch.concatenate([np.zeros((1, 4))], S.Batch.stack([np.zeros(3)]))
    tb = S.Batch.stack([(np.array([1.0]), {"k": np.array([2, 3])})])          # containers
    x, d = tb.materialise()
    assert x.shape == (1, 1) and d["k"].shape == (1, 2)


def test_run_inline_splits_by_batch_size_and_applies_client_functions():
    opts = {}
    s = (S.Serving.new(double, **opts).batch_size(2)
         .client_preprocessing(lambda xs: (S.Batch.stack(xs), len(xs)))
         .client_postprocessing(lambda out_meta, info: (out_meta[0], info)))
    out, info = s.run([np.array([1, 2]), np.array([3, 4]), np.array([5, 6])])
    assert info == 3 and np.array_equal(out, [[2, 4], [6, 8], [10, 12]])
    assert s.defn_options["calls"] == [(2, 2), (1, 2)]


def test_batched_run_stacks_concurrent_callers_into_one_execution():
    s = S.Serving.new(double)
    srv = s.start("stack", batch_size=4, batch_timeout_ms=10_000)
    try:
        results = {}

        def call(i, n):
            results[i] = S.batched_run("stack", S.Batch.stack([np.full(3, 10 * i + j) for j in range(n)]))
        ts = [threading.Thread(target=call, args=(i, 2)) for i in range(2)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=20)
        assert srv.executed == [(0, 4, 0)]                                      # one full batch, no padding
        for i in range(2):
            assert np.array_equal(results[i], 2 * np.array([np.full(3, 10 * i), np.full(3, 10 * i + 1)]))
    finally:
        S.stop("stack")


def test_timeout_executes_a_partial_batch_padded_to_the_batch_size():
    s = S.Serving.new(double)
    srv = s.start("timeout", batch_size=8, batch_timeout_ms=50)
    try:
        t0 = time.monotonic()
        out = S.batched_run("timeout", S.Batch.stack([np.arange(4), np.arange(4) + 1]))
        assert time.monotonic() - t0 < 5
        assert np.array_equal(out, [[0, 2, 4, 6], [2, 4, 6, 8]])
        assert srv.executed == [(0, 2, 6)]                                      # 2 entries + 6 rows of padding
        assert s.defn_options == {} or True
    finally:
        S.stop("timeout")


def test_a_large_batch_is_split_across_executions_and_partitions():
    seen = []

    def builder(opts):
        def run(batch):
            seen.append((opts["device"], batch.shape[0]))
            time.sleep(0.05)
            return batch + 1
        return run
    s = S.Serving.new(builder)
    srv = s.start("split", batch_size=3, batch_timeout_ms=20, partition_options=[{"device": 0}, {"device": 1}])
    try:
        x = np.arange(8 * 2).reshape(8, 2)
        out = S.batched_run("split", S.Batch.concatenate([x]))
        assert np.array_equal(out, x + 1)                                       # order restored across pieces
        assert sorted(n for _, n in seen) == [3, 3, 3]                          # 3 + 3 + (2 padded to 3)
        assert {d for d, _ in seen} == {0, 1}                                   # both partitions worked
        assert [e[1:] for e in srv.executed] == [(3, 0), (3, 0), (2, 1)]
    finally:
        S.stop("split")


def test_errors():
    with pytest.raises(ValueError, match="could not find Nx.Serving"):
        S.batched_run("nobody", S.Batch.stack([np.zeros(2)]))

    def boom(opts):
        def run(batch):
            raise RuntimeError("kernel failed")
        return run
    S.Serving.new(boom).start("boom", batch_size=1)
    try:
        with pytest.raises(RuntimeError, match="kernel failed"):
            S.batched_run("boom", S.Batch.stack([np.zeros(2)]))
        with pytest.raises(ValueError, match="already running"):
            S.Serving.new(boom).start("boom", batch_size=1)
    finally:
        S.stop("boom")


def test_many_concurrent_callers_each_get_exactly_their_rows():
    """Eight clients, forty requests each of 1 to 20 entries (up to 2.5 batches), three partitions, a 5 ms
    timeout: every caller's result must be the function of its own rows, in order, whatever the stacking,
    splitting and padding did around them; nobody may be left waiting."""
    import random

    def builder(opts):
        def run(batch):
            time.sleep(0.0005)
            return batch * 2.0 + 1.0, batch.sum(axis=1)
        return run

    srv = S.Serving.new(builder).start("stress", batch_size=8, batch_timeout_ms=5,
                                       partition_options=[{"device": 0}, {"device": 1}, {"device": 2}])
    wrong = []

    def client(cid):
        r = random.Random(cid)
        data = np.random.default_rng(cid)
        for i in range(40):
            n = r.randint(1, 20)
            x = data.standard_normal((n, 5))
            try:
                y, total = S.batched_run("stress", S.Batch.concatenate([x]))
                if y.shape != (n, 5) or not np.array_equal(y, x * 2.0 + 1.0) or not np.allclose(total, x.sum(axis=1)):
                    wrong.append((cid, i, n, y.shape))
            except Exception as e:          # noqa: BLE001 - reported below
                wrong.append((cid, i, repr(e)))
            if r.random() < 0.3:
                time.sleep(r.random() * 0.004)

    try:
        clients = [threading.Thread(target=client, args=(c,)) for c in range(8)]
        for t in clients:
            t.start()
        for t in clients:
            t.join(timeout=60)
        assert not [t for t in clients if t.is_alive()], "a caller never got its result"
        assert not wrong, wrong[:3]
        assert {p for p, _, _ in srv.executed} == {0, 1, 2}
        assert all(size + pad == 8 or pad == 0 for _, size, pad in srv.executed)
    finally:
        S.stop("stress")
