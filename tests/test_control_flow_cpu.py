"""`while`, `cond`, hooks and host calls inside a traced function, end to end without a GPU: the runner
that cuts the traced graph into programs (`defn._make_runner`) is run with the oracle as the executor of
every program, and its results are compared with the same computation written directly in numpy.

What this covers that the plan-level tests do not: the values that flow between the programs (initial
state, captured values from one and from several levels up, results entering later programs as
parameters), the look-ahead step program of a loop (several iterations queued per look at the condition),
hooks firing per iteration and per taken branch, and a host function between two programs."""
import random

import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import backend as B
from nx_b200 import defn, nx, types as T


@pytest.fixture
def on_the_oracle(monkeypatch):
    """Every program of the runner is interpreted by the oracle; tensors stay on the host."""
    def run(self, args, device=0):
        res = O.run_program(self.blob, [a.data.raw for a in args], "xla_like")
        return [host_tensor(np.asarray(v), T.short(t)) for v, t, _raw in res]

    monkeypatch.setattr(defn.Program, "run", run)
    monkeypatch.setattr(B, "backend_transfer", lambda t, device=None: t)

    def run_traced(fun, arrays, types, hooks=None):
        host = [host_tensor(a, t) for a, t in zip(arrays, types)]
        outs, _, params = defn._trace(fun, host)
        return [nx.to_numpy(r) for r in defn._make_runner(outs, params, None, hooks or {})(host, 0)]
    return run_traced


F = np.float32


def test_counted_loop_with_a_captured_value(on_the_oracle):
    def f(x, n):
        i, acc = defn.while_loop(lambda i, acc: nx.less(i, n), lambda i, acc: (i + 1, acc * 2.0 + x),
                                 (nx.tensor(0, "s32"), nx.broadcast(nx.tensor(0.0, "f32"), (3,))))
        return acc, i
    before = dict(defn.loop_stats)
    acc, i = on_the_oracle(f, [np.array([1, 2, 3], F), np.array(5, np.int32)], ["f32", "s32"])
    np.testing.assert_array_equal(acc, np.array([31, 62, 93], F))
    assert int(i) == 5
    # five iterations took one look at the condition: the steps were queued eight at a time
    assert defn.loop_stats["host_syncs"] - before["host_syncs"] == 1


@pytest.mark.parametrize("bound_uses_i,init_uses_s,body_uses_x", [(a, b, c) for a in (0, 1) for b in (0, 1) for c in (0, 1)])
def test_nested_loops_capture_from_every_level(on_the_oracle, bound_uses_i, init_uses_s, body_uses_x):
    """The inner loop reads the outer loop's counter (one level up) and the function's argument (two
    levels up, through the outer body's own parameters)."""
    def g(x):
        def outer(i, s):
            bound = (lambda j, t: nx.less(j, i + 1)) if bound_uses_i else (lambda j, t: nx.less(j, 2))
            step = (lambda j, t: (j + 1, t + x)) if body_uses_x else (lambda j, t: (j + 1, t + 1.0))
            _, t = defn.while_loop(bound, step, (nx.tensor(0, "s32"), s if init_uses_s else s * 0.0 + 1.0))
            return i + 1, t
        return defn.while_loop(lambda i, s: nx.less(i, 3), outer, (nx.tensor(0, "s32"), x * 0.0))[1]

    x = np.array([1.0, 10.0], F)
    s = x * 0
    for i in range(3):
        t = s if init_uses_s else s * 0 + 1
        for _ in range(i + 1 if bound_uses_i else 2):
            t = t + (x if body_uses_x else 1.0)
        s = t
    np.testing.assert_array_equal(on_the_oracle(g, [x], ["f32"])[0], s)


def test_consecutive_loops_and_code_between_them(on_the_oracle):
    def f(x):
        _, a = defn.while_loop(lambda i, a: nx.less(i, 3), lambda i, a: (i + 1, a + x), (nx.tensor(0, "s32"), x))
        mid = nx.tanh(a) * 2.0
        _, b = defn.while_loop(lambda i, b: nx.less(i, 2), lambda i, b: (i + 1, b * mid + a), (nx.tensor(0, "s32"), mid))
        return b + a, mid
    x = np.array([0.25, -0.5, 1.0], F)
    a = x * 4
    mid = (np.tanh(a) * 2).astype(F)
    b = mid
    for _ in range(2):
        b = b * mid + a
    got_b, got_mid = on_the_oracle(f, [x], ["f32"])
    np.testing.assert_allclose(got_mid, mid, rtol=1e-6)
    np.testing.assert_allclose(got_b, b + a, rtol=1e-5)


def test_data_dependent_loop_with_a_cond_in_its_body(on_the_oracle):
    """Collatz steps on every element until all are 1 (a cond on a reduced predicate picks the update)."""
    def f(x):
        def body(n, v):
            even = nx.equal(nx.remainder(v, 2), 0)
            nxt = nx.select(nx.equal(v, 1), v, nx.select(even, nx.quotient(v, 2), v * 3 + 1))
            bump = defn.cond(nx.greater(nx.reduce_max(nxt), 100), lambda c: c + 100, lambda c: c + 1, n)
            return bump, nxt
        return defn.while_loop(lambda n, v: nx.any(nx.not_equal(v, 1)), body, (nx.tensor(0, "s32"), x))
    x = np.array([6, 7, 27, 1], np.int32)
    n, v = 0, x.copy()
    while np.any(v != 1):
        v = np.where(v == 1, v, np.where(v % 2 == 0, v // 2, v * 3 + 1))
        n += 100 if v.max() > 100 else 1
    got_n, got_v = on_the_oracle(f, [x], ["s32"])
    assert int(got_n) == n and np.array_equal(got_v, v)


def test_hooks_fire_once_per_iteration_and_only_in_the_branch_taken(on_the_oracle):
    in_loop, in_then, in_else = [], [], []

    def f(x, flag):
        def body(i, s):
            return i + 1, defn.io_call(s + x, lambda v: in_loop.append(nx.to_numpy(v).copy()))
        _, s = defn.while_loop(lambda i, s: nx.less(i, 4), body, (nx.tensor(0, "s32"), x))
        return defn.cond(flag, lambda t: defn.io_call(t * 2.0, lambda v: in_then.append(nx.to_numpy(v).copy())),
                         lambda t: defn.io_call(t - 1.0, lambda v: in_else.append(nx.to_numpy(v).copy())), s)

    x = np.array([1.0, 2.0], F)
    out, = on_the_oracle(f, [x, np.array(1, np.uint8)], ["f32", "u8"])
    np.testing.assert_array_equal(out, x * 10)
    assert [v.tolist() for v in in_loop] == [(x * k).tolist() for k in (2, 3, 4, 5)]
    assert [v.tolist() for v in in_then] == [(x * 10).tolist()] and in_else == []
    out, = on_the_oracle(f, [x, np.array(0, np.uint8)], ["f32", "u8"])
    np.testing.assert_array_equal(out, x * 5 - 1)
    assert len(in_then) == 1 and [v.tolist() for v in in_else] == [(x * 5 - 1).tolist()]


def test_a_host_function_between_two_programs_and_a_loop_after_it(on_the_oracle):
    def f(x):
        y = x * 2.0
        z = defn.runtime_call(y, y, lambda t, opts: nx.tensor(nx.to_numpy(t)[::-1].copy() + opts["add"], "f32"), {"add": 0.5})
        _, w = defn.while_loop(lambda i, w: nx.less(i, 3), lambda i, w: (i + 1, w + z * x), (nx.tensor(0, "s32"), z))
        return w, z
    x = np.array([1.0, 2.0, 3.0], F)
    z = (x * 2)[::-1] + 0.5
    w, got_z = on_the_oracle(f, [x], ["f32"])
    np.testing.assert_array_equal(got_z, z)
    np.testing.assert_allclose(w, z + 3 * z * x, rtol=1e-6)


# ---- random loop bodies -----------------------------------------------------------------------------

OPS = [("add", lambda p, q: p + q), ("subtract", lambda p, q: p - q), ("multiply", lambda p, q: p * q),
       ("max", np.maximum), ("min", np.minimum)]


def _random_loop(seed):
    """A function with a loop whose body mixes its two state vectors, its counter and values captured from
    the enclosing function (an argument and something computed before the loop), optionally through an
    inner loop — and the same thing in numpy."""
    rng = random.Random(seed)
    trips, inner_trips = rng.randint(0, 11), rng.randint(1, 3)
    picks = [(rng.randrange(5), rng.randrange(5), rng.randrange(len(OPS))) for _ in range(rng.randint(2, 6))]
    with_inner = rng.random() < 0.5

    def body_values(a, b, x, y, i, lib):
        vals = [a, b, x, y, i]
        for p, q, k in picks:
            name, twin = OPS[k]
            made = (getattr(nx, name) if lib is nx else twin)(vals[p], vals[q])
            vals.append(lib.tanh(made) if lib is nx else np.tanh(made).astype(F))
        return vals[-1], vals[-2]

    def fun(x, n):
        y = nx.cos(x) * 0.5

        def body(i, a, b):
            fi = nx.as_type(i, "f32") * 0.125
            na, nb = body_values(a, b, x, y, nx.broadcast(fi, a.shape), nx)
            if with_inner:
                _, na = defn.while_loop(lambda j, t: nx.less(j, inner_trips), lambda j, t: (j + 1, t * 0.5 + y + fi),
                                        (nx.tensor(0, "s32"), na))
            return i + 1, na, nb
        return defn.while_loop(lambda i, a, b: nx.less(i, n), body, (nx.tensor(0, "s32"), x, x * 0.0 + 1.0))

    def twin(x, n):
        y = (np.cos(x) * F(0.5)).astype(F)
        a, b = x, (x * 0 + 1).astype(F)
        for i in range(int(n)):
            fi = F(i) * F(0.125)
            na, nb = body_values(a, b, x, y, np.full(a.shape, fi, F), np)
            if with_inner:
                for _ in range(inner_trips):
                    na = (na * F(0.5) + y + fi).astype(F)
            a, b = na.astype(F), nb.astype(F)
        return int(n), a, b

    x = np.random.default_rng(seed).standard_normal(rng.choice([1, 3, 8])).astype(F)
    return fun, twin, x, np.array(trips, np.int32)


@pytest.mark.parametrize("seed", range(30))
def test_random_loop_matches_its_numpy_statement(on_the_oracle, seed):
    fun, twin, x, n = _random_loop(seed)
    i, a, b = on_the_oracle(fun, [x, n], ["f32", "s32"])
    want_i, want_a, want_b = twin(x, n)
    assert int(i) == want_i
    np.testing.assert_allclose(a, want_a, rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(b, want_b, rtol=2e-5, atol=1e-6)
