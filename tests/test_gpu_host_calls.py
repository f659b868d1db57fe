"""io_call (hook) and runtime_call on the device: the scenarios of exla/test/exla/defn/api_test.exs:170-380,
exla/test/exla/defn/runtime_call_test.exs and nx/test/nx/defn/grad_test.exs:72-95."""
import numpy as np
import pytest

from nx_b200 import backend, defn, nx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def num(t):
    return nx.to_numpy(t).tolist()


def hook_default(a, b):
    return defn.io_call(a + b, "default", lambda t: DEFAULT.append(num(t)))


DEFAULT = []


def test_default_and_overriding_functions():
    DEFAULT.clear()
    assert num(defn.jit(hook_default)(nx.tensor(2), nx.tensor(3))) == 5 and DEFAULT == [5]
    got, other = [], []
    assert num(defn.jit(hook_default, hooks={"default": lambda t: got.append(num(t))})(nx.tensor(2), nx.tensor(3))) == 5
    assert got == [5] and DEFAULT == [5]
    # executing again with another function works (the functions are part of the compile key)
    assert num(defn.jit(hook_default, hooks={"default": lambda t: other.append(num(t))})(nx.tensor(2), nx.tensor(3))) == 5
    assert other == [5] and got == [5]


def test_optional_tap():
    f = lambda a, b: defn.io_call(a + b, "optional")
    assert num(defn.jit(f)(nx.tensor(2), nx.tensor(3))) == 5
    got = []
    assert num(defn.jit(f, hooks={"optional": lambda t: got.append(num(t))})(nx.tensor(2), nx.tensor(3))) == 5
    assert got == [5]


def test_tap_within_while_sees_every_iteration():
    def factorial(x):
        f, _ = defn.while_loop(lambda f, x: nx.greater(x, 1), lambda f, x: defn.io_call((f * x, x - 1), "factorial"), (nx.tensor(1.0), x))
        return f
    got = []
    out = defn.jit(factorial, hooks={"factorial": lambda pair: got.append((num(pair[0]), num(pair[1])))})(nx.tensor(5))
    assert num(out) == 120.0
    assert got == [(5.0, 4), (20.0, 3), (60.0, 2), (120.0, 1)]


def test_tap_within_cond_fires_in_the_taken_branch_only():
    def f(a, b):
        return defn.cond(nx.equal(a, -1), lambda b: defn.io_call(b * 2, "cond"),
                         lambda b: defn.cond(nx.equal(a, 1), lambda b: defn.io_call(b / 2, "cond"), lambda b: defn.io_call(nx.pow(b, 2), "cond"), b), b)
    got = []
    g = defn.jit(f, hooks={"cond": lambda t: got.append(num(t))})
    assert num(g(nx.tensor(1), nx.tensor(4))) == 2.0 and got == [2.0]
    assert num(g(nx.tensor(-1), nx.tensor(4))) == 8.0 and got == [2.0, 8]
    assert num(g(nx.tensor(0), nx.tensor(4))) == 16.0 and got == [2.0, 8, 16]


def test_container_and_order():
    got = []
    c = {"a": nx.tensor(1), "b": nx.tensor([2.0, 3.0])}
    out = defn.jit(lambda c: defn.io_call(c, "container"), hooks={"container": got.append})(c)
    assert num(out["a"]) == 1 and num(got[0]["a"]) == 1 and num(got[0]["b"]) == [2.0, 3.0]

    def chain(a, b, c):
        a = defn.io_call(a, "a")
        b = defn.io_call(b, "b")
        c = defn.io_call(c, "c")
        return a + c + b
    order = []
    send = lambda t: order.append(num(t))
    assert num(defn.jit(chain, hooks={"a": send, "b": send, "c": send})(nx.tensor(1), nx.tensor(2), nx.tensor(3))) == 6
    assert order == [1, 2, 3]                         # the order the calls were traced in


def test_a_raising_function_surfaces():
    def boom(_):
        raise RuntimeError("boom")
    with pytest.raises(RuntimeError, match="boom"):
        defn.jit(lambda a, b: defn.io_call(a + b, "raises", boom))(nx.tensor(2), nx.tensor(3))


def test_tap_with_gradients():
    got = []
    f = defn.jit(lambda t: defn.value_and_grad(lambda t: defn.io_call(nx.pow(t, 2), "grad"))(t), hooks={"grad": lambda t: got.append(num(t))})
    value, g = f(nx.tensor(3.0))
    assert num(value) == 9.0 and num(g) == 6.0 and got == [9.0]
    got.clear()
    h = defn.jit(lambda t: defn.io_call(defn.grad(lambda t: nx.pow(t, 2))(t), "grad"), hooks={"grad": lambda t: got.append(num(t))})
    assert num(h(nx.tensor(3.0))) == 6.0 and got == [6.0]


# ---- runtime_call ------------------------------------------------------------------------------------

def test_runtime_call_single_output_with_options():
    def add_offset(x):
        out = defn.template(x.shape, "f32")
        return defn.runtime_call(out, x, lambda t, opts: nx.as_type(t, "f32") + opts["offset"], {"offset": 10.0})
    assert num(defn.jit(add_offset)(nx.tensor([0, 1, 2, 3, 4]))) == [10.0, 11.0, 12.0, 13.0, 14.0]


def test_runtime_call_tuple_output_feeds_the_rest_of_the_graph():
    def split_and_sum(x):
        fx = nx.as_type(x, "f32")
        a, b = defn.runtime_call((fx, fx), fx, lambda t, opts: (t * 2.0, t + 1.0))
        return a + b
    assert num(defn.jit(split_and_sum)(nx.tensor([1, 2, 3]))) == [4.0, 7.0, 10.0]


def test_runtime_call_container_input_and_numpy_inside():
    seen = []

    def host(pair, opts):
        x, y = (nx.to_numpy(t) for t in pair)
        seen.append(opts["ref"])
        return {"sum": nx.tensor(x + y), "diff": nx.tensor(x - y)}

    def f(x, y):
        r = defn.runtime_call({"sum": x, "diff": x}, (x * 1, y), host, {"ref": 42})
        return r["sum"] * 10, r["diff"]
    s, d = defn.jit(f)(nx.tensor([1, 2, 3]), nx.tensor([4, 5, 6]))
    assert num(s) == [50, 70, 90] and num(d) == [-3, -3, -3] and seen == [42]


def test_runtime_call_wrong_result_raises():
    bad = lambda x: defn.runtime_call(defn.template(x.shape, "f32"), x, lambda t, opts: nx.tensor([1.0, 2.0, 3.0]))
    with pytest.raises(ValueError, match="expected the runtime_call function to match the given output template"):
        defn.jit(bad)(nx.tensor([0, 1]))


def test_runtime_call_inside_a_loop():
    calls = []

    def body(i, acc):
        acc = defn.runtime_call(acc, acc, lambda t, opts: (calls.append(num(t)), t + 1.0)[1])
        return i + 1, acc * 2.0
    f = lambda x: defn.while_loop(lambda i, acc: nx.less(i, 3), body, (nx.tensor(0), x))[1]
    assert num(defn.jit(f)(nx.tensor(1.0))) == 22.0          # ((1+1)*2+1)*2+1)*2
    assert calls == [1.0, 4.0, 10.0]
