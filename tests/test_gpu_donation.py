"""Buffer donation (Nx.donatable): the scenarios of exla/test/exla/defn/donation_test.exs."""
import numpy as np
import pytest

from nx_b200 import backend, defn, nif, nx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def address(t):
    import ctypes as C
    p = C.c_void_p()
    nif.check(nif.lib().nxb200_buffer_device_pointer(t.data.handle, C.byref(p)))
    return p.value


def consumed(t):
    with pytest.raises(RuntimeError, match="deallocated"):
        nx.to_numpy(t)
    return True


def test_donates_a_single_argument_and_consumes_its_buffer():
    x = nx.donatable(nx.tensor([1, 2, 3, 4]))
    where = address(x)
    f = defn.jit(lambda t: t + 1)
    y = f(x)
    assert nx.to_numpy(y).tolist() == [2, 3, 4, 5]
    assert address(y) == where, "an elementwise result is written into the donated buffer"
    assert consumed(x) and not nx.is_donatable(y)


def test_donates_both_args_of_a_two_arg_function():
    x, y = nx.donatable(nx.tensor([1, 2, 3])), nx.donatable(nx.tensor([10, 20, 30]))
    s, d = defn.jit(lambda a, b: (a + b, a - b))(x, y)
    assert nx.to_numpy(s).tolist() == [11, 22, 33] and nx.to_numpy(d).tolist() == [-9, -18, -27]
    assert consumed(x) and consumed(y)


def test_composite_argument_and_partial_marks():
    a, b = nx.donatable(nx.tensor([1, 2])), nx.tensor([3, 4])
    out = defn.jit(lambda m: {"x": m["x"] + 1, "y": m["y"] * 2})({"x": a, "y": b})
    assert nx.to_numpy(out["x"]).tolist() == [2, 3] and nx.to_numpy(out["y"]).tolist() == [6, 8]
    assert consumed(a)
    assert nx.to_numpy(b).tolist() == [3, 4]                       # not donated: still readable


def test_raises_when_no_output_matches():
    with pytest.raises(ValueError, match="no output with matching shape"):
        defn.jit(lambda t: nx.sum(t))(nx.donatable(nx.tensor([1, 2, 3, 4])))
    with pytest.raises(ValueError, match="not used by the computation"):
        defn.jit(lambda t, u: u + 1)(nx.donatable(nx.tensor([1, 2])), nx.tensor([1, 2]))


def test_donating_and_non_donating_calls_use_distinct_executables():
    f = defn.jit(lambda t: t + 1)
    x = nx.tensor([1, 2, 3])
    f(x)
    assert nx.to_numpy(x).tolist() == [1, 2, 3]
    x2 = nx.donatable(nx.tensor([1, 2, 3]))
    f(x2)
    assert consumed(x2)


def test_results_that_cannot_be_written_in_place_get_their_own_buffer():
    """A transposed read of the argument, a product, or a row kernel that reduces: the donated
    buffer is still consumed, the result is correct."""
    rng = np.random.default_rng(5)
    a = rng.normal(0, 1, (32, 32)).astype(np.float32)
    x = nx.donatable(nx.tensor(a))
    y = defn.jit(lambda t: nx.transpose(t) + t)(x)
    np.testing.assert_allclose(nx.to_numpy(y), a.T + a, rtol=1e-6)
    assert consumed(x)
    x = nx.donatable(nx.tensor(a))
    y = defn.jit(lambda t: nx.dot(t, t))(x)
    np.testing.assert_allclose(nx.to_numpy(y), a @ a, rtol=1e-4, atol=1e-4)
    assert consumed(x)
    x = nx.donatable(nx.tensor(a))
    where = address(x)
    y = defn.jit(lambda t: t / nx.sum(nx.exp(t), axes=[1], keep_axes=True))(x)     # row kernel, row kept in registers
    np.testing.assert_allclose(nx.to_numpy(y), a / np.exp(a).sum(axis=1, keepdims=True), rtol=1e-5)
    assert address(y) == where and consumed(x)


def test_kv_cache_step_updates_the_donated_cache_in_place():
    rng = np.random.default_rng(6)
    cache = rng.normal(0, 1, (4, 64, 16)).astype(np.float32)
    new = rng.normal(0, 1, (4, 1, 16)).astype(np.float32)
    step = defn.jit(lambda c, n, p: nx.put_slice(c, [0, p, 0], n))
    c = nx.donatable(nx.tensor(cache))
    where = address(c)
    want = cache.copy()
    for pos in range(5):
        c2 = step(c, nx.tensor(new * (pos + 1)), nx.tensor(pos))
        want[:, pos] = (new * (pos + 1))[:, 0]
        assert address(c2) == where and consumed(c)
        c = nx.donatable(c2)
    np.testing.assert_array_equal(nx.to_numpy(c), want)


def test_window_update_into_a_separate_result_buffer_starts_from_a_copy():
    """The same program run with a result buffer of the caller's choosing (run_into): nothing can be
    taken over, so the result is the argument's data with the window written on top."""
    from nx_b200 import expr as E
    rng = np.random.default_rng(7)
    cache = rng.normal(0, 1, (3, 32, 8)).astype(np.float32)
    new = rng.normal(0, 1, (3, 2, 8)).astype(np.float32)
    tmpl = [defn.template((3, 32, 8), "f32"), defn.template((3, 2, 8), "f32"), defn.template((), "s32")]
    outs, _, params = defn._trace(lambda c, n, p: nx.put_slice(c, [0, p, 0], n), tmpl)
    prog = defn.Program(E.serialize(outs, params, defn.alias_pairs([0], params, outs)))
    assert "written in place" in prog.describe()
    c, n, p = nx.tensor(cache), nx.tensor(new), nx.tensor(31)          # start 31 is clamped to 30
    out = [nx.tensor(np.zeros_like(cache))]
    prog.run_into([c, n, p], out, 0)
    want = cache.copy()
    want[:, 30:32] = new
    np.testing.assert_array_equal(nx.to_numpy(out[0]), want)
    np.testing.assert_array_equal(nx.to_numpy(c), cache)               # run_into consumes nothing
