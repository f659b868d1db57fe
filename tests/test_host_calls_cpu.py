"""io_call (hook) and runtime_call: what does not need a GPU — the behaviour outside a traced function,
the template check, and how a traced graph is lowered (extra results for taps, a cut at a host call)."""
import numpy as np
import pytest

from helpers import host_tensor
from nx_b200 import defn, nx


def test_outside_a_traced_function_the_functions_are_simply_called():
    # nx/lib/nx.ex:2366-2391
    seen = []
    x = host_tensor([1, 2, 3], "s32")
    out = defn.runtime_call(defn.template((3,), "s32"), x, lambda t, opts: (seen.append(opts["tag"]), t)[1], {"tag": "hello"})
    assert out is x and seen == ["hello"]
    assert defn.io_call(x, seen.append) is x and seen[-1] is x
    assert defn.io_call(x, "nobody_listens") is x


def test_result_must_match_the_template():
    x = host_tensor([1, 2, 3], "s32")
    with pytest.raises(ValueError, match="expected the runtime_call function to match the given output template"):
        defn.runtime_call(defn.template((2,), "s32"), x, lambda t, opts: t)
    with pytest.raises(ValueError, match="expected the runtime_call function to match the given output template"):
        defn.runtime_call((defn.template((3,), "s32"),) * 2, x, lambda t, opts: t)


def test_taps_become_extra_results_of_one_program():
    def f(a, b):
        return defn.io_call(a + b, "add"), defn.io_call(nx.exp(a) * b, "mult"), defn.io_call(a - b, "unheard")
    outs, _, params = defn._trace(f, [host_tensor([1.0, 2.0], "f32"), host_tensor([3.0, 4.0], "f32")])
    run = defn._make_runner(outs, params, None, {"add": print, "mult": print})
    plan = run.program.describe().splitlines()
    assert len(plan) == 1, plan                       # the tapped values are results already: nothing is computed twice
    # a tap on an intermediate adds a result, still one kernel
    g = lambda a, b: nx.sum(defn.io_call(a * b, "prod"))
    outs, _, params = defn._trace(g, [host_tensor([1.0, 2.0], "f32"), host_tensor([3.0, 4.0], "f32")])
    heard = defn._make_runner(outs, params, None, {"prod": print}).program
    silent = defn._make_runner(outs, params, None, {}).program
    assert len(heard.outputs) == 2 and len(silent.outputs) == 1
    assert len(heard.describe().splitlines()) == 1


def test_a_host_call_cuts_the_graph():
    def f(x):
        fx = nx.as_type(x, "f32")
        a, b = defn.runtime_call((fx, fx), fx, lambda t, opts: (t * 2.0, t + 1.0))
        return a + b
    outs, _, params = defn._trace(f, [host_tensor([1, 2, 3], "s32")])
    assert [o.shape for o in outs] == [(3,)] and outs[0].type == ("f", 32)
    run = defn._make_runner(outs, params, None, {})
    assert run.program is None                        # several programs with the host function between them


def test_cond_branches_are_brought_to_a_common_type():
    # nx/lib/nx/defn/expr.ex:251-290; exla/test/exla/defn/api_test.exs:246-278 relies on it
    f = lambda a, b: defn.cond(nx.equal(a, 1), lambda b: b / 2, lambda b: nx.pow(b, 2), b)
    outs, _, _ = defn._trace(f, [host_tensor(1, "s32"), host_tensor(4, "s32")])
    assert outs[0].type == ("f", 32) and outs[0].shape == ()
