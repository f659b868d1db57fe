"""The reference's known-answer vectors, run on the GPU through the C ABI."""
import numpy as np
import pytest

import nx_oracle as O
from golden.reference_vectors import CASES
from helpers import assert_close, assert_exact, host_tensor
from nx_b200 import backend, defn, nx, types as T

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


@pytest.mark.parametrize("c", CASES, ids=[c["name"] for c in CASES])
def test_golden_on_gpu(c):
    args = [backend.backend_transfer(host_tensor(v, t)) for v, t in c["args"]]
    out = defn.jit(c["fun"])(*args)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    assert len(outs) == len(c["expect"])
    for got, (want, wtype) in zip(outs, c["expect"]):
        wt = T.normalize(wtype)
        assert got.type == wt, c["cite"]
        w = host_tensor(want, wtype)
        assert got.shape == w.shape, c["cite"]
        if c["exact"]:
            assert_exact(nx.to_binary(got), w.data.raw, wtype, c["cite"])
        else:
            assert_close(nx.to_numpy(got), O.decode(w.data.raw, wt, w.shape), 1e-4, 1e-4, c["cite"])


@pytest.mark.parametrize("c", CASES[:12], ids=[c["name"] for c in CASES[:12]])
def test_golden_eager(c):
    """The same functions called eagerly: every Nx call is a one-node program
    (exla/lib/exla/backend.ex:409-431)."""
    args = [backend.backend_transfer(host_tensor(v, t)) for v, t in c["args"]]
    out = c["fun"](*args)
    (want, wtype), = c["expect"]
    w = host_tensor(want, wtype)
    assert out.type == T.normalize(wtype)
    assert_exact(nx.to_binary(out), w.data.raw, wtype, c["cite"])
