"""Pins the CPU oracle against known-answer vectors from the reference's tests."""
import numpy as np
import pytest

import nx_oracle as O
from golden.reference_vectors import CASES
from helpers import assert_close, assert_exact, host_tensor, oracle_run
from nx_b200 import types as T

PARAMS = [(c, m) for c in CASES for m in c["modes"]]


@pytest.mark.parametrize("c,mode", PARAMS, ids=[f"{c['name']}[{m}]" for c, m in PARAMS])
def test_golden(c, mode):
    args = [host_tensor(v, t) for v, t in c["args"]]
    _, res = oracle_run(c["fun"], args, mode)
    assert len(res) == len(c["expect"])
    for (arr, typ, raw), (want, wtype) in zip(res, c["expect"]):
        wt = T.normalize(wtype)
        assert typ == wt, f"{c['cite']}: type {typ} want {wt}"
        w = host_tensor(want, wtype)
        assert arr.shape == w.shape, f"{c['cite']}: shape {arr.shape} want {w.shape}"
        if c["exact"]:
            assert_exact(raw, w.data.raw, wtype, c["cite"])
        else:
            assert_close(arr, O.decode(w.data.raw, wt, w.shape), 1e-4, 1e-4, c["cite"])
