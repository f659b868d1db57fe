"""Shared test plumbing: build a program from a python function with the
front-end, evaluate it with the CPU oracle, and compare results."""
import numpy as np

import nx_oracle as O
from nx_b200 import defn, nx, types as T


def host_tensor(value, type):
    """(nested list | ndarray, type) -> host tensor with raw bytes."""
    from nx_b200 import backend
    prev = backend.default_backend()
    backend.set_default_backend(None)
    try:
        return nx.tensor(np.asarray(value, dtype=np.float64) if T.is_float(T.normalize(type)) else np.asarray(value), type)
    finally:
        backend._default["backend"] = prev


def oracle_run(fun, host_args, mode="xla_like"):
    blob, _ = defn.build_program(fun, host_args)
    res = O.run_program(blob, [a.data.raw for a in host_args], mode)
    return blob, res


def to_f64(arr, type):
    return np.asarray(arr, dtype=np.float64)


def assert_exact(got_raw, want_raw, type, what=""):
    """Bit-exact up to NaN payload (Nx.Testing.assert_equal treats NaN == NaN)."""
    t = T.normalize(type)
    g = O.decode(got_raw, t, (-1,))
    w = O.decode(want_raw, t, (-1,))
    if T.is_float(t):
        ok = np.array_equal(g, w, equal_nan=True)
    else:
        ok = np.array_equal(g, w)
    assert ok, f"{what}: got {g[:16]} want {w[:16]}"


def assert_close(got, want, rtol, atol, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    both_nan = np.isnan(got) & np.isnan(want)
    same_inf = np.isinf(want) & (got == want)
    err = np.abs(got - want)
    ok = both_nan | same_inf | (err <= atol + rtol * np.abs(want))
    if not ok.all():
        i = np.argmax(~ok)
        raise AssertionError(f"{what}: {int((~ok).sum())}/{ok.size} outside rtol={rtol} atol={atol}; "
                             f"first at flat {i}: got {got.ravel()[i]!r} want {want.ravel()[i]!r}")
