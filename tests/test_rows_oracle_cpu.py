"""Pins the C restatement of the fused-rows configuration (oracle/rows_oracle.c,
the timed CPU baseline and the checker of the full-size GPU run) against the
numpy oracle, which itself is pinned by the reference's known-answer vectors.

Shapes run from {3,5} to {16,1000}; a further table holds rows with infinities
and NaNs, including the reference's own non-finite argmax rows
(nx/test/nx_test.exs:1746-1798): with several NaNs in a row the sequential scan
of nx/lib/nx/binary_backend.ex:1415-1431 returns the last one, which is what the
C code restates.
"""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import nx_oracle as O
from helpers import assert_close
from nx_b200 import configs, defn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INF, NAN = np.inf, np.nan


def rows_oracle_lib():
    path = os.path.join(ROOT, "oracle", "librows_oracle.so")
    if not os.path.exists(path):
        subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle")], check=True)
    lib = C.CDLL(path)
    lib.rows_oracle.restype = None
    lib.rows_oracle.argtypes = [C.c_void_p, C.c_int64, C.c_int64] + [C.c_void_p] * 7
    return lib


def rows_oracle(x):
    """The seven outputs of the configuration, in the order of configs.fused_rows."""
    x = np.ascontiguousarray(x, np.float32)
    r, c = x.shape
    outs = [np.zeros(r, np.float32), np.zeros((r, c), np.float32), np.zeros(r, np.float32), np.zeros(r, np.float32),
            np.zeros((r, c), np.float32), np.zeros(r, np.int32), np.zeros((r, c), np.float32)]
    rows_oracle_lib().rows_oracle(x.ctypes.data, r, c, *[o.ctypes.data for o in outs])
    return outs


def numpy_oracle(x, mode):
    blob, _ = defn.build_program(configs.fused_rows, [defn.template(x.shape, "f32")])
    return [r[0] for r in O.run_program(blob, [np.ascontiguousarray(x, np.float32).tobytes()], mode)]


@pytest.mark.parametrize("rows,cols", [(3, 5), (1, 1), (4, 8), (7, 129), (16, 1000), (2, 4097)])
def test_c_restatement_matches_the_numpy_oracle(rows, cols):
    x = configs.fused_rows_input(rows, cols, seed=rows * 1000 + cols)
    got = rows_oracle(x)
    want = numpy_oracle(x, "xla_like")
    names = ["max", "exp", "sum", "logsumexp", "softmax", "argmax", "chain"]
    for n, g, w in zip(names, got, want):
        assert g.shape == w.shape, n
        if n == "argmax":
            assert np.array_equal(g, w)
        elif n == "max":
            assert np.array_equal(g, w)
        else:
            # f32 arithmetic on both sides; libm and numpy may differ in the last place of exp/tanh,
            # and the row sums in their order of addition
            assert_close(g, w, 1e-5, 1e-6, f"{n} {rows}x{cols}")


NON_FINITE_ROWS = np.array([
    [1.0, 2.0, INF, 0.0],          # +inf is the maximum; logsumexp is +inf
    [-INF, -INF, -INF, -INF],      # all -inf: max -inf, logsumexp -inf (the max is replaced by 0, nx/lib/nx.ex:18407-18416)
    [-INF, 3.0, -INF, 3.0],        # tie between finite maxima: lowest index
    [NAN, 1.0, 2.0, 3.0],          # one NaN: its index, NaN statistics
    [1.0, NAN, NAN, 2.0],          # several NaNs: the last one (nx/test/nx_test.exs:1778-1798)
    [NAN, NAN, 1.0, -INF],
    [INF, NAN, INF, 0.0],
    [0.0, -0.0, 0.0, -0.0],        # signed zeros compare equal: index 0
], np.float32)


def test_non_finite_rows():
    got = rows_oracle(NON_FINITE_ROWS)
    want = numpy_oracle(NON_FINITE_ROWS, "binary_backend")
    with np.errstate(all="ignore"):
        assert np.array_equal(got[5], want[5]), f"argmax {got[5]} want {want[5]}"
        assert list(got[5]) == [2, 0, 1, 0, 2, 1, 1, 0]
        for i, n in [(0, "max"), (2, "sum"), (3, "logsumexp")]:
            assert_close(got[i], want[i], 1e-6, 0, n)
        for i, n in [(1, "exp"), (4, "softmax"), (6, "chain")]:
            assert_close(got[i], want[i], 1e-6, 1e-7, n)


def test_reference_argmax_table_rows():
    """The non-finite rows of the reference's argmax test (nx/test/nx_test.exs:1774-1798)."""
    from golden.reference_vectors import CASES
    hits = 0
    for c in CASES:
        if "argmax" not in c["name"] or "non-finite" not in c["name"]:
            continue
        for (val, ty), (want, _) in zip(c["args"], c["expect"]):
            x = np.asarray(val, dtype=np.float64).astype(np.float32)
            if x.ndim != 2:
                continue
            hits += 1
            assert list(rows_oracle(x)[5]) == list(np.asarray(want).reshape(-1)), c["cite"]
    assert hits >= 1
