"""Integer semantics of the front-end and the oracle (wrapping arithmetic, bit operations, shifts,
conversions between widths and signs, comparisons, sums in the aggregate type) against numpy's fixed-width
integers on random compositions over all eight integer types, with the extreme values of every type among
the inputs.  Mixed types are merged by the reference's rule (`Nx.Type.merge`) before numpy computes."""
import random

import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import defn, nx, types as T

NP = {"u8": np.uint8, "u16": np.uint16, "u32": np.uint32, "u64": np.uint64, "s8": np.int8, "s16": np.int16, "s32": np.int32, "s64": np.int64}
OPS = {"add": np.add, "subtract": np.subtract, "multiply": np.multiply, "bitwise_and": np.bitwise_and, "bitwise_or": np.bitwise_or,
       "bitwise_xor": np.bitwise_xor, "max": np.maximum, "min": np.minimum}
CMP = {"equal": np.equal, "less": np.less, "greater_equal": np.greater_equal, "not_equal": np.not_equal}


def npt(t):
    return NP[T.short(t)]


def _xla_quotient(a, b):
    """Truncating division in Python integers, wrapped to the width; x / 0 is all ones, as XLA defines it."""
    info = np.iinfo(a.dtype)
    out = []
    for p, q in zip(a.ravel().tolist(), b.ravel().tolist()):
        v = -1 if q == 0 else abs(p) // abs(q) * (1 if (p < 0) == (q < 0) else -1)
        out.append((v - info.min) % (1 << info.bits) + info.min)
    return np.array(out, dtype=object).astype(a.dtype).reshape(a.shape)


def _xla_remainder(a, b):
    out = [p if q == 0 else (abs(p) % abs(q)) * (1 if p >= 0 else -1) for p, q in zip(a.ravel().tolist(), b.ravel().tolist())]
    return np.array(out, dtype=object).astype(a.dtype).reshape(a.shape)


def _xla_pow(a, b):
    info = np.iinfo(a.dtype)
    out = []
    for p, q in zip(a.ravel().tolist(), b.ravel().tolist()):
        v = pow(p, q) if q >= 0 else (1 if p == 1 else ((-1 if q % 2 else 1) if p == -1 else 0))
        out.append((v - info.min) % (1 << info.bits) + info.min)
    return np.array(out, dtype=object).astype(a.dtype).reshape(a.shape)


DIVISIONS = {"quotient": _xla_quotient, "remainder": _xla_remainder, "pow": _xla_pow}


def _case(seed):
    r = random.Random(seed)
    rng = np.random.default_rng(seed)
    n = r.choice([1, 5, 8])
    arrays, types = [], []
    for _ in range(r.randint(2, 3)):
        t = r.choice(list(NP))
        info = np.iinfo(NP[t])
        a = rng.integers(info.min, info.max, n, dtype=NP[t], endpoint=True)
        if r.random() < 0.5:
            a[: max(1, n // 3)] = r.choice([info.min, info.max, 0, 1])
        arrays.append(a)
        types.append(t)
    steps, op_seed = r.randint(1, 8), seed * 7 + 1
    expected = []

    def fun(*tensors):
        rr = random.Random(op_seed)
        vals = list(zip(tensors, arrays))
        for _ in range(steps):
            (x, a), (y, b) = rr.choice(vals), rr.choice(vals)
            kind = rr.choice(["op", "op", "cmp", "cast", "neg", "abs", "sum", "not", "shift", "division"])
            if kind == "op":
                name = rr.choice(list(OPS))
                out = npt(T.merge(x.type, y.type))
                vals.append((getattr(nx, name)(x, y), OPS[name](a.astype(out), b.astype(out)).astype(out)))
            elif kind == "cmp":
                name = rr.choice(list(CMP))
                out = npt(T.merge(x.type, y.type))
                vals.append((getattr(nx, name)(x, y), CMP[name](a.astype(out), b.astype(out)).astype(np.uint8)))
            elif kind == "division":
                name = rr.choice(list(DIVISIONS))
                out = npt(T.merge(x.type, y.type))
                p, q = np.broadcast_arrays(a.astype(out), b.astype(out))
                if name == "pow":                      # small exponents (the low bits mean the same in every type)
                    y, q = nx.bitwise_and(y, 3), q & np.array(3, q.dtype)
                vals.append((getattr(nx, name)(x, y), DIVISIONS[name](p, q)))
            elif kind == "cast":
                t = rr.choice(list(NP))
                vals.append((nx.as_type(x, t), a.astype(NP[t])))
            elif kind == "neg":
                vals.append((nx.negate(x), (np.zeros_like(a) - a).astype(a.dtype)))
            elif kind == "abs":
                vals.append((nx.abs(x), np.abs(a) if a.dtype.kind == "i" else a))
            elif kind == "not":
                vals.append((nx.bitwise_not(x), np.bitwise_not(a)))
            elif kind == "shift":
                # by a number: the operands are merged to a signed type for unsigned tensors, and the shift of
                # an unsigned RESULT is still logical (exla/lib/exla/defn.ex:1328-1335)
                k = rr.randint(0, a.dtype.itemsize * 8 - 1)
                name = rr.choice(["left_shift", "right_shift"])
                twin = np.left_shift if name == "left_shift" else np.right_shift
                vals.append((getattr(nx, name)(x, k), twin(a, np.array(k, a.dtype)).astype(a.dtype)))
            else:
                out = npt(T.to_aggregate(x.type))
                vals.append((nx.sum(x), np.sum(a.astype(out), dtype=out)))
        made = vals[len(tensors):]
        del expected[:]
        expected.extend(w for _, w in made)
        return tuple(v for v, _ in made)

    host = [host_tensor(a, t) for a, t in zip(arrays, types)]
    with np.errstate(all="ignore"):
        blob, _ = defn.build_program(fun, host)
        results = O.run_program(blob, [h.data.raw for h in host], "xla_like")
    return results, list(expected)


@pytest.mark.parametrize("seed", range(400))
def test_integer_results_are_numpys_fixed_width_results(seed):
    results, expected = _case(seed)
    assert len(results) == len(expected)
    for (value, type_, _raw), want in zip(results, expected):
        want = np.asarray(want)
        assert npt(type_) == want.dtype, (type_, want.dtype)
        np.testing.assert_array_equal(np.asarray(value).astype(want.dtype), want)


def test_right_shift_of_an_unsigned_result_is_logical_whatever_the_operands_were_merged_to():
    a = np.array([2**64 - 1, 2**63, 5, 2**63 + 12345], dtype=np.uint64)
    h = host_tensor(a, "u64")
    for k in (0, 1, 58, 63, 64, 200):
        blob, _ = defn.build_program(lambda x: nx.right_shift(x, k), [h])
        defn.Program(blob)                                   # the generated kernel compiles
        got = O.run_program(blob, [h.data.raw], "xla_like")[0][0]
        np.testing.assert_array_equal(got, (a >> np.uint64(k)) if k < 64 else np.zeros_like(a))


def test_zero_divisors_negative_exponents_and_the_most_negative_value():
    """What XLA defines where Elixir's integers raise: x / 0 is all ones, x rem 0 is x, the most negative
    value divided by -1 is itself, and a negative exponent gives 1, +-1 or 0 by the base."""
    a = np.array([-128, 127, -7, 0, 7, -7, 1, -1, -1, 5], dtype=np.int8)
    b = np.array([-1, 0, 2, 0, -2, -2, -3, -3, -4, -1], dtype=np.int8)
    ha, hb = host_tensor(a, "s8"), host_tensor(b, "s8")
    for name, want in [("quotient", [-128, -1, -3, -1, -3, 3, 0, 0, 0, -5]), ("remainder", [0, 127, -1, 0, 1, -1, 1, -1, -1, 0]),
                       ("pow", [0, 1, 49, 1, 0, 0, 1, -1, 1, 0])]:
        blob, _ = defn.build_program(lambda x, y: getattr(nx, name)(x, y), [ha, hb])
        defn.Program(blob)
        np.testing.assert_array_equal(O.run_program(blob, [ha.data.raw, hb.data.raw], "xla_like")[0][0], np.array(want, np.int8), name)
    u = host_tensor(np.array([200, 0, 7], np.uint8), "u8")
    z = host_tensor(np.array([0, 0, 2], np.uint8), "u8")
    blob, _ = defn.build_program(lambda x, y: (nx.quotient(x, y), nx.remainder(x, y)), [u, z])
    q, r = (o[0] for o in O.run_program(blob, [u.data.raw, z.data.raw], "xla_like"))
    np.testing.assert_array_equal(q, np.array([255, 255, 3], np.uint8))
    np.testing.assert_array_equal(r, np.array([200, 0, 1], np.uint8))


@pytest.mark.parametrize("src", ["f32", "f64", "bf16", "f16"])
def test_float_to_integer_conversion_truncates_and_saturates(src):
    """NaN becomes 0, anything at or beyond a limit becomes the limit (the limits of the 64-bit types are
    not representable as floats), everything else loses its fraction: exla/test/exla/defn/expr_test.exs:1117-1130."""
    rng = np.random.default_rng(0)
    special = [np.nan, np.inf, -np.inf, 0.0, -0.0, 0.5, -0.5, 0.999, -0.999, 1.5, -1.5, 2.5, 127.0, 127.9, 128.0, -128.0,
               -128.9, -129.0, 255.0, 255.5, 256.0, 32767.5, -32768.5, 65535.9, 65536.0, 2147483647.0, 2147483648.0,
               -2147483648.0, -2147483904.0, 4294967295.0, 4294967296.0, 9.2233720368547758e18, -9.2233720368547758e18,
               1.8446744073709552e19, 1e30, -1e30, 3e-40, 123456.789]
    values = np.concatenate([special, rng.standard_normal(200) * rng.choice([1, 1e3, 1e6, 1e10, 1e19], 200)])
    with np.errstate(all="ignore"):
        x = values.astype({"f32": np.float32, "f64": np.float64, "bf16": np.float32, "f16": np.float16}[src])
    if src == "bf16":
        x = (x.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    h = host_tensor(x.astype(np.float64), src)
    for dst, dtype in NP.items():
        blob, _ = defn.build_program(lambda t: nx.as_type(t, dst), [h])
        with np.errstate(all="ignore"):
            got = O.run_program(blob, [h.data.raw], "xla_like")[0][0]
        info = np.iinfo(dtype)
        want = [0 if v != v else info.max if v >= info.max else info.min if v <= info.min else int(v)
                for v in x.astype(np.float64).tolist()]
        np.testing.assert_array_equal(got, np.array(want, dtype=object).astype(dtype), f"{src} -> {dst}")
