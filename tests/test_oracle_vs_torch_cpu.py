"""The oracle's floating-point model (`xla_like`: operands converted to the merged type, arithmetic at that
type's precision with 16-bit types computed in f32 and rounded to nearest even after every operation)
against PyTorch's CPU kernels, which implement the same model independently: bf16 / f16 / f32 / f64
element-wise arithmetic and conversions must agree bit for bit, transcendental functions to a few units in
the last place of the result type (numpy's and PyTorch's f32 functions are each a few units off the exact
value; the 16-bit types see one rounding of an f32 result)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

import nx_oracle as O                                   # noqa: E402
from helpers import host_tensor                         # noqa: E402
from nx_b200 import defn, nx, types as T                # noqa: E402

TORCH = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "f64": torch.float64,
         "s32": torch.int32, "s8": torch.int8, "u8": torch.uint8, "s64": torch.int64}
FLOATS = ["bf16", "f16", "f32", "f64"]


def _values(n, seed, type):
    rng = np.random.default_rng(seed)
    if type in FLOATS:
        v = rng.standard_normal(n) * rng.choice([1e-3, 1.0, 1.0, 30.0, 1e4], n)
        v[:6] = [0.0, -0.0, 1.0, -1.0, 0.333333333, 65504.0 if type != "bf16" else 3.0e38]
        return v
    info = np.iinfo({"s32": np.int32, "s8": np.int8, "u8": np.uint8, "s64": np.int64}[type])
    return rng.integers(max(info.min, -1000), min(info.max, 1000), n, endpoint=True)


def _to_torch(values, type):
    if type in FLOATS:
        return torch.tensor(np.asarray(values, np.float64)).to(TORCH[type])
    return torch.tensor(np.asarray(values, np.int64)).to(TORCH[type])


def _run(fun, arrays, types):
    host = [host_tensor(a, t) for a, t in zip(arrays, types)]
    blob, _ = defn.build_program(fun, host)
    with np.errstate(all="ignore"):
        (value, type_, _raw), = O.run_program(blob, [h.data.raw for h in host], "xla_like")
    # what the host holds is the value after the store into its type; read it back as f64
    return np.asarray(value, dtype=np.float64), T.short(type_)


def _host_values(values, type):
    """The f64 values a tensor of `type` holds after `values` were stored into it (round to nearest even)."""
    return _to_torch(values, type).to(torch.float64).numpy()


@pytest.mark.parametrize("op", ["add", "subtract", "multiply", "divide", "max", "min"])
@pytest.mark.parametrize("left", ["bf16", "f16", "f32", "f64", "s32", "u8"])
@pytest.mark.parametrize("right", ["bf16", "f16", "f32", "f64", "s8"])
def test_mixed_type_arithmetic_is_bit_identical(op, left, right):
    a, b = _values(300, 1, left), _values(300, 2, right)
    a, b = _host_values(a, left), _host_values(b, right)
    got, out_type = _run(lambda x, y: getattr(nx, op)(x, y), [a, b], [left, right])
    merged = T.short(T.merge(T.normalize(left), T.normalize(right)))
    want_type = merged if merged in FLOATS or op != "divide" else "f32"
    assert out_type == want_type
    if want_type not in FLOATS:
        pytest.skip("integer result: covered by the integer test")
    ta, tb = _to_torch(a, left).to(TORCH[want_type]), _to_torch(b, right).to(TORCH[want_type])
    twin = {"add": torch.add, "subtract": torch.sub, "multiply": torch.mul, "divide": torch.div,
            "max": torch.maximum, "min": torch.minimum}[op]
    want = twin(ta, tb).to(torch.float64).numpy()
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("type", FLOATS)
@pytest.mark.parametrize("op", ["exp", "tanh", "sigmoid", "log1p", "sqrt", "rsqrt", "cos", "sin", "erf", "expm1", "log", "atan", "cbrt"])
def test_unary_functions_agree_to_a_few_units_in_the_last_place(op, type):
    x = _host_values(np.abs(_values(400, 3, type)) if op in ("sqrt", "rsqrt", "log") else _values(400, 3, type), type)
    x = x[np.abs(x) < 80] if op in ("exp", "expm1", "cos", "sin") else x
    got, out_type = _run(lambda t: getattr(nx, op)(t), [x], [type])
    assert out_type == type
    t = _to_torch(x, type)
    twin = {"cbrt": lambda v: torch.sign(v) * torch.pow(torch.abs(v.to(torch.float64)), 1.0 / 3.0).to(v.dtype), "rsqrt": torch.rsqrt,
            "erf": torch.erf, "sigmoid": torch.sigmoid}.get(op) or getattr(torch, op)
    want = twin(t).to(torch.float64).numpy()
    if op == "erf" and type in ("bf16", "f16"):
        # PyTorch's 16-bit erf is itself a few units off at small arguments: take the exact value, rounded
        import math
        want = _host_values(np.vectorize(math.erf, otypes=[np.float64])(x), type)
    ulp = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11, "f32": 2.0 ** -24, "f64": 2.0 ** -53}[type] * {"bf16": 4, "f16": 4, "f32": 8, "f64": 8}[type]
    scale = np.maximum(np.abs(want), np.finfo(np.float32).tiny)
    with np.errstate(all="ignore"):
        ok = (np.abs(got - want) <= ulp * scale * 1.01) | (np.isnan(got) & np.isnan(want)) | (got == want)
    tiny = np.abs(want) < {"bf16": 1e-30, "f16": 7e-5, "f32": 1e-36, "f64": 1e-300}[type]      # subnormal results
    assert np.all(ok | tiny), (x[~(ok | tiny)][:5], got[~(ok | tiny)][:5], want[~(ok | tiny)][:5])


@pytest.mark.parametrize("src", FLOATS + ["s32", "s64", "u8"])
@pytest.mark.parametrize("dst", FLOATS)
def test_conversions_between_float_types_round_to_nearest_even(src, dst):
    x = _host_values(_values(500, 4, src), src)
    got, _ = _run(lambda t: nx.as_type(t, dst), [x], [src])
    want = _to_torch(x, src).to(TORCH[dst]).to(torch.float64).numpy()
    np.testing.assert_array_equal(got, want)
