"""Tensor-core matrix products (tcgen05 + TMA) against the CPU oracle.

bf16 / f16 products accumulate in f32 on the device; the oracle accumulates the
same bf16 values exactly and rounds once, so the stated bf16 tolerance
(rtol 2e-2, atol 1e-2) is far wider than the observed difference.  Integer
products must be bit-exact.
"""
import numpy as np
import pytest

import nx_oracle as O
from helpers import assert_close
from nx_b200 import backend, defn, nx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def run_both(fun, arrays, types):
    host = []
    for a, t in zip(arrays, types):
        backend.set_default_backend(None)
        host.append(nx.tensor(a, t))
        backend.set_default_backend("b200", 0)
    dev = [backend.backend_transfer(h) for h in host]
    jitted = defn.jit(fun)
    out = jitted(*dev)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    blob, _ = defn.build_program(fun, host)
    ref = O.run_program(blob, [h.data.raw for h in host], "xla_like")
    return [(nx.to_numpy(g), r[0], r[1]) for g, r in zip(outs, ref)]


# the last two have more row tiles than one panel of the tile walk, the final panel being partial
# (200, 320, ..), (130, 576, ..), (96, 288, ..): n is a multiple of 64 / 32 but not of the tile width, so the
# four-dimensional tensor maps of a [k][n] operand and of the result clip whole groups at the right edge
SHAPES = [(128, 256, 64), (1, 8, 8), (130, 260, 72), (257, 513, 136), (64, 1000, 4096), (384, 768, 512),
          (1024, 1024, 1024), (1100, 200, 64), (4500, 2056, 136), (200, 320, 192), (130, 576, 72), (96, 288, 64)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_bf16_dot(m, n, k):
    rng = np.random.default_rng(2)
    a = rng.normal(0, 1 / np.sqrt(k), (m, k)).astype(np.float32)
    b = rng.normal(0, 1, (k, n)).astype(np.float32)
    bt = np.ascontiguousarray(b.T)
    # b given as {k,n} (reduction index strided) and as {n,k} (contiguous)
    for fun, arrs in [(lambda x, y: nx.dot(x, y), [a, b]), (lambda x, y: nx.dot(x, [1], y, [1]), [a, bt])]:
        (g, r, t), = run_both(fun, arrs, ["bf16", "bf16"])
        assert t == ("bf", 16)
        assert_close(g, r, rtol=2e-2, atol=1e-2, what=f"bf16 dot {m}x{n}x{k}")
        # much tighter than the stated tolerance: at most one bf16 ulp (2^-8 relative) away
        assert_close(g, r, rtol=2 ** -7, atol=2 ** -9, what=f"bf16 dot {m}x{n}x{k} (1 ulp)")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (192, 320, 136), (130, 200, 72), (320, 64, 264)])
def test_bf16_dot_with_both_operands_stored_k_first(m, n, k):
    """x^T . w with x stored {k,m} and w stored {k,n}: both operands reach the tensor cores with their
    free index contiguous (the layout of a weight gradient).  m and n a multiple of 64: one TMA copy per
    tile through the four-dimensional map, including tiles whose groups are clipped; otherwise one per 64 rows."""
    rng = np.random.default_rng(9)
    a = rng.normal(0, 1 / np.sqrt(k), (k, m)).astype(np.float32)
    b = rng.normal(0, 1, (k, n)).astype(np.float32)
    (g, r, t), = run_both(lambda x, y: nx.dot(x, [0], y, [0]), [a, b], ["bf16", "bf16"])
    assert g.shape == (m, n)
    assert_close(g, r, rtol=2 ** -7, atol=2 ** -9, what=f"bf16 dot, k-first operands {m}x{n}x{k}")


def test_bf16_dot_uses_tensor_cores():
    prog = defn.compile(lambda x, y: nx.dot(x, y), [defn.template((256, 512), "bf16"), defn.template((512, 256), "bf16")]).program
    assert "gemm" in prog.describe()


@pytest.mark.parametrize("n", [300, 320])
def test_bf16_batched_dot(n):
    rng = np.random.default_rng(3)
    a = rng.normal(0, 0.2, (5, 200, 72)).astype(np.float32)
    b = rng.normal(0, 1, (5, 72, n)).astype(np.float32)
    (g, r, t), = run_both(lambda x, y: nx.dot(x, [2], [0], y, [1], [0]), [a, b], ["bf16", "bf16"])
    assert g.shape == (5, 200, n)
    assert_close(g, r, rtol=2 ** -7, atol=2 ** -9, what="batched bf16 dot")


@pytest.mark.parametrize("m,n,k,out", [(130, 264, 72, "bf16"), (257, 520, 136, "f32"), (64, 1000, 2048, "bf16"), (384, 100, 512, "bf16"),
                                       (3, 200, 136, "f32")])
def test_fused_epilogue_ragged(m, n, k, out):
    """relu(x . w + bias) * gate as one kernel: the epilogue's result leaves through the staged TMA
    store when rows are 16-byte aligned (tiles clipped at both edges) and through per-lane stores otherwise
    (n = 100: 200-byte rows)."""
    rng = np.random.default_rng(6)
    a = rng.normal(0, 1 / np.sqrt(k), (m, k)).astype(np.float32)
    b = rng.normal(0, 1, (k, n)).astype(np.float32)
    bias = rng.normal(0, 0.5, (n,)).astype(np.float32)
    gate = rng.normal(0, 1, (m, n)).astype(np.float32)

    def fun(x, w, c, gt):
        y = nx.max(nx.dot(x, w) + c, 0.0) * gt
        return nx.as_type(y, out)

    types = ["bf16", "bf16", "bf16", "bf16"]
    (g, r, t), = run_both(fun, [a, b, bias, gate], types)
    assert g.shape == (m, n)
    assert_close(g, r, rtol=2e-2, atol=1e-2, what=f"fused epilogue {m}x{n}x{k} -> {out}")
    prog = defn.compile(fun, [defn.template(x.shape, "bf16") for x in (a, b, bias, gate)]).program
    d = prog.describe()
    assert "fused epilogue" in d
    assert ("staged TMA store" in d) == ((n * (2 if out == "bf16" else 4)) % 16 == 0)


def test_f16_dot():
    rng = np.random.default_rng(4)
    a = rng.normal(0, 0.1, (200, 264)).astype(np.float32)
    b = rng.normal(0, 1, (264, 136)).astype(np.float32)
    (g, r, t), = run_both(lambda x, y: nx.dot(x, y), [a, b], ["f16", "f16"])
    assert_close(g, r, rtol=2 ** -10, atol=2 ** -11, what="f16 dot")


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (33, 50, 304), (300, 520, 4096)])
def test_s8_dot_exact(m, n, k):
    rng = np.random.default_rng(5)
    a = rng.integers(-127, 128, (m, k))
    b = rng.integers(-127, 128, (n, k))
    res = run_both(lambda x, y: (nx.dot(nx.as_type(x, "s32"), [1], nx.as_type(y, "s32"), [1]), nx.dot(x, [1], y, [1])),
                   [a, b], ["s8", "s8"])
    for g, r, t in res:
        assert np.array_equal(g, r), f"s8 dot {m}x{n}x{k} -> {t}"


def test_quantised_linear():
    """y = x . (as_type(W, f32) * scale)^T with W s8 {N,K}, per-output-channel f32 scales, x bf16 {M,K}."""
    rng = np.random.default_rng(3)
    n, k = 704, 512
    w = rng.integers(-127, 128, (n, k))
    scale = rng.uniform(1e-3, 2e-2, (n,)).astype(np.float32)
    for m in (1, 16, 256):
        x = rng.normal(0, 1, (m, k)).astype(np.float32)

        def linear(x, w, s):
            wdq = nx.as_type(w, "f32") * nx.reshape(s, (n, 1))
            return nx.dot(x, [1], wdq, [1])

        (g, r, t), = run_both(linear, [x, w, scale], ["bf16", "s8", "f32"])
        assert t == ("f", 32) and g.shape == (m, n)
        # f32 sums of 512 products of size ~1: the absolute floor is 1e-5 of the output's scale
        assert_close(g, r, rtol=1e-5, atol=1e-5 * float(np.abs(r).max()), what=f"dequant linear M={m}")
