"""The five configurations on the GPU at reduced sizes, against the CPU oracle,
plus size-independent properties at larger sizes."""
import numpy as np
import pytest

import nx_oracle as O
from helpers import assert_close
from nx_b200 import backend, configs, defn, nx

pytestmark = pytest.mark.gpu
BF16 = dict(rtol=2e-2, atol=1e-2)


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def run_both(fun, inputs, mode="xla_like"):
    host = []
    for a, t in inputs:
        backend.set_default_backend(None)
        host.append(nx.tensor(a, t))
        backend.set_default_backend("b200", 0)
    dev = [backend.backend_transfer(h) for h in host]
    out = defn.jit(fun)(*dev)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    blob, _ = defn.build_program(fun, host)
    ref = O.run_program(blob, [h.data.raw for h in host], mode)
    return [(nx.to_numpy(g), r[0], r[1]) for g, r in zip(outs, ref)]


def test_concatenate_and_slices():
    rng = np.random.default_rng(20)
    a = rng.normal(0, 1, (3, 5, 8)).astype(np.float32)
    b = rng.normal(0, 1, (3, 2, 8)).astype(np.float32)
    c = rng.integers(-5, 5, (3, 5, 4))

    def f(a, b, c):
        return (nx.concatenate([a, b], axis=1), nx.concatenate([a, c, a * 2.0], axis=2),
                nx.concatenate([nx.negate(nx.slice_along_axis(a, 4, 4, axis=2)), nx.slice_along_axis(a, 0, 4, axis=2)], axis=2) + 1.0)

    for g, r, t in run_both(f, [(a, "f32"), (b, "f32"), (c, "s32")]):
        assert_close(g, r, rtol=1e-6, atol=0, what="concatenate")


def test_rope_tables_and_rotation():
    rng = np.random.default_rng(21)
    t = rng.normal(0, 1, (2, 3, 16, 8)).astype(np.float32)

    def f(t):
        cos, sin = configs.rope_tables(16, 8, 10000.0, "f32")
        return configs.rope(t, cos, sin), cos, sin

    for g, r, _ in run_both(f, [(t, "f32")]):
        assert_close(g, r, rtol=1e-5, atol=2e-6, what="rope")


def test_rms_norm_bf16():
    rng = np.random.default_rng(22)
    x = rng.normal(0, 1, (4, 33, 512)).astype(np.float32)
    gain = (1 + rng.normal(0, 0.02, (512,))).astype(np.float32)
    (g, r, t), = run_both(lambda x, g: configs.rms_norm(x, g), [(x, "bf16"), (gain, "bf16")])
    assert_close(g, r, what="rms_norm", **BF16)


@pytest.mark.parametrize("batch,seq,hidden,heads,inter", [(2, 16, 64, 4, 176), (1, 64, 256, 4, 344), (2, 128, 512, 8, 688),
                                                          (1, 256, 512, 4, 688), (2, 200, 256, 2, 344), (1, 640, 384, 3, 344)])
def test_decoder_block(batch, seq, hidden, heads, inter):
    block = configs.make_decoder_block(n_heads=heads)
    inputs = configs.decoder_inputs(batch=batch, seq=seq, hidden=hidden, inter=inter)
    (g, r, t), = run_both(block, inputs)
    assert t == ("bf", 16) and g.shape == (batch, seq, hidden)
    assert np.isfinite(g).all()
    assert_close(g, r, what="decoder block", **BF16)


def _attention(q, k, v, causal=True, scale=0.0884):
    s = nx.dot(q, [3], [0, 1], k, [3], [0, 1]) * scale
    if causal:
        sq, sk = s.shape[2], s.shape[3]
        mask = nx.greater_equal(nx.iota((sq, sk), axis=0), nx.iota((sq, sk), axis=1))
        s = nx.select(nx.broadcast(mask, s.shape), s, float("-inf"))
    m = nx.reduce_max(s, axes=[-1], keep_axes=True)
    e = nx.exp(s - m)
    p = e / nx.sum(e, axes=[-1], keep_axes=True)
    return nx.dot(p, [3], [0, 1], v, [2], [0, 1])


@pytest.mark.parametrize("b,h,sq,sk,causal", [(1, 2, 128, 128, True), (2, 3, 384, 384, True), (1, 2, 200, 200, True),
                                               (1, 2, 130, 260, False), (2, 1, 512, 64, False)])
def test_fused_attention(b, h, sq, sk, causal):
    """head_dim 128 attention is lowered to the fused tensor-core kernel; compare with the oracle
    (which evaluates the graph node by node) and with the unfused plan."""
    rng = np.random.default_rng(30)
    q = rng.normal(0, 1, (b, h, sq, 128)).astype(np.float32)
    k = rng.normal(0, 1, (b, h, sk, 128)).astype(np.float32)
    v = rng.normal(0, 1, (b, h, sk, 128)).astype(np.float32)
    fun = lambda q, k, v: _attention(q, k, v, causal)
    prog = defn.compile(fun, [defn.template(a.shape, "bf16") for a in (q, k, v)]).program
    assert "attention" in prog.describe(), prog.describe()
    (g, r, t), = run_both(fun, [(q, "bf16"), (k, "bf16"), (v, "bf16")])
    assert g.shape == (b, h, sq, 128)
    assert_close(g, r, what="fused attention", **BF16)


def _attention_with(q, k, v, transform):
    s = transform(nx.dot(q, [3], [0, 1], k, [3], [0, 1]))
    m = nx.reduce_max(s, axes=[-1], keep_axes=True)
    e = nx.exp(s - m)
    p = e / nx.sum(e, axes=[-1], keep_axes=True)
    return nx.dot(p, [3], [0, 1], v, [2], [0, 1])


def _causal(s):
    sq, sk = s.shape[2], s.shape[3]
    mask = nx.greater_equal(nx.iota((sq, sk), axis=0), nx.iota((sq, sk), axis=1))
    return nx.select(nx.broadcast(mask, s.shape), s, float("-inf"))


@pytest.mark.parametrize("name", ["causal_no_scale", "causal_scale_and_bias", "causal_negative_scale", "bias_only", "scale_only"])
def test_fused_attention_forms_of_the_score_transform(name):
    """The kernel compiles the score transform in up to three forms (full; without a proven causal mask
    for key blocks below the diagonal; scale folded into the exponent when the unmasked transform is a
    multiplication by a positive constant).  Each case here takes another combination of them; 384 rows
    give key blocks below, on and (skipped) above the diagonal."""
    rng = np.random.default_rng(31)
    b, h, sq = 1, 2, 384
    # unscaled scores keep a standard deviation near 1 (q and k at 0.3): the oracle rounds every node to
    # bf16, the kernel keeps f32 in between, and with scores of 10 and more that alone moves probabilities by 10 %
    sd = 0.3 if name == "causal_no_scale" else 1.0
    q, k = (rng.normal(0, sd, (b, h, sq, 128)).astype(np.float32) for _ in range(2))
    v = rng.normal(0, 1, (b, h, sq, 128)).astype(np.float32)
    bias = rng.normal(0, 1, (h, sq, sq)).astype(np.float32)
    inputs = [(q, "bf16"), (k, "bf16"), (v, "bf16")]
    if name == "causal_no_scale":
        fun = lambda q, k, v: _attention_with(q, k, v, _causal)
    elif name == "causal_scale_and_bias":
        inputs.append((bias, "bf16"))
        fun = lambda q, k, v, bb: _attention_with(q, k, v, lambda s: _causal(s * 0.0884 + nx.broadcast(bb, s.shape, axes=[1, 2, 3])))
    elif name == "causal_negative_scale":
        fun = lambda q, k, v: _attention_with(q, k, v, lambda s: _causal(s * -0.0884))
    elif name == "bias_only":
        inputs.append((bias, "bf16"))
        fun = lambda q, k, v, bb: _attention_with(q, k, v, lambda s: s * 0.0884 + nx.broadcast(bb, s.shape, axes=[1, 2, 3]))
    else:
        fun = lambda q, k, v: _attention_with(q, k, v, lambda s: s * 0.0884)
    prog = defn.compile(fun, [defn.template(a.shape, t) for a, t in inputs]).program
    assert "attention" in prog.describe(), prog.describe()
    (g, r, t), = run_both(fun, inputs)
    # two more bf16 roundings per score than the scale-only form (the sum with the bias, the bias itself):
    # the absolute tolerance is doubled; a missing bias or mask would move every row by tens of percent
    assert_close(g, r, what=f"fused attention ({name})", rtol=BF16["rtol"], atol=2 * BF16["atol"])


def test_dense_bias_gelu_reduced():
    inputs = configs.dense_inputs(m=384, n=512, k=1024)
    (g, r, t), = run_both(configs.dense_bias_gelu, inputs)
    assert_close(g, r, what="dense+bias+gelu", **BF16)


def test_batched_dot_reduced():
    (g, r, t), = run_both(configs.batched_dot, configs.batched_inputs(batch=6, m=256, k=128, n=512))
    assert_close(g, r, what="batched dot", **BF16)


@pytest.mark.parametrize("m", [1, 16, 256])
def test_quantised_linear_reduced(m):
    f_in, i_in = configs.quantised_inputs(m=m, n=1024, k=512)
    (g, r, t), = run_both(configs.quantised_linear, f_in)
    assert t == ("f", 32)
    assert_close(g, r, rtol=1e-5, atol=1e-5 * float(np.abs(r).max()), what=f"quantised linear M={m}")
    (gi, ri, ti), = run_both(configs.integer_linear, i_in)
    assert ti == ("s", 32) and np.array_equal(gi, ri)


@pytest.mark.parametrize("m,n,k", [(5, 1000, 528), (48, 136, 4096), (300, 392, 80), (512, 128, 64), (513, 256, 128),
                                   # up to 16 rows and k a multiple of 64 up to 4096: the register-streaming kernel
                                   (3, 1003, 576), (9, 520, 4096), (16, 136, 1024), (8, 2052, 64), (13, 1000, 4160)])
def test_quantised_linear_ragged(m, n, k):
    """Edges of the in-kernel conversion path: rows that do not fill a batch tile, a second batch
    tile, channels and k that end inside a tile, and (513 rows) the hand-over to the general path; for
    the streaming kernel: channels that end inside a group of 8, k chunks that leave warps idle, 8 and
    9 rows (with and without the upper half of the fragment), and k beyond its reach."""
    f_in, _ = configs.quantised_inputs(m=m, n=n, k=k)
    (g, r, t), = run_both(configs.quantised_linear, f_in)
    assert t == ("f", 32) and g.shape == (m, n)
    assert_close(g, r, rtol=1e-5, atol=1e-5 * float(np.abs(r).max()), what=f"quantised linear {m}x{n}x{k}")


def test_softmax_rows_sum_to_one_at_full_width():
    """Size-independent property at the full row width: softmax rows sum to 1,
    exp(x-max) has a 1 at the argmax, logsumexp = log(sum) + max."""
    x = configs.fused_rows_input(rows=64, cols=32768)
    m, e, s, lse, p, am, chain = [nx.to_numpy(t) for t in defn.jit(configs.fused_rows)(nx.tensor(x))]
    np.testing.assert_allclose(p.sum(axis=1, dtype=np.float64), 1.0, rtol=1e-5)
    assert np.array_equal(am, x.argmax(axis=1))
    assert np.all(e[np.arange(64), am] == 1.0)
    np.testing.assert_allclose(lse, np.log(s.astype(np.float64)) + m, rtol=1e-6)
    assert np.array_equal(m, x.max(axis=1))
