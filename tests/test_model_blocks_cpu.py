"""Common model blocks at the sizes real models use (hidden sizes that are not powers of two, vocabulary
sizes that are not multiples of the vector width, ragged sequence lengths, several head sizes) must plan and
compile without a GPU, and the plans must have the shape the design promises: one row kernel for a
normalisation or a softmax, one fused kernel for bf16 attention with 128-wide heads, three kernels for the
attention forms the fused kernel does not take."""
import math

import pytest

from nx_b200 import defn, nx


def tm(shape, type="bf16"):
    return defn.template(tuple(shape), type)


def plan(fun, templates):
    blob, _ = defn.build_program(fun, templates)
    program = defn.Program(blob)
    return program.launch_count(), program.describe()


def layernorm(x, gain, bias):
    xf = nx.as_type(x, "f32")
    mu = nx.mean(xf, axes=[-1], keep_axes=True)
    var = nx.mean((xf - mu) * (xf - mu), axes=[-1], keep_axes=True)
    return nx.as_type((xf - mu) * nx.rsqrt(var + 1e-5), x.type) * gain + bias


@pytest.mark.parametrize("type", ["bf16", "f32"])
@pytest.mark.parametrize("hidden", [768, 1000, 1024, 4096, 5120, 8192, 12288])
def test_layernorm_is_one_row_kernel(hidden, type):
    launches, text = plan(layernorm, [tm((4, 128, hidden), type), tm((hidden,), type), tm((hidden,), type)])
    assert launches == 1 and "_row" in text, text


def softmax(x):
    e = nx.exp(x - nx.reduce_max(x, axes=[-1], keep_axes=True))
    return e / nx.sum(e, axes=[-1], keep_axes=True)


@pytest.mark.parametrize("vocab", [1000, 32000, 50257, 128256, 151936])
def test_softmax_and_cross_entropy_over_a_vocabulary(vocab):
    launches, text = plan(softmax, [tm((8, vocab), "f32")])
    assert launches == 1 and "_row" in text, text

    def cross_entropy(logits, labels):
        picked = nx.squeeze(nx.take_along_axis(logits, nx.reshape(labels, (labels.shape[0], 1)), axis=1), [1])
        return nx.mean(nx.logsumexp(logits, axes=[-1]) - picked)
    # today: the row kernel, two copies of the looked-up positions, the mean's row kernel and its division
    launches, _ = plan(cross_entropy, [tm((8, vocab), "f32"), tm((8,), "s32")])
    assert launches <= 5


def attention(q, k, v, causal, upcast=False):
    scores = nx.dot(q, [3], [0, 1], k, [3], [0, 1]) * (1.0 / math.sqrt(q.shape[-1]))
    if causal:
        sq, sk = scores.shape[2], scores.shape[3]
        keep = nx.greater_equal(nx.iota((sq, sk), axis=0), nx.iota((sq, sk), axis=1))
        scores = nx.select(nx.broadcast(keep, scores.shape), scores, float("-inf"))
    if upcast:
        scores = nx.as_type(scores, "f32")
    p = softmax(scores)
    if upcast:
        p = nx.as_type(p, q.type)
    return nx.dot(p, [3], [0, 1], v, [2], [0, 1])


@pytest.mark.parametrize("sq,sk,causal", [(77, 77, False), (77, 77, True), (128, 128, True), (1000, 1000, False),
                                          (1000, 1000, True), (2048, 2048, True), (64, 300, False), (1, 2048, False)])
def test_bf16_attention_with_128_wide_heads_is_one_kernel_at_any_length(sq, sk, causal):
    launches, text = plan(lambda q, k, v: attention(q, k, v, causal), [tm((2, 8, sq, 128)), tm((2, 8, sk, 128)), tm((2, 8, sk, 128))])
    assert launches == 1 and "attention#" in text, text
    assert ("causal" in text) == causal, text


@pytest.mark.parametrize("type,head", [("bf16", 64), ("bf16", 80), ("bf16", 256), ("f16", 128), ("f32", 128)])
def test_other_attention_forms_take_the_three_kernel_path(type, head):
    launches, text = plan(lambda q, k, v: attention(q, k, v, True), [tm((2, 8, 197, head), type)] * 3)
    assert launches == 3 and "attention#" not in text, text


def test_softmax_upcast_to_f32_by_hand_is_not_yet_recognised_as_attention():
    """Scores converted to f32 before the softmax and the probabilities converted back (a common way to
    write it) stay product + row kernel + product; the fused kernel computes the softmax in f32 anyway."""
    launches, text = plan(lambda q, k, v: attention(q, k, v, True, upcast=True), [tm((2, 8, 2048, 128))] * 3)
    assert launches == 3 and "attention#" not in text, text


def gelu_tanh(x):
    return 0.5 * x * (1.0 + nx.tanh(0.7978845608 * (x + 0.044715 * x * x * x)))


@pytest.mark.parametrize("rows,hidden,inner", [(512, 768, 3072), (1000, 1024, 4096), (77, 768, 3072), (333, 1000, 2000)])
def test_mlp_with_bias_gelu_and_residual_is_two_products_with_fused_epilogues(rows, hidden, inner):
    launches, text = plan(lambda x, w1, b1, w2, b2: nx.dot(gelu_tanh(nx.dot(x, w1) + b1), w2) + b2 + x,
                          [tm((rows, hidden)), tm((hidden, inner)), tm((inner,)), tm((inner, hidden)), tm((hidden,))])
    assert launches == 2, text


def test_lookups_convolutions_pooling_and_sorting_compile():
    assert plan(lambda ids, tok, pos: nx.take(tok, ids, axis=0) + pos, [tm((4, 128), "s32"), tm((32000, 768)), tm((128, 768))])[0] == 1
    assert plan(lambda x, w: nx.conv(x, w, strides=[16, 16]), [tm((2, 3, 224, 224), "f32"), tm((768, 3, 16, 16), "f32")])[0] >= 1
    assert plan(lambda x, w: nx.conv(x, w, padding="same"), [tm((2, 64, 56, 56)), tm((64, 64, 3, 3))])[0] >= 1
    assert plan(lambda x: nx.window_max(x, (1, 1, 3, 3), strides=[1, 1, 2, 2], padding="same"), [tm((2, 64, 112, 112), "f32")])[0] == 1
    assert plan(lambda l: nx.argsort(l, axis=1, direction="desc"), [tm((4, 16000), "f32")])[0] >= 1
    with pytest.raises(Exception, match="at most 16384"):
        plan(lambda l: nx.sort(l, axis=1), [tm((4, 32000), "f32")])


@pytest.mark.parametrize("n,k,type", [(32000, 50, "f32"), (151936, 64, "f32"), (20000, 7, "s32"),
                                      (16385, 1, "f32"), (40000, 100, "bf16")])
def test_top_k_over_a_vocabulary_longer_than_one_sorted_row(n, k, type):
    """Sampling takes the k best of 32,000 to 150,000 logits: more than the sort kernel holds in one row.
    The front-end sorts chunks and then the chunks' candidates; values, positions and the order among equal
    values (lowest position first, NaN highest) must be those of one stable descending sort."""
    import numpy as np
    import nx_oracle as O
    from helpers import host_tensor
    rng = np.random.default_rng(n)
    x = rng.integers(-1000, 1000, (3, n)) if type == "s32" else rng.standard_normal((3, n)).astype(np.float32)
    if type != "s32":
        x[0, 100:200] = x[0, 100]
        x[1, 5], x[1, n - 1] = np.nan, np.inf
        x[2, :] = np.round(x[2] * 4) / 4
    h = host_tensor(x, type)
    blob, _ = defn.build_program(lambda t: nx.top_k(t, k=k), [h])
    assert defn.Program(blob).launch_count() >= 1
    (values, _, _), (positions, position_type, _) = O.run_program(blob, [h.data.raw], "xla_like")
    stored = np.asarray(O.run_program(defn.build_program(lambda t: t + 0, [h])[0], [h.data.raw], "xla_like")[0][0], np.float64)
    want = np.stack([sorted(range(n), key=lambda j: (not np.isnan(row[j]), -row[j] if not np.isnan(row[j]) else 0.0, j))[:k]
                     for row in stored])
    assert position_type == ("s", 32)
    np.testing.assert_array_equal(np.asarray(positions), want)
    np.testing.assert_array_equal(np.asarray(values, np.float64), np.take_along_axis(stored, want, axis=1))
    with pytest.raises(ValueError, match="supports k up to"):
        nx.top_k(h, k=9000)
