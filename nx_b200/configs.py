"""The five workload configurations of the hot path, written as `defn` functions
against the Nx API exactly as a user of the reference would write them, plus
seeded synthetic inputs (numpy PCG64; distributions and seeds as listed in the
configuration table).  Tests, the benchmark and the smoke check share these.

Sizes can be scaled down through the keyword arguments; the defaults are the
full-size configurations.
"""
from __future__ import annotations

import math

import numpy as np

from . import nx


# ---- C1: MLP forward -------------------------------------------------------------------
def mlp(x, w1, b1, w2, b2):
    """relu(x.W1+b1).W2+b2 -> softmax along axis 1 -> argmax."""
    h = nx.max(nx.dot(x, w1) + b1, 0.0)
    logits = nx.dot(h, w2) + b2
    m = nx.reduce_max(logits, axes=[1], keep_axes=True)
    e = nx.exp(logits - m)
    p = e / nx.sum(e, axes=[1], keep_axes=True)
    return logits, p, nx.argmax(p, axis=1)


def mlp_inputs(batch=64, seed=0):
    rng = np.random.default_rng(seed)
    return [(rng.uniform(0, 1, (batch, 784)).astype(np.float32), "f32"),
            (rng.normal(0, 0.05, (784, 128)).astype(np.float32), "f32"),
            (rng.normal(0, 0.05, (128,)).astype(np.float32), "f32"),
            (rng.normal(0, 0.05, (128, 10)).astype(np.float32), "f32"),
            (rng.normal(0, 0.05, (10,)).astype(np.float32), "f32")]


# ---- C2: bandwidth-bound fused rows --------------------------------------------------------
def fused_rows(x):
    """Row max, exp(x-max), its sum, logsumexp, softmax, argmax, and the chain
    tanh(x*0.5+0.1)*sigmoid(x); shared sub-expressions are shared nodes."""
    m = nx.reduce_max(x, axes=[1], keep_axes=True)
    e = nx.exp(x - m)
    s = nx.sum(e, axes=[1], keep_axes=True)
    return (nx.squeeze(m, [1]), e, nx.squeeze(s, [1]), nx.logsumexp(x, axes=[1]), e / s,
            nx.argmax(x, axis=1), nx.tanh(x * 0.5 + 0.1) * nx.sigmoid(x))


def fused_rows_input(rows=8192, cols=32768, seed=1):
    rng = np.random.default_rng(seed)
    out = np.empty((rows, cols), dtype=np.float32)
    step = max(1, (1 << 24) // cols)
    for r in range(0, rows, step):
        out[r:r + step] = rng.standard_normal((min(step, rows - r), cols), dtype=np.float32) * 2.0
    return out


# ---- C3: dense dot_general -----------------------------------------------------------------
def gelu_erf(x):
    return 0.5 * x * (1.0 + nx.erf(x * (1.0 / math.sqrt(2.0))))


def dense_bias_gelu(a, b, bias):
    """bf16 {M,K}.{K,N} with f32 accumulation inside the product, bias add and
    erf-gelu; every node's type is bf16, as the graph says."""
    return gelu_erf(nx.dot(a, b) + bias)


def dense_inputs(m=8192, n=8192, k=8192, seed=2):
    rng = np.random.default_rng(seed)
    s = 1.0 / math.sqrt(k)
    return [(rng.standard_normal((m, k), dtype=np.float32) * s, "bf16"),
            (rng.standard_normal((k, n), dtype=np.float32) * s, "bf16"),
            (rng.standard_normal((n,), dtype=np.float32), "bf16")]


def batched_dot(a, b):
    """{B,M,K} x {B,K,N}: contract axis 2 with axis 1, batch axis 0."""
    return nx.dot(a, [2], [0], b, [1], [0])


def batched_inputs(batch=64, m=2048, k=128, n=2048, seed=2):
    rng = np.random.default_rng(seed + 100)
    s = 1.0 / math.sqrt(k)
    return [(rng.standard_normal((batch, m, k), dtype=np.float32) * s, "bf16"),
            (rng.standard_normal((batch, k, n), dtype=np.float32) * s, "bf16")]


# ---- C4: int8 weight-only quantised linear --------------------------------------------------------
def quantised_linear(x, w, scale):
    """y = x . (as_type(W, f32) * scale)^T, W s8 {N,K}, per-output-channel f32 scales."""
    wdq = nx.as_type(w, "f32") * nx.reshape(scale, (scale.shape[0], 1))
    return nx.dot(x, [1], wdq, [1])


def integer_linear(xq, w):
    """The integer-accumulate check: s8 activations and weights widened to s32."""
    return nx.dot(nx.as_type(xq, "s32"), [1], nx.as_type(w, "s32"), [1])


def quantised_inputs(m=256, n=11008, k=4096, seed=3):
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, (n, k)).astype(np.int8)
    scale = rng.uniform(1e-3, 2e-2, (n,)).astype(np.float32)
    x = rng.standard_normal((m, k), dtype=np.float32)
    xq = rng.integers(-127, 128, (m, k)).astype(np.int8)
    return [(x, "bf16"), (w, "s8"), (scale, "f32")], [(xq, "s8"), (w, "s8")]


# ---- C5: Llama-style decoder block ---------------------------------------------------------------
def rms_norm(x, gain, eps=1e-5):
    ms = nx.mean(x * x, axes=[-1], keep_axes=True)
    return x * nx.rsqrt(ms + eps) * gain


def rope_tables(seq, head_dim, base=10000.0, type="bf16"):
    """cos/sin tables {seq, head_dim} computed inside the defn from two iotas."""
    pos = nx.as_type(nx.iota((seq, 1), axis=0), "f32")
    i = nx.as_type(nx.iota((1, head_dim // 2), axis=1), "f32")
    inv_freq = nx.exp(i * (-2.0 * math.log(base) / head_dim))
    ang = pos * inv_freq
    ang = nx.concatenate([ang, ang], axis=1)
    return nx.as_type(nx.cos(ang), type), nx.as_type(nx.sin(ang), type)


def rope(t, cos, sin):
    """t {B,heads,S,D}: rotate-half form."""
    d = t.shape[-1]
    t1 = nx.slice_along_axis(t, 0, d // 2, axis=3)
    t2 = nx.slice_along_axis(t, d // 2, d // 2, axis=3)
    rot = nx.concatenate([nx.negate(t2), t1], axis=3)
    return t * cos + rot * sin


def make_decoder_block(n_heads=32, eps=1e-5, rope_base=10000.0):
    def decoder_block(x, wq, wk, wv, wo, wgate, wup, wdown, g1, g2):
        b, s, h = x.shape
        hd = h // n_heads

        def heads(t):
            return nx.transpose(nx.reshape(t, (b, s, t.shape[-1] // hd, hd)), [0, 2, 1, 3])

        hn = rms_norm(x, g1, eps)
        q, k, v = heads(nx.dot(hn, wq)), heads(nx.dot(hn, wk)), heads(nx.dot(hn, wv))
        cos, sin = rope_tables(s, hd, rope_base, x.type)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        scores = nx.dot(q, [3], [0, 1], k, [3], [0, 1]) * (1.0 / math.sqrt(hd))
        causal = nx.greater_equal(nx.iota((s, s), axis=0), nx.iota((s, s), axis=1))
        scores = nx.select(nx.broadcast(causal, scores.shape), scores, float("-inf"))
        m = nx.reduce_max(scores, axes=[-1], keep_axes=True)
        e = nx.exp(scores - m)
        p = e / nx.sum(e, axes=[-1], keep_axes=True)
        ctx = nx.dot(p, [3], [0, 1], v, [2], [0, 1])
        ctx = nx.reshape(nx.transpose(ctx, [0, 2, 1, 3]), (b, s, ctx.shape[1] * hd))
        x1 = x + nx.dot(ctx, wo)
        h2 = rms_norm(x1, g2, eps)
        gate, up = nx.dot(h2, wgate), nx.dot(h2, wup)
        act = gate * nx.sigmoid(gate) * up
        return x1 + nx.dot(act, wdown)
    return decoder_block


def decoder_inputs(batch=8, seq=2048, hidden=4096, inter=11008, seed=4):
    rng = np.random.default_rng(seed)

    def w(*shape):
        return rng.standard_normal(shape, dtype=np.float32) * 0.02

    x = rng.standard_normal((batch, seq, hidden), dtype=np.float32)
    return [(x, "bf16"), (w(hidden, hidden), "bf16"), (w(hidden, hidden), "bf16"), (w(hidden, hidden), "bf16"),
            (w(hidden, hidden), "bf16"), (w(hidden, inter), "bf16"), (w(hidden, inter), "bf16"),
            (w(inter, hidden), "bf16"), (np.ones(hidden, np.float32) + w(hidden), "bf16"),
            (np.ones(hidden, np.float32) + w(hidden), "bf16")]
