"""Nx.conv lowered to pad / strided slices / dot: checked against a direct convolution written with
numpy loops (the option matrix of exla/test/exla/defn/expr_test.exs:2697-2790), on the CPU through
the oracle; tests/test_gpu_parity.py runs the same function on the GPU."""
import itertools

import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import defn, nx


def conv_direct(x, w, strides, pads, idil, kdil, groups):
    n, c = x.shape[:2]
    co, ci = w.shape[:2]
    nsp = x.ndim - 2
    sh = [n, c] + [(d - 1) * i + 1 for d, i in zip(x.shape[2:], idil)]
    xd = np.zeros(sh)
    xd[(slice(None), slice(None)) + tuple(slice(0, None, i) for i in idil)] = x
    for ax, (lo, hi) in enumerate(pads):
        a = ax + 2
        xd = np.pad(xd, [(0, 0)] * a + [(max(lo, 0), max(hi, 0))] + [(0, 0)] * (xd.ndim - a - 1))
        sl = [slice(None)] * xd.ndim
        sl[a] = slice(max(-lo, 0), xd.shape[a] - max(-hi, 0))
        xd = xd[tuple(sl)]
    ks = w.shape[2:]
    kd = [(k - 1) * d + 1 for k, d in zip(ks, kdil)]
    osp = [(d - k) // s + 1 for d, k, s in zip(xd.shape[2:], kd, strides)]
    out = np.zeros([n, co] + osp)
    cg = co // groups
    axes = list(range(1, nsp + 2))
    for o in itertools.product(*[range(v) for v in osp]):
        for g in range(groups):
            patch = xd[(slice(None), slice(g * ci, (g + 1) * ci)) +
                       tuple(slice(oo * s, oo * s + k, d) for oo, s, k, d in zip(o, strides, kd, kdil))]
            out[(slice(None), slice(g * cg, (g + 1) * cg)) + o] = np.tensordot(patch, w[g * cg:(g + 1) * cg], axes=(axes, axes))
    return out


CASES = [
    ("valid", dict(), dict(strides=[1, 1], pads=[(0, 0), (0, 0)], idil=[1, 1], kdil=[1, 1], groups=1)),
    ("valid stride", dict(strides=[2, 2]), dict(strides=[2, 2], pads=[(0, 0), (0, 0)], idil=[1, 1], kdil=[1, 1], groups=1)),
    ("same stride", dict(strides=[3, 3], padding="same"), dict(strides=[3, 3], pads=[(1, 1), (0, 1)], idil=[1, 1], kdil=[1, 1], groups=1)),
    ("general padding", dict(padding=[(-1, 2), (3, -1)]), dict(strides=[1, 1], pads=[(-1, 2), (3, -1)], idil=[1, 1], kdil=[1, 1], groups=1)),
    ("kernel dilation", dict(padding="same", kernel_dilation=[1, 2]), dict(strides=[1, 1], pads=[(1, 1), (1, 1)], idil=[1, 1], kdil=[1, 2], groups=1)),
    ("input dilation", dict(padding="same", input_dilation=[2, 1]), dict(strides=[1, 1], pads=[(1, 1), (0, 1)], idil=[2, 1], kdil=[1, 1], groups=1)),
    ("both dilations", dict(strides=[2, 1], padding="same", kernel_dilation=[2, 1], input_dilation=[1, 2]),
     dict(strides=[2, 1], pads=[(2, 2), (0, 1)], idil=[1, 2], kdil=[2, 1], groups=1)),
]


def run_oracle(fun, arrays, types):
    host = [host_tensor(a, t) for a, t in zip(arrays, types)]
    blob, _ = defn.build_program(fun, host)
    defn.Program(blob)                       # the kernels compile (no GPU needed)
    return O.run_program(blob, [h.data.raw for h in host], "xla_like")[0][0]


@pytest.mark.parametrize("name,opts,ref", CASES, ids=[c[0] for c in CASES])
def test_conv_options(name, opts, ref):
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (2, 4, 9, 8)).astype(np.float32)
    w = rng.normal(0, 1, (6, 4, 3, 2)).astype(np.float32)
    got = run_oracle(lambda a, b: nx.conv(a, b, **opts), [x, w], ["f32", "f32"])
    np.testing.assert_allclose(got, conv_direct(x, w, **ref), rtol=1e-5, atol=1e-5)


def test_conv_groups_permutations_and_3d():
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, (2, 4, 9, 8)).astype(np.float32)
    w = rng.normal(0, 1, (6, 2, 3, 2)).astype(np.float32)
    got = run_oracle(lambda a, b: nx.conv(a, b, feature_group_size=2), [x, w], ["f32", "f32"])
    np.testing.assert_allclose(got, conv_direct(x, w, [1, 1], [(0, 0), (0, 0)], [1, 1], [1, 1], 2), rtol=1e-5, atol=1e-5)
    w = rng.normal(0, 1, (6, 4, 3, 2)).astype(np.float32)
    want = conv_direct(x, w, [1, 1], [(0, 0), (0, 0)], [1, 1], [1, 1], 1)
    xl = np.ascontiguousarray(x.transpose(0, 2, 3, 1))                    # channels last in, channels last out
    got = run_oracle(lambda a, b: nx.conv(a, b, input_permutation=[0, 3, 1, 2], output_permutation=[0, 3, 1, 2]), [xl, w], ["f32", "f32"])
    np.testing.assert_allclose(got, want.transpose(0, 2, 3, 1), rtol=1e-5, atol=1e-5)
    x3 = rng.normal(0, 1, (1, 2, 5, 6, 4)).astype(np.float32)
    w3 = rng.normal(0, 1, (3, 2, 2, 3, 2)).astype(np.float32)
    got = run_oracle(lambda a, b: nx.conv(a, b, strides=[1, 2, 1], padding="same"), [x3, w3], ["f32", "f32"])
    np.testing.assert_allclose(got, conv_direct(x3, w3, [1, 2, 1], [(0, 1), (1, 1), (0, 1)], [1, 1, 1], [1, 1, 1], 1), rtol=1e-5, atol=1e-5)
    outs, _ = defn.trace(lambda a, b: nx.conv(a, b), [defn.template((1, 1, 3, 3), "s32"), defn.template((4, 1, 1, 1), "s32")])
    assert outs[0].type == ("f", 32) and outs[0].shape == (1, 4, 3, 3)           # integers convolve in f32
    with pytest.raises(ValueError, match="feature groups"):
        defn.trace(lambda a, b: nx.conv(a, b, feature_group_size=2), [defn.template(x.shape, "f32"), defn.template(w.shape, "f32")])


@pytest.mark.parametrize("seed", range(40))
def test_random_conv_configurations(seed):
    """One to three spatial dimensions, strides, signed explicit padding, both dilations and feature groups
    drawn at random, with the operands handed over in a random layout."""
    import random
    r = random.Random(seed)
    nsp = r.choice([1, 2, 2, 3])
    groups = r.choice([1, 1, 2, 3])
    ci, cg, n = r.randint(1, 3), r.randint(1, 2), r.randint(1, 2)
    sp = [r.randint(3, 7) for _ in range(nsp)]
    ks = [r.randint(1, 3) for _ in range(nsp)]
    strides = [r.randint(1, 3) for _ in range(nsp)]
    pads = [(r.randint(-1, 2), r.randint(-1, 2)) for _ in range(nsp)]
    idil = [r.randint(1, 2) for _ in range(nsp)]
    kdil = [r.randint(1, 2) for _ in range(nsp)]
    extent = [(d - 1) * i + 1 + lo + hi for d, i, (lo, hi) in zip(sp, idil, pads)]
    if any(d < (k - 1) * kd + 1 for d, k, kd in zip(extent, ks, kdil)):
        pytest.skip("the window does not fit the padded input")
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 1, [n, ci * groups] + sp).astype(np.float32)
    w = rng.normal(0, 1, [cg * groups, ci] + ks).astype(np.float32)
    want = conv_direct(x.astype(np.float64), w.astype(np.float64), strides, pads, idil, kdil, groups)
    # the caller's layouts: `permutation[i]` names the caller's axis that holds canonical axis i
    perm_x, perm_w, perm_o = (r.sample(range(nsp + 2), nsp + 2) for _ in range(3))
    x_given = np.ascontiguousarray(x.transpose(np.argsort(perm_x)))
    w_given = np.ascontiguousarray(w.transpose(np.argsort(perm_w)))
    got = run_oracle(lambda a, b: nx.conv(a, b, strides=strides, padding=pads, input_dilation=idil, kernel_dilation=kdil,
                                          feature_group_size=groups, input_permutation=perm_x, kernel_permutation=perm_w,
                                          output_permutation=perm_o), [x_given, w_given], ["f32", "f32"])
    np.testing.assert_allclose(got, want.transpose(np.argsort(perm_o)), rtol=1e-4, atol=1e-4)
