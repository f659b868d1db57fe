"""The five configurations trace, serialise, evaluate on the oracle (reduced
sizes) and compile for sm_100a without a GPU."""
import os

import numpy as np
import pytest

import nx_oracle as O
from helpers import host_tensor
from nx_b200 import configs, defn, nx


def build(fun, inputs):
    host = [host_tensor(a, t) for a, t in inputs]
    blob, _ = defn.build_program(fun, host)
    return blob, host


def test_mlp_traces_and_evaluates():
    blob, host = build(configs.mlp, configs.mlp_inputs())
    res = O.run_program(blob, [h.data.raw for h in host], "binary_backend")
    assert res[0][0].shape == (64, 10) and res[2][0].dtype == np.int32
    np.testing.assert_allclose(res[1][0].sum(axis=1), 1.0, rtol=1e-5)
    prog = defn.Program(blob)
    assert prog.n_outputs == 3


def test_fused_rows_is_a_single_kernel():
    blob, _ = defn.build_program(configs.fused_rows, [defn.template((8192, 32768), "f32")])
    prog = defn.Program(blob)
    assert prog.launch_count() == 1, prog.describe()
    assert "row-in-registers" in prog.describe()


def test_dense_and_quantised_compile():
    for fun, tmpl in [
        (configs.dense_bias_gelu, [defn.template((8192, 8192), "bf16"), defn.template((8192, 8192), "bf16"), defn.template((8192,), "bf16")]),
        (configs.batched_dot, [defn.template((64, 2048, 128), "bf16"), defn.template((64, 128, 2048), "bf16")]),
        (configs.quantised_linear, [defn.template((16, 4096), "bf16"), defn.template((11008, 4096), "s8"), defn.template((11008,), "f32")]),
        (configs.integer_linear, [defn.template((16, 4096), "s8"), defn.template((11008, 4096), "s8")]),
    ]:
        blob, _ = defn.build_program(fun, tmpl)
        prog = defn.Program(blob)
        assert "gemm" in prog.describe()


def test_decoder_block_small_on_oracle_and_compiles():
    block = configs.make_decoder_block(n_heads=4)
    inputs = configs.decoder_inputs(batch=2, seq=16, hidden=64, inter=176)
    blob, host = build(block, inputs)
    (out, typ, _), = O.run_program(blob, [h.data.raw for h in host], "xla_like")
    assert typ == ("bf", 16) and out.shape == (2, 16, 64) and np.isfinite(out).all()
    # causal: the first position only attends to itself, so changing later tokens must not change it
    x2 = inputs[0][0].copy()
    x2[:, 8:, :] += 1.0
    blob2, host2 = build(block, [(x2, "bf16")] + inputs[1:])
    (out2, _, _), = O.run_program(blob2, [h.data.raw for h in host2], "xla_like")
    np.testing.assert_array_equal(out[:, :8], out2[:, :8])
    prog = defn.Program(blob)
    assert prog.n_outputs == 1


def test_decoder_block_full_size_compiles():
    block = configs.make_decoder_block()
    tmpl = [defn.template(a.shape if hasattr(a, "shape") else (), t) for a, t in
            [(np.empty((8, 2048, 4096), np.bool_), "bf16")] + [(np.empty(s, np.bool_), "bf16") for s in
             [(4096, 4096)] * 4 + [(4096, 11008)] * 2 + [(11008, 4096), (4096,), (4096,)]]]
    blob, _ = defn.build_program(block, tmpl)
    prog = defn.Program(blob)
    plan = prog.describe()
    # seven linear layers as tensor-core products, the attention as one fused kernel
    assert plan.count("gemm#") == 7 and plan.count("attention#") == 1, plan


def test_logsumexp_shares_the_softmax_sum():
    """The planner replaces logsumexp's own sum(exp(x - m0)) by the softmax's sum(exp(x - m)) (selected
    against the infinite-maximum cases): the generated kernel evaluates one exponential per element for
    the two of them, and NXB200_NO_SIMPLIFY=1 keeps the graph as written."""
    import subprocess
    import sys
    prog = defn.compile(configs.fused_rows, [defn.template((64, 4096), "f32")]).program
    assert prog.launch_count() == 1
    src = prog.kernel_sources()[0]
    assert src.count("nx_exp(") == 1, src
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (f"import sys; sys.path.insert(0, {root!r})\n"
            "from nx_b200 import configs, defn\n"
            "p = defn.compile(configs.fused_rows, [defn.template((64, 4096), 'f32')]).program\n"
            "print(p.kernel_sources()[0].count('nx_exp('))\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, NXB200_NO_SIMPLIFY="1"))
    assert r.returncode == 0 and r.stdout.strip() == "2", r.stdout + r.stderr[-500:]


def test_rotary_tables_are_computed_once_and_identical_pieces_need_no_buffer():
    """The decoder block's plan: the angle table concatenate([freqs, freqs]) is index arithmetic (no
    concatenate node), cos and sin of it are ONE small kernel writing two tables, and the kernel that
    rotates q and k loads them instead of evaluating cosf / sinf for every element of {batch, head,
    position, dim}.  NXB200_NO_TABLES=1 keeps them inline."""
    block = configs.make_decoder_block(n_heads=4)
    inputs = configs.decoder_inputs(batch=8, seq=512, hidden=512, inter=688)     # rope space 2 M elements
    prog = defn.compile(block, [defn.template(a.shape, t) for a, t in inputs]).program
    plan = prog.describe()
    assert "concatenate" not in plan
    ew = [l for l in plan.split("\n") if "_ew" in l]
    assert len(ew) == 2 and "space={512,128}" in ew[0] and ew[0].count("as_type#") == 2, plan
    rope = [s for s in prog.kernel_sources() if "space" not in s and "nxb_k2_ew" in s]
    assert rope and "cosf" not in rope[0] and "sinf" not in rope[0]
    assert prog.launch_count() == 12, plan


def test_identical_pieces_side_by_side_match_the_oracle():
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    for axis in (0, 1, 2, -1):
        fun = lambda t: nx.concatenate([t * 2.0, t * 2.0][:1] * 3, axis=axis) + 1.0
        blob, _ = defn.build_program(fun, [defn.template(x.shape, "f32")])
        nodes, _ = O.parse_program(blob)
        assert not [n for n in nodes if n.op == "concatenate"]
        (got, _, _), = O.run_program(blob, [x.tobytes()], "xla_like")
        np.testing.assert_array_equal(got, np.concatenate([x * 2.0] * 3, axis=axis) + 1.0)


def test_results_far_larger_than_the_cache_are_stored_with_the_streaming_hint():
    big = defn.compile(configs.fused_rows, [defn.template((8192, 32768), "f32")]).program.describe()
    small = defn.compile(configs.fused_rows, [defn.template((64, 32768), "f32")]).program.describe()
    assert "streaming-stores" in big and "streaming-stores" not in small
