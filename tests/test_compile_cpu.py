"""Host-only checks of the native library: it loads, exports every symbol the
header declares, and the planner + code generator produce kernels that compile
for sm_100a (NVRTC needs no GPU) for every golden graph."""
import ctypes
import os
import re

import pytest

from golden.reference_vectors import CASES
from helpers import host_tensor
from nx_b200 import defn, nif

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "nxb200.h")).read()
    names = set(re.findall(r"\b(nxb200_[a-z_0-9]+)\s*\(", header))
    assert len(names) > 25
    lib = ctypes.CDLL(nif.lib_path())
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_init_without_gpu_reports_zero_or_more_devices():
    assert nif.device_count() >= 0


@pytest.mark.parametrize("c", CASES, ids=[c["name"] for c in CASES])
def test_golden_graphs_compile(c):
    args = [host_tensor(v, t) for v, t in c["args"]]
    blob, _ = defn.build_program(c["fun"], args)
    prog = defn.Program(blob)
    assert prog.n_outputs == len(c["expect"])
    assert prog.launch_count() >= 1


def test_bad_program_bytes_are_rejected():
    with pytest.raises(ValueError):
        defn.Program(b"nope")
    with pytest.raises(ValueError):
        defn.Program(b"NXB1" + b"\x01\x00\x00\x00")


def test_unsupported_op_is_reported():
    import struct
    name = b"while"
    blob = b"NXB1" + struct.pack("<I", 1) + struct.pack("<B", len(name)) + name + struct.pack("<BB", 10, 0) \
        + struct.pack("<H", 0) + struct.pack("<H", 0) + struct.pack("<H", 0) + struct.pack("<Q", 0) \
        + struct.pack("<I", 1) + struct.pack("<I", 0)
    with pytest.raises(nif.Unsupported):
        defn.Program(blob)


def test_donation_pairs_and_plans():
    """Nx.donatable bookkeeping without a GPU: pairing rules (exla/lib/exla/defn.ex:598-645) and what
    the planner decides for each pair."""
    from nx_b200 import expr as E, nx
    t = [defn.template((4, 64, 16), "f32"), defn.template((4, 1, 16), "f32"), defn.template((), "s32")]
    outs, _, params = defn._trace(lambda c, n, p: nx.put_slice(c, [0, p, 0], n), t)
    d = defn.Program(E.serialize(outs, params, defn.alias_pairs([0], params, outs))).describe()
    assert "space={4,1,16}" in d and "argument 0 -> result 0 (written in place)" in d      # only the window is written
    outs, _, params = defn._trace(lambda a: nx.transpose(a) + a, [defn.template((32, 32), "f32")])
    d = defn.Program(E.serialize(outs, params, defn.alias_pairs([0], params, outs))).describe()
    assert "own buffer" in d                                                                # a transposed read forbids in-place
    outs, _, params = defn._trace(lambda a, b: (a + b, a - b), [defn.template((3,), "s32")] * 2)
    assert defn.alias_pairs([0, 1], params, outs) == [(0, 0), (1, 1)]
    outs, _, params = defn._trace(lambda a: nx.sum(a), [defn.template((4,), "s32")])
    with pytest.raises(ValueError, match="no output with matching shape"):
        defn.alias_pairs([0], params, outs)
    outs, _, params = defn._trace(lambda a, b: b + 1, [defn.template((2,), "s32")] * 2)
    with pytest.raises(ValueError, match="not used by the computation"):
        defn.alias_pairs([0], params, outs)


def test_static_scratch_product_checks_arguments_before_touching_a_device():
    """Every argument check of the allocation-free product runs on the host before
    the first CUDA call, so a refused call cannot have written the shared scratch
    or enqueued anything (the addresses below are never dereferenced)."""
    lib = nif.lib()
    ok = ctypes.c_void_p(0x7F0000001000)
    odd = ctypes.c_void_p(0x7F0000001002)
    call = lib.nxb200_dot_bf16_static_scratch
    for a, b, c in [(odd, ok, ok), (ok, odd, ok), (ok, ok, odd)]:
        assert call(0, a, b, c, 128, 128, 128, None) == nif.ERR_INVALID
        assert "16-byte aligned" in nif.last_error()
    assert call(0, ok, ok, ok, 8, 8192, 4096, None) == nif.ERR_INVALID      # k*n beyond the built-in scratch
    assert "scratch" in nif.last_error()
    assert call(0, ok, ok, ok, 8, 8, 12, None) == nif.ERR_INVALID           # rows not on 16-byte boundaries
    assert call(0, ok, ok, None, 8, 8, 8, None) == nif.ERR_INVALID


def test_compilation_telemetry_fires_once_per_cache_miss():
    """[:exla, :compilation] of the reference (exla/lib/exla/defn.ex:515-523): eval_time, compile_time
    and total_time on a cache miss, nothing on a hit."""
    from nx_b200 import nx
    events = []
    handler = defn.attach_telemetry(lambda event, measurements, metadata: events.append((event, measurements, metadata)))
    try:
        fun = lambda x: nx.exp(x) + 1.0
        first = defn.compile(fun, [defn.template((4, 4), "f32")])
        assert len(events) == 1
        event, m, meta = events[0]
        assert event == ("b200", "compilation") and "key" in meta
        assert m["eval_time"] > 0 and m["compile_time"] > 0
        assert abs(m["total_time"] - (m["eval_time"] + m["compile_time"])) < 1e-9
        assert 0 < m["codegen_time"] <= m["compile_time"] and m["plan_time"] > 0
        defn.compile(fun, [defn.template((4, 4), "f32")])              # same function, same signature: a cache hit
        assert len(events) == 1
        defn.compile(fun, [defn.template((8, 4), "f32")])              # another signature: compiled again
        assert len(events) == 2
        assert first.program.build_times()["codegen_time"] == m["codegen_time"]
    finally:
        defn.detach_telemetry(handler)
