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


def test_loop_step_program_guards_the_state_and_updates_a_cache_window_in_place():
    """A `while` whose body writes one row of a cache per iteration (put_slice at a computed position):
    the step program the host queues several times per look at the condition keeps the state when the
    condition is false, and writes the donated cache in place, a window at a time."""
    import numpy as np
    import nx_oracle as O
    from nx_b200 import nx
    T_, H = 12, 8
    w = np.linspace(-1, 1, H).astype(np.float32)

    def step(toks, pos, cache):
        tok = nx.slice(toks, [pos], [1])
        k = nx.as_type(nx.broadcast(tok, (1, H)), "f32") * nx.tensor(w) + 0.5
        cache = nx.put_slice(cache, [pos, 0], k)
        nxt = nx.as_type(nx.argmax(nx.dot(k, [1], cache, [1]), axis=1), "s32") + 1
        return nx.put_slice(toks, [pos + 1], nxt), pos + 1, cache

    tm = [defn.template((T_,), "s32"), defn.template((), "s32"), defn.template((T_, H), "f32")]
    outs, _, _ = defn._trace(lambda t, p, c: defn.while_loop(lambda t, p, c: nx.less(p, T_ - 1), step, (t, p, c)), tm)
    prog = defn._look_ahead_step(outs[0].data.payload)
    plan = prog.describe()
    assert "argument 2 -> result 2 (written in place)" in plan, plan
    assert "space={1,8}" in plan and "space={12,8}" not in plan, plan        # the cache is never copied
    # semantics, with the oracle as the executor: steps queued past the end of the loop change nothing
    toks, pos, cache = np.array([3] + [0] * (T_ - 1), np.int32), np.array(0, np.int32), np.zeros((T_, H), np.float32)
    rt, rp, rk = toks.copy(), 0, cache.copy()
    while rp < T_ - 1:
        k = rt[rp].astype(np.float32) * w + 0.5
        rk[rp] = k
        rt[rp + 1] = int(np.argmax(rk @ k)) + 1
        rp += 1
    state, looks = [toks, pos, cache], 0
    while True:
        for _ in range(8):
            res = O.run_program(prog.blob, [x.tobytes() for x in state])
            state, pred = [r[0] for r in res[:3]], res[3][0]
        looks += 1
        if not pred:
            break
    assert looks == 2 and np.array_equal(state[0], rt) and int(state[1]) == rp and np.allclose(state[2], rk)


def test_kernels_compile_with_the_runtime_compiler_another_package_loaded_first():
    """A process that imported torch before this library runs its kernels through torch's copy of the
    runtime compiler, one CUDA release older than the toolkit's: the generated tensor-core kernels
    (attention with the scale folded into the exponent among them) must build there too."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import torch, sys\n"
        f"sys.path.insert(0, {root!r})\n"
        "from nx_b200 import configs, defn\n"
        "block = configs.make_decoder_block(n_heads=4)\n"
        "inputs = configs.decoder_inputs(batch=1, seq=256, hidden=512, inter=688)\n"
        "prog = defn.compile(block, [defn.template(a.shape, t) for a, t in inputs]).program\n"
        "assert 'attention' in prog.describe()\n"
        "f_in, _ = configs.quantised_inputs(m=16, n=1024, k=512)\n"
        "defn.compile(configs.quantised_linear, [defn.template(a.shape, t) for a, t in f_in])\n"
        "print('built')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "built" in r.stdout, r.stderr[-2000:]


def test_the_nif_shim_and_the_elixir_stubs_cover_every_entry_point():
    """`c_src/nxb200_nif.c` (not compiled here) must call every function `include/nxb200.h` declares, and
    `lib/nx_b200/nif.ex` must hold a stub of the same arity for every NIF the shim registers."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "nxb200.h")).read()
    shim = open(os.path.join(root, "c_src", "nxb200_nif.c")).read()
    stubs = open(os.path.join(root, "lib", "nx_b200", "nif.ex")).read()
    declared = set(re.findall(r"\b(?:int|size_t)\s+(nxb200_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 40
    missing = sorted(f for f in declared if not re.search(r"\b" + f + r"\s*\(", shim))
    assert not missing, missing
    registered = re.findall(r'\{"([a-z0-9_]+)",\s*(\d+),\s*([a-z0-9_]+),', shim)
    assert len(registered) >= 40
    for name, arity, fun in registered:
        assert re.search(r"static ERL_NIF_TERM " + fun + r"\(", shim), fun
        m = re.search(r"def " + name + r"(\(([^)]*)\))?, do: err\(\)", stubs)
        assert m, f"no Elixir stub for {name}/{arity}"
        got = 0 if not m.group(2) else len([a for a in m.group(2).split(",") if a.strip()])
        assert got == int(arity), (name, arity, got)


def test_the_elixir_walker_emits_only_operations_the_library_knows():
    """`lib/nx_b200/compiler.ex` (not compiled here) writes operation names into the program bytes: literal
    strings given to `emit`, and the atoms of the clauses that go through `simple`.  Each of them must be a
    name the planner accepts (its operation tables and its support check in `csrc/compiler.cpp`); an Expr
    operation the device lacks (`:stack`, `:eye`, `:cond`, `:block`) must be lowered to other operations,
    never emitted under its own name."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    walker = open(os.path.join(root, "lib", "nx_b200", "compiler.ex")).read()
    planner = open(os.path.join(root, "nx_b200", "csrc", "compiler.cpp")).read()

    known = set()
    for table in re.findall(r"const std::set<std::string> k\w+ = \{([^}]*)\}", planner):
        known |= set(re.findall(r'"([a-z0-9_]+)"', table))
    known |= set(re.findall(r'\.op == "([a-z0-9_]+)"', planner))
    assert {"add", "reshape", "dot", "concatenate", "gather", "sort"} <= known

    emitted = set(re.findall(r'emit\([^\n]*?, "([a-z0-9_]+)",', walker))
    table = re.search(r"@elementwise \[(.*?)\]", walker, re.S).group(1)
    emitted |= set(re.findall(r":([a-z0-9_]+)", table))
    # clauses that call simple(...) or emit Atom.to_string(op) write the clause's own operation name(s)
    for clause in re.split(r"\n  defp lower\(", walker)[1:]:
        head, _, body = clause.partition(" do")
        own = body.split("\n  defp ")[0]
        if "simple(" not in own and "simple(" not in head and "Atom.to_string(op)" not in own:
            continue
        one = re.search(r"op: :([a-z0-9_]+)", head)
        if one:
            emitted.add(one.group(1))
        for guard in re.findall(r"when op in \[([^\]]*)\]", head):
            emitted |= set(re.findall(r":([a-z0-9_]+)", guard))
    emitted.discard("elementwise")
    assert len(emitted) > 80, sorted(emitted)
    unknown = sorted(emitted - known)
    assert not unknown, unknown
    for lowered in ("stack", "eye", "cond", "block"):
        assert lowered not in emitted
        assert re.search(r"op: :" + lowered + r"\b", walker), lowered
