"""`Nx.Defn.Compiler` for the B200 runtime.

The callbacks mirror nx/lib/nx/defn/compiler.ex:29-101 as EXLA.Defn implements
them (exla/lib/exla/defn.ex:15-72, :151-191):

``__jit__(key, vars, fun, args_list, opts)``   trace + build (cached), then run
``__compile__(key, vars, fun, opts)``          returns the runner closure
``__partitions_options__(opts)``               one option set per visible GPU
``__to_backend__(opts)``                       where results live
``__shard_jit__``                              lives in `nx_b200.sharding`

`jit` / `compile` are the ``Nx.Defn.jit/2`` / ``Nx.Defn.compile/3`` entry
points (nx/lib/nx/defn.ex:240-271, :331-354) bound to this compiler.

Caching follows exla/lib/exla/defn.ex:337-397: the key is the function plus
the ``{type, shape}`` of every flattened argument — never the values — and the
traced graph is built into a native program once per key.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
import time

from . import backend as B
from . import expr as E
from . import nif
from . import types as T
from .nx import HostData, Tensor


class Program:
    """A built program: ``%EXLA.Executable{}`` (exla/lib/exla/executable.ex)."""

    def __init__(self, blob):
        self.blob = blob
        l = nif.lib()
        h = C.c_void_p()
        nif.check(l.nxb200_program_build(blob, len(blob), C.byref(h)))
        self.handle = h.value
        n_in, n_out = C.c_int(), C.c_int()
        nif.check(l.nxb200_program_io(self.handle, C.byref(n_in), C.byref(n_out)))
        self.n_params, self.n_outputs = n_in.value, n_out.value
        self.outputs = []
        for i in range(self.n_outputs):
            dt, rank = C.c_int(), C.c_int()
            dims = nif.dims_array([])
            nif.check(l.nxb200_program_output_info(self.handle, i, C.byref(dt), dims, C.byref(rank)))
            self.outputs.append((T.CODE_DTYPES[dt.value], tuple(dims[k] for k in range(rank.value))))

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        lib = getattr(nif, "_LIB", None)          # the module is already torn down at interpreter exit
        if h and lib is not None:
            try:
                lib.nxb200_program_release(h)
            except Exception:
                pass

    def describe(self):
        l = nif.lib()
        n = l.nxb200_program_describe(self.handle, None, 0)
        buf = C.create_string_buffer(n + 1)
        l.nxb200_program_describe(self.handle, buf, n + 1)
        return buf.value.decode()

    def kernel_sources(self):
        """Generated CUDA source of each fused kernel (diagnostics)."""
        l = nif.lib()
        out, i = [], 0
        while True:
            n = l.nxb200_program_kernel_source(self.handle, i, None, 0)
            if n == 0:
                return out
            buf = C.create_string_buffer(n + 1)
            l.nxb200_program_kernel_source(self.handle, i, buf, n + 1)
            out.append(buf.value.decode())
            i += 1

    def build_times(self):
        """Seconds spent planning (parse, fusion, code generation) and compiling the generated sources."""
        a, b = C.c_double(), C.c_double()
        nif.check(nif.lib().nxb200_program_build_times(self.handle, C.byref(a), C.byref(b)))
        return {"plan_time": a.value, "codegen_time": b.value}

    def launch_count(self):
        n = C.c_int()
        nif.check(nif.lib().nxb200_program_launch_count(self.handle, C.byref(n)))
        return n.value

    def _arg_array(self, args):
        if len(args) != self.n_params:
            raise ValueError(f"program expects {self.n_params} arguments, got {len(args)}")
        arr = (C.c_void_p * max(1, len(args)))()
        for i, a in enumerate(args):
            if not isinstance(a.data, B.DeviceBuffer):
                raise TypeError("program arguments must be device tensors")
            arr[i] = a.data.handle
        return arr

    def run(self, args, device=0):
        """exla/lib/exla/executable.ex:130-148 (run -> NIF run_io)."""
        arr = self._arg_array(args)
        outs = (C.c_void_p * max(1, self.n_outputs))()
        nif.check(nif.lib().nxb200_program_run(self.handle, device, arr, len(args), outs, self.n_outputs))
        return [Tensor(B.DeviceBuffer(outs[i], device), t, s) for i, (t, s) in enumerate(self.outputs)]

    def run_into(self, args, outs, device=0):
        arr = self._arg_array(args)
        oarr = (C.c_void_p * max(1, len(outs)))(*[o.data.handle for o in outs])
        nif.check(nif.lib().nxb200_program_run_into(self.handle, device, arr, len(args), oarr, len(outs)))
        return outs


# ---- containers (Nx.Defn.Composite) ------------------------------------------------

def _flatten(c, acc):
    if isinstance(c, Tensor):
        acc.append(c)
        return ("t",)
    if isinstance(c, (tuple, list)):
        return ("seq", type(c), [_flatten(x, acc) for x in c])
    if isinstance(c, dict):
        return ("map", [(k, _flatten(c[k], acc)) for k in sorted(c)])
    from . import nx
    acc.append(nx._as_operand(c))
    return ("t",)


def _unflatten(spec, it):
    if spec[0] == "t":
        return next(it)
    if spec[0] == "seq":
        return spec[1](_unflatten(s, it) for s in spec[2])
    return {k: _unflatten(s, it) for k, s in spec[1]}


# ---- compiler callbacks ----------------------------------------------------------------

_cache = {}
_cache_lock = threading.Lock()

# ---- compile telemetry -----------------------------------------------------------------
# The reference emits ``[:exla, :compilation]`` once per cache miss with ``eval_time`` (tracing the
# function into an expression), ``compile_time`` (lowering + compiling) and ``total_time``
# (exla/lib/exla/defn.ex:515-523).  Handlers attached here get the same three measurements, in
# seconds, under the event name ``("b200", "compilation")``, plus ``plan_time`` / ``codegen_time``
# (how compile_time splits into planning and NVRTC) and the cache key as metadata.
_telemetry_handlers = []


def attach_telemetry(handler):
    """``:telemetry.attach/4`` for the compilation event: ``handler(event, measurements, metadata)``."""
    _telemetry_handlers.append(handler)
    return handler


def detach_telemetry(handler):
    if handler in _telemetry_handlers:
        _telemetry_handlers.remove(handler)


def _emit_compilation(key, eval_time, compile_time, program):
    if not _telemetry_handlers:
        return
    m = {"eval_time": eval_time, "compile_time": compile_time, "total_time": eval_time + compile_time}
    if program is not None:
        m.update(program.build_times())
    for h in list(_telemetry_handlers):
        h(("b200", "compilation"), m, {"key": key})


def trace(fun, templates):
    """Run ``fun`` with parameter nodes in place of its tensor arguments
    (nx/lib/nx/defn/compiler.ex:184-205, :890-917) and return
    ``(flat_outputs, output_spec)``."""
    outs, ospec, _ = _trace(fun, templates)
    return outs, ospec


def _trace(fun, templates):
    """`trace` plus the parameter nodes (the serialiser keeps the unused ones)."""
    flat = []
    spec = [_flatten(t, flat) for t in templates]
    params = [E.parameter(t.type, t.shape, i) for i, t in enumerate(flat)]
    it = iter(params)
    args = [_unflatten(s, it) for s in spec]
    with B.trace_scope():
        result = fun(*args)
        outs = []
        ospec = _flatten(result, outs)
        outs = [B.to_expr(o) for o in outs]
    return outs, ospec, params


def __compile__(key, templates, fun, opts):
    """Build (or fetch) the program for ``key`` + argument templates and return
    a closure that runs it on lists of argument thunks."""
    flat = []
    for t in templates:
        _flatten(t, flat)
    # the donation marks are part of the key: a donating call must not reuse the
    # non-donating executable (exla/lib/exla/defn.ex:337-353)
    args_key = tuple((t.type, t.shape, bool(getattr(t, "donatable", False))) for t in flat)
    hooks = opts.get("hooks") or {}
    ck = (key, args_key, opts.get("device"), tuple(sorted((k, id(v)) for k, v in hooks.items())))
    with _cache_lock:
        entry = _cache.get(ck)
    if entry is None:
        t0 = time.perf_counter()
        outs, ospec, params = _trace(fun, templates)
        t1 = time.perf_counter()
        # outputs that are parameters or constants still need a buffer of
        # their own: results are always fresh tensors (exla/lib/exla/defn.ex:387-393)
        donated = [i for i, t in enumerate(flat) if getattr(t, "donatable", False)]
        entry = (_make_runner(outs, params, alias_pairs(donated, params, outs), hooks), ospec)
        _emit_compilation(key, t1 - t0, time.perf_counter() - t1, getattr(entry[0], "program", None))
        with _cache_lock:
            _cache.setdefault(ck, entry)
    run_graph, ospec = entry
    device = B._device_of(opts.get("device"))

    def runner(args_list):
        results = []
        for thunks in args_list:
            args = [B.backend_transfer(th() if callable(th) else th, device) for th in thunks]
            outs = run_graph(args, device)
            results.append(_unflatten(ospec, iter(outs)))
        return results

    runner.program = run_graph.program
    return runner


def _make_runner(outs, params, aliases=None, hooks=None):
    """A callable ``(device tensors, device) -> result tensors`` for a traced graph.  Without control
    flow or host calls that is one program.  ``io_call`` nodes become extra outputs of the program whose
    values are handed to their callbacks after it ran.  A graph with ``while`` or ``runtime_call`` nodes
    is cut at them: one program computes a loop's initial state and captured values (a host call's
    arguments), the host iterates the condition and body programs reading the one-byte predicate back
    (calls the function), and the results enter the programs after it as extra parameters."""
    hooks = hooks or {}
    order = E.topo_order(outs)[0]
    taps = {}
    for t in order:
        if t.data.op == "io_call":
            taps.setdefault(id(t.data.payload), (t.data.payload, {}))[1][t.data.ints[0]] = t
    if taps:
        repl, calls, extra = {}, [], []
        # in the order the calls were traced (api_test.exs "executes independent io_calls in program
        # order"); a tap inside a tapped value was traced before it, so inner taps come first
        for tap, leaves in sorted(taps.values(), key=lambda entry: entry[0].seq):
            # the value as this graph holds it; a leaf the result does not use is taken as traced
            values = E.substitute([leaves[i].data.args[0] if i in leaves else v for i, v in enumerate(tap.values)], repl)
            for i, node in leaves.items():
                repl[node.data.id] = values[i]
            fun = hooks.get(tap.name, tap.fun) if tap.name is not None else tap.fun
            if fun is None:                           # a named tap nobody listens to costs nothing
                continue
            guards = E.substitute([g for g, _ in tap.guards], repl)
            calls.append((fun, tap, values, guards, [want for _, want in tap.guards]))
        # a tapped value that is a result anyway is read from that result, not computed twice
        new_outs = E.substitute(outs, repl)
        n = len(outs)
        slot = {}
        for i, t in enumerate(new_outs):
            slot.setdefault(t.data.id, i)
        for _, _, values, guards, _ in calls:
            for t in values + guards:
                if t.data.id not in slot:
                    slot[t.data.id] = n + len(extra)
                    extra.append(t)
        inner = _make_runner(new_outs + extra, params, aliases, hooks)

        def run_tapped(vals, device):
            from . import nx
            res = inner(vals, device)
            for fun, tap, values, guards, wants in calls:
                if all(bool(nx.to_number(res[slot[g.data.id]])) == w for g, w in zip(guards, wants)):
                    fun(_unflatten(tap.spec, iter([res[slot[v.data.id]] for v in values])))
            return res[:n]
        run_tapped.program = inner.program
        return run_tapped

    # the loops and host calls of this graph, and their result nodes AS THIS GRAPH HOLDS THEM: a graph
    # that went through a substitution (the body of an enclosing loop, whose captured values became
    # parameters) holds rebuilt nodes with other ids and other arguments than the ones traced
    groups, members = [], {}
    for t in order:
        if t.data.op in ("while", "runtime_call"):
            if id(t.data.payload) not in members:
                members[id(t.data.payload)] = {}
                groups.append(t.data.payload)
            members[id(t.data.payload)][t.data.ints[0]] = t
    if not groups:
        prog = Program(E.serialize(outs, params, aliases))

        def run_one(vals, device):
            return prog.run(vals, device)
        run_one.program = prog
        return run_one

    from . import nx
    all_params = list(params)
    repl, stages = {}, []
    for g in groups:
        held = members[id(g)]
        inputs = next(iter(held.values())).data.args
        stage = _make_runner(E.substitute(inputs, repl), list(all_params), None, hooks)
        if isinstance(g, _WhileGroup):
            cond = _make_runner(g.cond_outs, g.sub_params, None, hooks)
            body = _make_runner(g.body_outs, g.sub_params, None, hooks)
            stages.append((stage, g, cond, body))
        else:
            stages.append((stage, g, None, None))
        for i, r in enumerate(g.results):         # the results: parameters of everything downstream
            p = E.parameter(r.type, r.shape, len(all_params))
            all_params.append(p)
            repl[r.data.id] = p
            if i in held:
                repl[held[i].data.id] = p
    final = _make_runner(E.substitute(outs, repl), list(all_params), None, hooks)

    def run_segments(vals, device):
        vals = list(vals)
        for stage, g, cond, body in stages:
            ins = stage(vals, device)
            if cond is None:
                vals += g.call(ins, device)
                continue
            k = g.n_state
            state, caps = list(ins[:k]), list(ins[k:])
            ahead = _look_ahead_step(g)
            if ahead is None:
                while nx.to_number(cond(state + caps, device)[0]):
                    loop_stats["iterations"] += 1
                    loop_stats["host_syncs"] += 1
                    state = list(body(state + caps, device))
                loop_stats["host_syncs"] += 1
            else:
                # The loop stays on the device for LOOK_AHEAD iterations at a time: every step computes
                # the condition on the state it receives and keeps that state when it is false, so
                # steps queued past the end of the loop change nothing, and only the last step's
                # predicate is read back.  The state buffers are donated from step to step.
                while True:
                    for _ in range(LOOK_AHEAD):
                        out = ahead.run([nx.donatable(t) for t in state] + caps, device)
                        state, pred = list(out[:k]), out[k]
                    loop_stats["iterations"] += LOOK_AHEAD
                    loop_stats["host_syncs"] += 1
                    if not nx.to_number(pred):
                        break
            vals += state
        return final(vals, device)
    run_segments.program = None
    return run_segments


# How many iterations of a `while` are queued before the host looks at the condition again, and what
# the loops of this process have cost so far (read by tests and diagnostics).
_eager_loops = {}
LOOK_AHEAD = max(1, int(os.environ.get("NXB200_WHILE_AHEAD", "8")))
loop_stats = {"iterations": 0, "host_syncs": 0}


def _look_ahead_step(g):
    """The program ``(state ++ captures) -> (next state ++ [condition])`` of a while group in which
    the next state is the body's result where the condition holds and the unchanged state where it
    does not.  The reference lowers a loop into the executable, one dispatch per loop
    (exla/lib/exla/defn.ex:670-723); here the host queues several of these steps per look at the
    condition.  None when the loop has host effects that must follow the real iteration count (taps,
    host calls, nested loops): those keep the iteration-by-iteration path."""
    if hasattr(g, "ahead"):
        return g.ahead
    from . import nx
    g.ahead = None
    k = g.n_state
    if any(t.data.op in ("io_call", "while", "runtime_call") for t in E.topo_order(g.cond_outs + g.body_outs)[0]):
        return None
    with B.trace_scope():
        pred = g.cond_outs[0]
        # A window update of a state element (a KV cache written by put_slice) is guarded at the window:
        # the slice written is the new piece where the condition holds and the old content where it
        # does not.  The guarded tensor also replaces the updated one inside the body (what the body
        # computes from it is discarded anyway when the condition is false), so that one tensor per
        # cache exists and the donated buffer is updated in place, a window at a time.
        position = {t.data.id: n for n, t in enumerate(E.topo_order(g.body_outs)[0])}
        repl, outs = {}, [None] * k
        for i in sorted(range(k), key=lambda i: position.get(g.body_outs[i].data.id, -1)):
            old, new = g.sub_params[i], E.substitute([g.body_outs[i]], repl)[0]
            e = new.data
            if e.id == old.data.id:
                outs[i] = new                                             # passed through unchanged
            elif e.op == "put_slice" and e.args[0].data.id == old.data.id and new.type == old.type:
                piece, starts = e.args[1], list(e.args[2:])
                kept = nx.slice(old, starts, list(piece.shape))
                outs[i] = nx.put_slice(old, starts, nx.select(pred, piece, nx.as_type(kept, piece.type)))
                repl[g.body_outs[i].data.id] = outs[i]
            else:
                outs[i] = nx.select(pred, new, old)
        outs.append(nx.not_equal(pred, 0))
    outs = [B.to_expr(o) for o in outs]
    try:
        pairs = alias_pairs(list(range(k)), g.sub_params, outs)
    except ValueError:
        pairs = None                                                     # a state element nothing reads: no donation
    g.ahead = Program(E.serialize(outs, g.sub_params, pairs))
    return g.ahead


def alias_pairs(donated, params, outs):
    """(parameter, output) pairs for the donated parameters: each takes the first output of its
    type and shape that no earlier donation took (exla/lib/exla/defn.ex:598-645)."""
    reachable = {t.data.id for t in E.topo_order(outs)[0]}
    pairs, used = [], set()
    for i in donated:
        p = params[i]
        if p.data.id not in reachable:
            raise ValueError("argument marked for donation is not used by the computation; only used inputs can be donated")
        j = next((j for j, o in enumerate(outs) if j not in used and o.type == p.type and o.shape == p.shape), None)
        if j is None:
            raise ValueError(f"input marked for donation has no output with matching shape {p.shape} and type "
                             f"{T.short(p.type)}; cannot alias this argument")
        used.add(j)
        pairs.append((i, j))
    return pairs


def __jit__(key, templates, fun, args_list, opts):
    return __compile__(key, templates, fun, opts)(args_list)


def __partitions_options__(opts):
    """One option set per device (exla/lib/exla/defn.ex:15-20)."""
    n = nif.device_count()
    return [dict(opts, device=i) for i in range(max(1, n))]


def __to_backend__(opts):
    """exla/lib/exla/defn.ex:23-32."""
    return ("b200", B._device_of(opts.get("device")))


# ---- Nx.Defn entry points ------------------------------------------------------------------

def _templates(args):
    flat = []
    spec = [_flatten(a, flat) for a in args]
    return flat, spec


def jit(fun, **opts):
    """``Nx.Defn.jit(fun, compiler: B200)``: returns a function that traces and
    builds on first call per argument signature, then runs."""
    def wrapped(*args):
        flat, _ = _templates(args)
        res = __jit__(fun, list(args), fun, [flat], opts)
        return res[0]
    wrapped.__wrapped__ = fun
    return wrapped


def compile(fun, templates, **opts):
    """``Nx.Defn.compile/3``: build ahead of time for the given templates."""
    runner = __compile__(fun, list(templates), fun, opts)

    def compiled(*args):
        flat, _ = _templates(args)
        return runner([flat])[0]
    compiled.program = runner.program
    return compiled


def template(shape, type):
    """``Nx.template/2``."""
    return Tensor(None, T.normalize(type), tuple(shape))


def build_program(fun, templates):
    """Trace ``fun`` and return ``(serialised_graph, output_spec)`` without
    touching the native library (used by tests of the front-end and by the
    oracle, which interprets the same bytes)."""
    outs, ospec, params = _trace(fun, list(templates))
    return E.serialize(outs, params), ospec



# ---- control flow (nx/lib/nx/defn/kernel.ex while/cond; Expr :while / :cond) --------------------
# Host-orchestrated: the condition and the body are compiled programs and the loop runs on the
# host, reading the one-byte predicate back each iteration (what Nx.Defn.Evaluator does with a
# device backend).  A loop at the top level (an autoregressive decode loop over a KV cache) runs
# as is; a loop inside a traced defn cuts the traced graph into the programs around it.

def _traced(values):
    flat = []
    for v in values:
        _flatten(v, flat)
    return any(isinstance(t, Tensor) and isinstance(getattr(t, "data", None), E.Expr) and t.data.op != "constant" for t in flat)


def _signature(state):
    flat = []
    _flatten(state, flat)
    return [(t.type, t.shape) for t in flat]


def while_loop(cond_fun, body_fun, init, max_iterations=None, **opts):
    """``while state = init, cond_fun.(state) do body_fun.(state) end``.

    `init` is a tuple of tensors (containers allowed); both functions take the state's
    elements as positional arguments.  As in the reference (nx/lib/nx/defn/expr.ex while/4)
    the body must return the state's exact types and shapes and the condition a scalar.
    Returns the final state."""
    from . import nx
    state = tuple(init)
    if _traced(state):
        return _traced_while(cond_fun, body_fun, state)
    state = tuple(_map_tensors(nx.tensor, s) for s in state)
    want = _signature(state)
    if max_iterations is None:
        # the same loop as a traced one: its steps are queued several at a time (see _look_ahead_step)
        key = (cond_fun, body_fun, tuple(sorted(opts.items())))
        loop = _eager_loops.get(key)
        if loop is None:
            loop = _eager_loops.setdefault(key, jit(lambda *st: while_loop(cond_fun, body_fun, st), **opts))
        return tuple(loop(*state))
    cond_c, body_c = jit(cond_fun, **opts), jit(body_fun, **opts)
    n = 0
    while True:
        pred = cond_c(*state)
        if not isinstance(pred, Tensor) or pred.shape != ():
            raise ValueError(f"condition must be a scalar tensor, got {getattr(pred, 'shape', type(pred))}")
        if not nx.to_number(pred):
            return state
        if max_iterations is not None and n >= max_iterations:
            raise RuntimeError(f"while_loop did not finish within {max_iterations} iterations")
        new = body_c(*state)
        new = tuple(new) if isinstance(new, (tuple, list)) else (new,)
        got = _signature(new)
        if got != want:
            raise ValueError(f"the do-block in while must return tensors with the same shape, type, and names as the initial arguments: {got} vs {want}")
        state = new
        n += 1


class _WhileGroup:
    """What a traced ``while`` carries to the compiler: its inputs in the enclosing graph (initial
    state, then the enclosing values its functions captured), the condition and body graphs over
    parameters ``state ++ captures``, and its result nodes."""
    __slots__ = ("inputs", "cond_outs", "body_outs", "sub_params", "n_state", "results", "ahead")


def _traced_while(cond_fun, body_fun, state):
    """``while`` inside a traced defn (Expr :while, nx/lib/nx/defn/expr.ex while/4): both functions are
    traced over fresh parameters; enclosing values they use become extra, loop-invariant parameters."""
    from . import nx
    flat = []
    spec = [_flatten(x, flat) for x in state]
    flat = [B.to_expr(nx.tensor(t) if not isinstance(t, Tensor) else t) for t in flat]
    k = len(flat)
    mark = E.watermark()
    sub = [E.parameter(t.type, t.shape, i) for i, t in enumerate(flat)]
    it = iter(sub)
    args = [_unflatten(sp, it) for sp in spec]
    with B.trace_scope():
        c = B.to_expr(cond_fun(*args))
        body = body_fun(*args)
        body = tuple(body) if isinstance(body, (tuple, list)) else (body,)
        bflat = []
        bspec = [_flatten(x, bflat) for x in body]
        bflat = [B.to_expr(nx.tensor(t) if not isinstance(t, Tensor) else t) for t in bflat]
    if c.shape != ():
        raise ValueError(f"condition must be a scalar tensor, got shape {c.shape}")
    if [(t.type, t.shape) for t in bflat] != [(t.type, t.shape) for t in flat] or repr(bspec) != repr(spec):
        raise ValueError("the do-block in while must return tensors with the same shape, type, and names as the initial arguments")
    # values of the enclosing trace used inside: nodes older than the watermark
    own = {p.data.id for p in sub}
    captures, repl = [], {}
    inner_taps = _taps_since(mark, [c] + bflat)
    guard_roots = [g for tap in inner_taps for g, _ in tap.guards]
    for t in E.topo_order([c] + bflat + guard_roots)[0]:
        e = t.data
        if isinstance(e.id, int) and e.id < mark and e.id not in own and e.id not in repl and e.op not in ("constant",):
            # only the outermost captured node of a chain matters; inner ones are cut off by the substitution
            repl[e.id] = None
    # keep only captures that are not reachable solely through other captures
    def frontier(roots):
        found, seen = [], set()
        stack = list(roots)
        while stack:
            t = stack.pop()
            e = t.data
            if e.id in seen:
                continue
            seen.add(e.id)
            if e.id in repl:
                found.append(t)
                continue
            stack.extend(e.args)
        return found
    for t in frontier([c] + bflat + guard_roots):
        if not any(t.data.id == x.data.id for x in captures):
            captures.append(t)
    repl = {t.data.id: E.parameter(t.type, t.shape, k + j) for j, t in enumerate(captures)}
    for tap in inner_taps:
        tap.guards = [(E.substitute([g], repl)[0], want) for g, want in tap.guards]
        tap.values = E.substitute(tap.values, repl)
    g = _WhileGroup()
    g.n_state = k
    g.inputs = flat + captures
    g.sub_params = sub + [repl[t.data.id] for t in captures]
    g.cond_outs = E.substitute([c], repl)
    g.body_outs = E.substitute(bflat, repl)
    g.results = [Tensor(E.Expr("while", g.inputs, ints=[i, k], payload=g), t.type, t.shape) for i, t in enumerate(flat)]
    it = iter(g.results)
    return tuple(_unflatten(sp, it) for sp in spec)


def cond(pred, then_fun, else_fun, *operands):
    """``cond do pred -> then_fun.(operands) ; true -> else_fun.(operands) end`` with a scalar
    predicate.  At the top level the predicate is read back and one branch runs; inside a traced
    defn both branches become part of the graph and ``select`` picks (identical results for
    these side-effect-free functions; the reference's single-branch execution only saves work)."""
    from . import nx
    p = pred if isinstance(pred, Tensor) else nx.tensor(pred)
    if p.shape != ():
        raise ValueError(f"condition must be a scalar tensor, got shape {p.shape}")
    if not _traced((p,) + tuple(operands)):
        return then_fun(*operands) if nx.to_number(p) else else_fun(*operands)
    p = B.to_expr(p)
    mark = E.watermark()
    a = then_fun(*operands)
    fa, fb = [], []
    spec_a = _flatten(a, fa)
    for tap in _taps_since(mark, [B.to_expr(t) for t in fa]):
        tap.guards.append((p, True))                  # a tap fires only in the branch that is taken
    mark = E.watermark()
    b = else_fun(*operands)
    spec_b = _flatten(b, fb)
    for tap in _taps_since(mark, [B.to_expr(t) for t in fb]):
        tap.guards.append((p, False))
    if repr(spec_a) != repr(spec_b):
        raise ValueError("cond expects all branches to return compatible tensor types and shapes")
    out = []
    for x, y in zip(fa, fb):
        # branches are brought to a common type and shape (nx/lib/nx/defn/expr.ex:251-290)
        ty, shape = T.merge(x.type, y.type), nx.binary_broadcast(x.shape, y.shape)
        x, y = (nx.broadcast(nx.as_type(v, ty), shape) for v in (x, y))
        out.append(nx.select(p, x, y))
    return _unflatten(spec_a, iter(out))


def _map_tensors(fun, c):
    if isinstance(c, (tuple, list)):
        return type(c)(_map_tensors(fun, x) for x in c)
    if isinstance(c, dict):
        return {k: _map_tensors(fun, v) for k, v in c.items()}
    return fun(c)


# ---- host callbacks: Nx.runtime_call/4 and Nx.Defn.Kernel.io_call (hook) ------------------------------

def _check_call_result(result, output):
    """nx/lib/nx.ex ensure_call_compatible!: same container structure, types and shapes."""
    got, want = [], []
    gs, ws = _flatten(result, got), _flatten(output, want)
    if repr(gs) != repr(ws) or [(t.type, t.shape) for t in got] != [(t.type, t.shape) for t in want]:
        raise ValueError("expected the runtime_call function to match the given output template "
                         f"{[(T.short(t.type), t.shape) for t in want]}, got: {[(T.short(t.type), t.shape) for t in got]}")
    return got


class _HostCall:
    """What a traced ``runtime_call`` carries to the compiler: its argument nodes, the host function
    and the templates of what it returns."""
    __slots__ = ("inputs", "spec", "fun", "opts", "output", "results")

    def call(self, ins, device):
        from . import nx
        arg = _unflatten(self.spec, iter(ins))
        flat = _check_call_result(self.fun(arg, self.opts), self.output)
        return [B.backend_transfer(t if not isinstance(t.data, E.Expr) else nx.tensor(nx.to_numpy(t), t.type), device) for t in flat]


def runtime_call(output, tensor_or_container, fun, opts=None):
    """``Nx.runtime_call(output, tensor_or_container, opts, fun)`` (nx/lib/nx.ex:2394-2419): run the
    host function ``fun(tensors, opts)`` in the middle of a computation.  ``output`` is a template
    (or container of templates, see `template`) the result must match.  Outside a traced function
    the function is simply called; inside, the graph is cut at the call."""
    flat = []
    spec = _flatten(tensor_or_container, flat)
    if not _traced(flat):
        result = fun(tensor_or_container, opts)
        _check_call_result(result, output)
        return result
    g = _HostCall()
    g.inputs = [B.to_expr(t) for t in flat]
    g.spec, g.fun, g.opts, g.output = spec, fun, opts, output
    want = []
    ospec = _flatten(output, want)
    g.results = [Tensor(E.Expr("runtime_call", g.inputs, ints=[i], payload=g), t.type, t.shape) for i, t in enumerate(want)]
    return _unflatten(ospec, iter(g.results))


class _Tap:
    """What a traced ``io_call`` carries to the compiler: the tapped values (the leaves of the
    container; identity nodes stand for them in the graph), the name and default function, and the
    predicates of the `cond` branches it was traced in (it fires only when they all held)."""
    __slots__ = ("name", "fun", "spec", "values", "guards", "seq")


def io_call(expr, name_or_function, function=None):
    """``Nx.Defn.Kernel.io_call/2,3`` (nx/lib/nx/defn/kernel.ex:1318-1430; `hook` is its older name):
    hand the runtime value of ``expr`` (a tensor or container) to a host function and return ``expr``.
    A name lets ``jit(fun, hooks={name: function})`` supply or override the function; a named call
    without any function is dropped and its value never leaves the device.  As in the reference the
    result of ``io_call`` must be used by the function's result for the call to happen.  The values
    leave the device as extra results of the program they are computed in and the functions run, in
    the order the calls were traced, when that program has finished."""
    name, fun = (None, name_or_function) if callable(name_or_function) else (name_or_function, function)
    flat = []
    spec = _flatten(expr, flat)
    if not _traced(flat):
        if fun is not None:
            fun(expr)
        return expr
    tap = _Tap()
    tap.name, tap.fun, tap.spec, tap.guards, tap.seq = name, fun, spec, [], E.watermark()
    tap.values = [B.to_expr(t) for t in flat]
    return _unflatten(spec, iter([Tensor(E.Expr("io_call", [v], ints=[i], payload=tap), v.type, v.shape) for i, v in enumerate(tap.values)]))


def _taps_since(mark, roots):
    found = []
    for t in E.topo_order(roots)[0]:
        if t.data.op == "io_call" and t.data.id > mark and not any(t.data.payload is f for f in found):
            found.append(t.data.payload)
    return found


hook = io_call


# Nx.Defn.grad / value_and_grad (nx/lib/nx/defn.ex:760-850) live in grad.py; re-exported here because
# that is where a caller of the reference looks for them.
from .grad import grad, value_and_grad  # noqa: E402,F401
