"""Batched serving on top of compiled programs: the host-side mirror of ``Nx.Serving`` and
``Nx.Batch`` (nx/lib/nx/serving.ex, nx/lib/nx/batch.ex).

A serving wraps a function over a *batch* (tensors whose leading axis is the batch axis).
`run` executes inline.  `start` spawns a server that stacks the batches of concurrent
callers up to ``batch_size`` entries, pads the last one, executes it on an idle partition
(one partition per GPU when ``partitions=True``, as ``__partitions_options__`` dictates,
serving.ex:1362-1378) and hands every caller the slice that belongs to it - the algorithm
of serving.ex:1418-1475.  Threads stand in for the reference's processes.

Tensors may be `nx_b200.nx.Tensor` values or numpy arrays (containers: tuples, lists and
dicts of them); a batch is assembled on the host and moved to the partition's device by the
compiled function itself.
"""
import threading
import time
from collections import deque

import numpy as np

from . import defn as _defn
from . import nx

_SERVINGS = {}
_SERVINGS_LOCK = threading.Lock()


# ---- containers -----------------------------------------------------------------------------

def _map(fun, c):
    if isinstance(c, (tuple, list)):
        return type(c)(_map(fun, x) for x in c)
    if isinstance(c, dict):
        return {k: _map(fun, v) for k, v in c.items()}
    return fun(c)


def _leaves(c, acc):
    if isinstance(c, (tuple, list)):
        for x in c:
            _leaves(x, acc)
    elif isinstance(c, dict):
        for k in c:
            _leaves(c[k], acc)
    else:
        acc.append(c)
    return acc


def _rebuild(template, it):
    if isinstance(template, (tuple, list)):
        return type(template)(_rebuild(x, it) for x in template)
    if isinstance(template, dict):
        return {k: _rebuild(v, it) for k, v in template.items()}
    return next(it)


def _host(x):
    return nx.to_numpy(x) if isinstance(x, nx.Tensor) else np.asarray(x)


def _slice0(x, start, size):
    """``Nx.slice_along_axis(x, start, size, axis: 0)`` for either kind of tensor."""
    if isinstance(x, nx.Tensor):
        return x if (start == 0 and size == x.shape[0]) else nx.slice_along_axis(x, start, size, axis=0)
    return x[start:start + size]


def _concat0(parts):
    if len(parts) == 1:
        return parts[0]
    if isinstance(parts[0], nx.Tensor):
        return nx.concatenate(list(parts), axis=0)
    return np.concatenate(parts, axis=0)


# ---- Nx.Batch ---------------------------------------------------------------------------------

class Batch:
    """``Nx.Batch``: entries stacked or concatenated along axis 0, plus padding (batch.ex)."""

    def __init__(self, key="default"):
        self.key = key
        self.size = 0
        self.pad_size = 0
        self._chunks = []          # containers of host arrays with a leading batch axis
        self._template = None

    @staticmethod
    def stack(entries, batch=None):
        """batch.ex:306: each entry is one element of the batch."""
        return Batch.concatenate([_map(lambda t: _host(t)[None, ...], e) for e in entries], batch)

    @staticmethod
    def concatenate(entries, batch=None):
        """batch.ex:249: each entry already has the batch axis."""
        b = batch or Batch()
        for e in entries:
            e = _map(_host, e)
            leaves = _leaves(e, [])
            if not leaves or any(l.ndim < 1 for l in leaves):
                raise ValueError("cannot concatenate scalars into a batch")
            n = leaves[0].shape[0]
            if any(l.shape[0] != n for l in leaves):
                raise ValueError("all tensors of a batch entry must have the same leading dimension")
            sig = [(l.dtype, l.shape[1:]) for l in leaves]
            if b._template is None:
                b._template = sig
            elif sig != b._template:
                raise ValueError(f"batch entries must agree in type and trailing shape: {sig} vs {b._template}")
            b._chunks.append(e)
            b.size += n
        return b

    def key_(self, key):
        self.key = key
        return self

    def pad(self, n):
        """batch.ex:180: zero entries appended when the batch is materialised."""
        self.pad_size = n
        return self

    def split(self, n):
        """batch.ex:125: the first `n` entries, and the rest."""
        if n <= 0:
            raise ValueError("split size must be positive")
        if n >= self.size:
            return self, Batch(self.key)
        left, right = Batch(self.key), Batch(self.key)
        left._template = right._template = self._template
        need = n
        for c in self._chunks:
            m = _leaves(c, [])[0].shape[0]
            if need >= m:
                left._chunks.append(c)
                left.size += m
                need -= m
            elif need > 0:
                left._chunks.append(_map(lambda a: a[:need], c))
                right._chunks.append(_map(lambda a, k=need: a[k:], c))
                left.size += need
                right.size += m - need
                need = 0
            else:
                right._chunks.append(c)
                right.size += m
        right.pad_size = self.pad_size
        return left, right

    @staticmethod
    def merge(batches):
        """batch.ex:72."""
        out = Batch(batches[0].key if batches else "default")
        for b in batches:
            if b.key != out.key:
                raise ValueError("cannot merge batches with different keys")
            Batch.concatenate(b._chunks, out)
        return out

    def materialise(self):
        """One container of host arrays with leading dimension size + pad."""
        if not self._chunks:
            raise ValueError("cannot materialise an empty batch")
        cols = [_leaves(c, []) for c in self._chunks]
        out = []
        for j in range(len(cols[0])):
            a = np.concatenate([c[j] for c in cols], axis=0) if len(cols) > 1 else cols[0][j]
            if self.pad_size:
                a = np.concatenate([a, np.zeros((self.pad_size,) + a.shape[1:], a.dtype)], axis=0)
            out.append(a)
        return _rebuild(self._chunks[0], iter(out))


# ---- Nx.Serving -------------------------------------------------------------------------------

class Serving:
    """``Nx.Serving.new/2`` and ``jit/2`` (serving.ex:454-529)."""

    def __init__(self, builder, defn_options=None):
        self.builder = builder                      # defn_options -> (batch container -> output container)
        self.defn_options = dict(defn_options or {})
        self.pre = lambda x: (x, None)
        self.post = lambda out_meta, info: out_meta[0]      # serving.ex default: the output alone
        self.limit = None

    @staticmethod
    def new(builder, **defn_options):
        return Serving(builder, defn_options)

    @staticmethod
    def jit(fun, types=None, **defn_options):
        """The function is compiled on first use per partition, with that partition's options
        (e.g. its device).  `fun` takes the batch's tensors as positional arguments; `types`
        optionally names their Nx types in order (numpy has no bf16)."""
        def builder(opts):
            compiled = _defn.jit(fun, **opts)

            def run(batch):
                leaves = _leaves(batch, [])
                tys = list(types) if types is not None else [None] * len(leaves)
                return compiled(*[nx.tensor(a, t) for a, t in zip(leaves, tys)])
            return run
        return Serving(builder, defn_options)

    def batch_size(self, n):
        if n <= 0:
            raise ValueError("batch size must be positive")
        self.limit = n
        return self

    def client_preprocessing(self, fun):
        """fun(input) -> (Batch, info)   (serving.ex:540)."""
        self.pre = fun
        return self

    def client_postprocessing(self, fun):
        """fun((output, metadata), info) -> result   (serving.ex:556)."""
        self.post = fun
        return self

    def _preprocess(self, x):
        batch, info = self.pre(x)
        if not isinstance(batch, Batch):
            raise ValueError("client_preprocessing must return a Batch")
        return batch, info

    # -- inline execution (serving.ex:674-719) --
    def run(self, x):
        batch, info = self._preprocess(x)
        fn = self.builder(self.defn_options)
        pieces = []
        rest = batch
        while True:
            if self.limit is not None and rest.size > self.limit:
                head, rest = rest.split(self.limit)
            else:
                head, rest = rest, None
            out = fn(head.materialise())
            pieces.append(_map(lambda t, n=head.size: _slice0(t, 0, n), out))
            if rest is None or rest.size == 0:
                break
        return self.post((_join(pieces), None), info)

    # -- process API (serving.ex:846-1020) --
    def start(self, name, batch_size=None, batch_timeout_ms=100, partitions=False, partition_options=None):
        limit = batch_size or self.limit or 1
        if partition_options is None:
            partition_options = _defn.__partitions_options__(self.defn_options) if partitions else [dict(self.defn_options)]
        server = _Server(name, self, limit, batch_timeout_ms / 1000.0, partition_options)
        with _SERVINGS_LOCK:
            if name in _SERVINGS:
                raise ValueError(f"a serving named {name!r} is already running")
            _SERVINGS[name] = server
        server.start()
        return server


def _join(pieces):
    if len(pieces) == 1:
        return pieces[0]
    cols = [_leaves(p, []) for p in pieces]
    return _rebuild(pieces[0], iter([_concat0([c[j] for c in cols]) for j in range(len(cols[0]))]))


def batched_run(name, x):
    """``Nx.Serving.batched_run/2`` (serving.ex:998-1104)."""
    with _SERVINGS_LOCK:
        server = _SERVINGS.get(name)
    if server is None:
        raise ValueError(f"could not find Nx.Serving with name {name!r}. Make sure your serving is running")
    return server.batched_run(x)


def stop(name):
    with _SERVINGS_LOCK:
        server = _SERVINGS.pop(name, None)
    if server is not None:
        server.stop()


class _Ref:
    def __init__(self, size):
        self.size = size
        self.pieces = {}            # start -> output container
        self.received = 0
        self.error = None
        self.done = threading.Event()


class _Server:
    """The serving process: a stack per key that fills up to `limit`, a timer, idle partitions."""

    def __init__(self, name, serving, limit, timeout, partition_options):
        self.name, self.serving, self.limit, self.timeout = name, serving, limit, timeout
        self.cv = threading.Condition()
        self.stack = []             # [(ref, start_in_ref, batch)]
        self.count = 0
        self.deadline = None
        self.ready = deque()        # merged batches waiting for a partition
        self.running = True
        self.executed = []          # (partition, size, padded) per execution, for inspection
        self.workers = [threading.Thread(target=self._partition_loop, args=(i, o), daemon=True) for i, o in enumerate(partition_options)]
        self.timer = threading.Thread(target=self._tick, daemon=True)

    def start(self):
        for w in self.workers:
            w.start()
        self.timer.start()

    def stop(self):
        with self.cv:
            self.running = False
            self.cv.notify_all()
        for w in self.workers:
            w.join(timeout=5)

    # client side
    def batched_run(self, x):
        batch, info = self.serving._preprocess(x)
        if batch.size == 0:
            raise ValueError("cannot run an empty batch")
        ref = _Ref(batch.size)
        with self.cv:
            if not self.running:
                raise RuntimeError(f"serving {self.name!r} is not running")
            self._stack_and_execute(ref, batch)
            self.cv.notify_all()
        ref.done.wait()
        if ref.error is not None:
            raise ref.error
        out = _join([ref.pieces[s] for s in sorted(ref.pieces)])
        return self.serving.post((out, None), info)

    # server side (all under self.cv)
    def _stack_and_execute(self, ref, batch):
        """serving.ex:1418-1443: fill the current stack; split the caller's batch as necessary."""
        start = 0
        while batch.size > 0:
            room = self.limit - self.count
            head, batch = batch.split(room)
            self.stack.append((ref, start, head))
            self.count += head.size
            start += head.size
            if self.count == self.limit:
                self._execute()
            elif self.deadline is None:
                self.deadline = time.monotonic() + self.timeout

    def _execute(self):
        if not self.stack:
            return
        merged = Batch.merge([b for _, _, b in self.stack])
        merged.pad(self.limit - merged.size)
        offsets, at = [], 0
        for ref, start, b in self.stack:
            offsets.append((ref, start, at, b.size))
            at += b.size
        self.ready.append((merged, offsets))
        self.stack, self.count, self.deadline = [], 0, None

    def _tick(self):
        with self.cv:
            while self.running:
                if self.deadline is not None and time.monotonic() >= self.deadline:
                    self._execute()
                    self.cv.notify_all()
                wait = 0.05 if self.deadline is None else max(0.0, min(0.05, self.deadline - time.monotonic()))
                self.cv.wait(timeout=wait)

    def _partition_loop(self, index, options):
        fn = None
        while True:
            with self.cv:
                while self.running and not self.ready:
                    self.cv.wait()
                if not self.running:
                    return
                merged, offsets = self.ready.popleft()
                self.executed.append((index, merged.size, merged.pad_size))
            try:
                if fn is None:
                    fn = self.serving.builder(options)
                out = fn(merged.materialise())
                for ref, start, at, size in offsets:
                    ref.pieces[start] = _map(lambda t, a=at, n=size: _slice0(t, a, n), out)
            except Exception as e:          # every caller of the failed batch sees the error
                for ref, _, _, _ in offsets:
                    ref.error = e
            with self.cv:
                for ref, _, _, size in offsets:
                    ref.received += size
                    if ref.received >= ref.size or ref.error is not None:
                        ref.done.set()
