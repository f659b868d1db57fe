"""Sharded execution: ``Nx.Mesh`` + ``input_shardings`` -> one program per GPU.

Mirrors the caller-facing contract of ``EXLA.shard_jit/3``
(exla/lib/exla.ex:357-387) and ``EXLA.Defn.__shard_jit__/6``
(exla/lib/exla/defn.ex:40-72, validation :74-148): the user writes the GLOBAL
program, describes how every argument is split over a device mesh
(``%{tensor_dim => [mesh_axis]}``), passes the slices each partition owns and
gets each partition's slice of the result back.  Partition i runs on device i,
partitions are numbered row-major over the mesh (exla_client.cc:163-173).

Where the reference hands the global program to XLA's SPMD partitioner, this
module partitions it itself, and only for the two patterns the hot path needs:

* batch data-parallel: an axis of the inputs is split and every op is
  independent along it -> no communication;
* column -> row tensor-parallel linears: a ``dot`` whose contracted axis is split
  on both operands produces partial sums -> one ``all_reduce`` (NCCL over NVLink)
  right after it.

Anything that would need another collective (all-gather, halo exchange …)
raises.  Execution model: one process per GPU; a process holds one partition,
so `shard_jit(...)` returns a function from THIS partition's arguments to this
partition's results (the reference's list-of-partitions view is the
concatenation of those over ranks).
"""
from __future__ import annotations

import math

from . import expr as E
from . import types as T


class Mesh:
    """``%Nx.Mesh{name, shape}`` (nx/lib/nx/mesh.ex:14)."""

    def __init__(self, name, shape):
        self.name, self.shape = name, tuple(int(d) for d in shape)

    @property
    def size(self):
        return math.prod(self.shape)

    def coords(self, partition):
        """Row-major position of a partition in the mesh."""
        out = []
        for d in reversed(self.shape):
            out.append(partition % d)
            partition //= d
        return tuple(reversed(out))


class ShardingError(ValueError):
    pass


def validate_shardings(mesh, shapes, input_shardings):
    """exla/lib/exla/defn.ex:74-148: one sharding per argument, dims and mesh
    axes in range, a mesh axis used at most once per tensor, sizes divisible."""
    if len(input_shardings) != len(shapes):
        raise ShardingError(f"expected {len(shapes)} input shardings, got {len(input_shardings)}")
    specs = []
    for shape, sh in zip(shapes, input_shardings):
        spec = [None] * len(shape)
        used = set()
        for dim, axes in (sh or {}).items():
            if not 0 <= dim < len(shape):
                raise ShardingError(f"sharding refers to dimension {dim} of a rank-{len(shape)} tensor")
            axes = list(axes)
            if len(axes) != 1:
                raise ShardingError("a tensor dimension can be split over exactly one mesh axis")
            a = axes[0]
            if not 0 <= a < len(mesh.shape):
                raise ShardingError(f"mesh axis {a} out of range for mesh {mesh.shape}")
            if a in used:
                raise ShardingError(f"mesh axis {a} is used for two dimensions of the same tensor")
            used.add(a)
            if mesh.shape[a] > 1:
                spec[dim] = a
        specs.append(tuple(spec))
    return specs


def global_shape(local_shape, spec, mesh):
    """Shard shape -> global shape (exla/lib/exla/defn.ex:2451-2468)."""
    return tuple(d * (mesh.shape[a] if a is not None else 1) for d, a in zip(local_shape, spec))


# ---- the partitioner ---------------------------------------------------------------------

class _Part:
    """Rewrites a traced global graph into the program of one partition."""

    def __init__(self, mesh, coords):
        self.mesh, self.coords = mesh, coords
        self.memo = {}          # global node id -> (local tensor, spec)

    def local(self, shape, spec):
        return tuple(d // self.mesh.shape[a] if a is not None else d for d, a in zip(shape, spec))

    def node(self, type, shape, op, args, ints=(), flts=()):
        from .nx import Tensor
        return Tensor(E.Expr(op, args, ints, flts), type, tuple(shape))

    def _split_extent(self, extent, axis):
        n = self.mesh.shape[axis]
        if extent % n:
            raise ShardingError(f"dimension of size {extent} is not divisible by mesh axis of size {n}")
        return extent // n

    def reshard_replicated(self, t, gshape, spec_have, spec_want):
        """A value replicated along a dim the consumer has split: take this
        partition's slice (pure index arithmetic, fused into the consumer)."""
        if spec_have == spec_want:
            return t
        e = t.data
        if getattr(e, "op", None) == "broadcast":
            # a dimension the broadcast created holds the same values at every index: broadcast to the
            # local extent instead of slicing the full one (and a mask stays recognisable as a broadcast)
            src, axes = e.args[0], list(e.ints[1:])
            made = lambda d: d not in axes or src.shape[axes.index(d)] == 1
            if all(h == w or (h is None and made(d)) for d, (h, w) in enumerate(zip(spec_have, spec_want))):
                shape = [n if h == w else self._split_extent(gshape[d], w) for d, (n, h, w) in enumerate(zip(t.shape, spec_have, spec_want))]
                return self.node(t.type, shape, "broadcast", [src], e.ints)
        starts, lengths = [], []
        for d, (h, w) in enumerate(zip(spec_have, spec_want)):
            if h == w:
                starts.append(0)
                lengths.append(t.shape[d])
            elif h is None and w is not None:
                n = self.mesh.shape[w]
                if gshape[d] % n:
                    raise ShardingError(f"dimension of size {gshape[d]} is not divisible by mesh axis of size {n}")
                starts.append(self.coords[w] * (gshape[d] // n))
                lengths.append(gshape[d] // n)
            else:
                raise ShardingError("operands are split differently along the same dimension (needs an all-gather)")
        return self.node(t.type, lengths, "slice", [t], starts + lengths + [1] * len(lengths))

    def visit(self, gt, param_specs):
        e = gt.data
        if e.id in self.memo:
            return self.memo[e.id]
        res = self._visit(gt, e, param_specs)
        used = [a for a in res[1] if a is not None]
        if len(set(used)) != len(used):
            # e.g. x + transpose(x) with x split along its rows: every partition would hold a diagonal
            # block only, and the other blocks need rows that live on another partition
            raise ShardingError(f"{e.op}: the same mesh axis would split two dimensions of the result (needs an all-gather)")
        self.memo[e.id] = res
        return res

    def _visit(self, gt, e, param_specs):
        op, gshape, rank = e.op, gt.shape, len(gt.shape)
        args = [self.visit(a, param_specs) for a in e.args]
        gargs = e.args
        rep = (None,) * rank

        if op == "parameter":
            spec = param_specs[e.ints[0]]
            return E.parameter(gt.type, self.local(gshape, spec), e.ints[0]), spec
        if op in ("constant", "tensor"):
            return gt, rep
        if op == "iota":
            return gt, rep            # replicated; a consumer that is split takes its slice of it
        if op == "metadata":
            return args[0]

        if op in E.UNARY_MATH or op in E.UNARY_OTHER or op == "as_type":
            t, spec = args[0]
            return self.node(gt.type, t.shape, op, [t]), spec

        if op in E.BINARY_ARITH or op in E.BINARY_PRED or op in ("select", "clip"):
            # right-aligned broadcasting: decide the split of every output dim
            spec = [None] * rank
            for (t, s), ga in zip(args, gargs):
                off = rank - len(ga.shape)
                for d, a in enumerate(s):
                    if a is None or ga.shape[d] == 1:
                        continue
                    if spec[off + d] is not None and spec[off + d] != a:
                        raise ShardingError(f"{op}: operands are split over different mesh axes")
                    spec[off + d] = a
            spec = tuple(spec)
            new_args = []
            for (t, s), ga in zip(args, gargs):
                off = rank - len(ga.shape)
                want = tuple(spec[off + d] if ga.shape[d] != 1 else None for d in range(len(ga.shape)))
                new_args.append(self.reshard_replicated(t, ga.shape, s, want))
            return self.node(gt.type, self.local(gshape, spec), op, new_args), spec

        if op in ("sum", "product", "reduce_max", "reduce_min", "all", "any"):
            t, s = args[0]
            keep, n = e.ints[0], e.ints[1]
            axes = list(e.ints[2:2 + n])
            split = [s[a] for a in axes if s[a] is not None]
            if split and op != "sum":
                raise ShardingError(f"{op} over a split dimension is not supported")
            spec = tuple((None if d in axes else s[d]) for d in range(len(s)) if keep or d not in axes)
            out = self.node(gt.type, self.local(gshape, spec), op, [t], e.ints)
            for a in split:
                out = self.node(gt.type, out.shape, "all_reduce", [out], [a])
            return out, spec
        if op in ("argmax", "argmin"):
            t, s = args[0]
            ax, keep = e.ints[1], e.ints[2]
            if ax < 0 and any(a is not None for a in s) or (ax >= 0 and s[ax] is not None):
                raise ShardingError(f"{op} over a split dimension is not supported")
            spec = rep if ax < 0 else tuple((None if d == ax else s[d]) for d in range(len(s)) if keep or d != ax)
            return self.node(gt.type, self.local(gshape, spec), op, [t], e.ints), spec

        if op == "dot":
            (a, sa), (b, sb) = args
            it = iter(e.ints)
            lists = []
            for _ in range(4):
                k = next(it)
                lists.append([next(it) for _ in range(k)])
            c1, b1, c2, b2 = lists
            partial = []
            for x, y in zip(c1, c2):
                if sa[x] != sb[y]:
                    raise ShardingError("dot: the contracted dimension is split on one operand only (needs an all-gather)")
                if sa[x] is not None:
                    partial.append(sa[x])
            for x, y in zip(b1, b2):
                if sa[x] != sb[y]:
                    raise ShardingError("dot: batch dimensions are split differently")
            f1 = [d for d in range(len(sa)) if d not in c1 and d not in b1]
            f2 = [d for d in range(len(sb)) if d not in c2 and d not in b2]
            spec = tuple([sa[d] for d in b1] + [sa[d] for d in f1] + [sb[d] for d in f2])
            used = [s for s in spec if s is not None]
            if len(set(used)) != len(used):
                raise ShardingError("dot: the same mesh axis would split two output dimensions")
            out = self.node(gt.type, self.local(gshape, spec), "dot", [a, b], e.ints)
            for ax in partial:
                out = self.node(gt.type, out.shape, "all_reduce", [out], [ax])
            return out, spec

        if op == "transpose":
            t, s = args[0]
            spec = tuple(s[p] for p in e.ints)
            return self.node(gt.type, self.local(gshape, spec), op, [t], e.ints), spec
        if op == "squeeze":
            t, s = args[0]
            axes = set(e.ints[1:])
            if any(s[a] is not None for a in axes):
                raise ShardingError("squeeze of a split dimension")
            spec = tuple(s[d] for d in range(len(s)) if d not in axes)
            return self.node(gt.type, self.local(gshape, spec), op, [t], e.ints), spec
        if op == "broadcast":
            t, s = args[0]
            spec = [None] * rank
            for d, ax in enumerate(e.ints[1:]):
                if gargs[0].shape[d] != 1:
                    spec[ax] = s[d]
            spec = tuple(spec)
            return self.node(gt.type, self.local(gshape, spec), op, [t], e.ints), spec
        if op == "reshape":
            t, s = args[0]
            spec = self.reshape_spec(gargs[0].shape, s, gshape)
            return self.node(gt.type, self.local(gshape, spec), op, [t]), spec
        if op == "slice":
            t, s = args[0]
            r = len(s)
            st, ln, sd = list(e.ints[:r]), list(e.ints[r:2 * r]), list(e.ints[2 * r:])
            for d in range(r):
                if s[d] is not None:
                    if st[d] != 0 or ln[d] != gargs[0].shape[d] or sd[d] != 1:
                        raise ShardingError("slice along a split dimension")
                    ln[d] = t.shape[d]
            return self.node(gt.type, self.local(gshape, s), op, [t], st + ln + sd), s
        if op == "pad":
            # padding along dimensions that are not split; the split ones pass through unchanged
            (t, s), (pv, _) = args
            r = len(s)
            lo, hi, it = e.ints[:r], e.ints[r:2 * r], e.ints[2 * r:3 * r]
            if any(s[d] is not None and (lo[d] or hi[d] or it[d]) for d in range(r)):
                raise ShardingError("pad along a split dimension")
            return self.node(gt.type, self.local(gshape, s), op, [t, pv], e.ints), s
        if op == "concatenate":
            ax = e.ints[0]
            spec = [None] * rank
            for (t, s), ga in zip(args, gargs):
                if s[ax] is not None:
                    raise ShardingError("concatenate along a split dimension")
                for d, a in enumerate(s):
                    if a is not None:
                        if spec[d] not in (None, a):
                            raise ShardingError("concatenate: inputs are split differently")
                        spec[d] = a
            spec = tuple(spec)
            new_args = [self.reshard_replicated(t, ga.shape, s, spec) for (t, s), ga in zip(args, gargs)]
            return self.node(gt.type, self.local(gshape, spec), op, new_args, e.ints), spec
        raise ShardingError(f"op :{op} cannot be partitioned by this compiler")

    def reshape_spec(self, ishape, ispec, oshape):
        """Carry a split through a reshape: allowed when the split dimension is the
        most significant one of its group of merged / divided dimensions."""
        spec = [None] * len(oshape)
        i = j = 0
        while i < len(ishape) or j < len(oshape):
            gi, gj = [i], [j]
            pi = ishape[i] if i < len(ishape) else 1
            pj = oshape[j] if j < len(oshape) else 1
            i, j = i + 1, j + 1
            while pi != pj:
                if pi < pj:
                    pi *= ishape[i]; gi.append(i); i += 1
                else:
                    pj *= oshape[j]; gj.append(j); j += 1
            gi = [d for d in gi if d < len(ishape)]
            gj = [d for d in gj if d < len(oshape)]
            split = [d for d in gi if ispec[d] is not None]
            if not split:
                continue
            lead_i = [d for d in gi if ishape[d] != 1]
            lead_j = [d for d in gj if oshape[d] != 1]
            if len(split) > 1 or split[0] != lead_i[0] or not lead_j:
                raise ShardingError("reshape moves a split dimension to a minor position")
            a = ispec[split[0]]
            if oshape[lead_j[0]] % self.mesh.shape[a]:
                raise ShardingError("reshape: the split does not divide the new leading dimension")
            spec[lead_j[0]] = a
        return tuple(spec)


def partition(fun, mesh, input_shardings, local_templates, partition_index):
    """Trace ``fun`` on global shapes and return ``(serialised local program,
    output container spec, output shardings)`` for one partition."""
    from . import backend as B
    from . import defn
    flat = []
    spec_tree = [defn._flatten(t, flat) for t in local_templates]
    shardings = validate_shardings(mesh, [t.shape for t in flat], input_shardings)
    gparams = [E.parameter(t.type, global_shape(t.shape, s, mesh), i) for i, (t, s) in enumerate(zip(flat, shardings))]
    it = iter(gparams)
    args = [defn._unflatten(s, it) for s in spec_tree]
    with B.trace_scope():
        result = fun(*args)
        outs = []
        ospec = defn._flatten(result, outs)
        outs = [B.to_expr(o) for o in outs]
    part = _Part(mesh, mesh.coords(partition_index))
    local_outs, out_specs = [], []
    for o in outs:
        t, s = part.visit(o, shardings)
        local_outs.append(t)
        out_specs.append(s)
    return E.serialize(local_outs), ospec, out_specs


def fused_all_reduce_launches():
    """How many products this process ran as one kernel with their all-reduce."""
    import ctypes as C
    from . import nif
    n = C.c_uint64(0)
    nif.check(nif.lib().nxb200_comm_fused_launches(C.byref(n)))
    return n.value


def tensor_parallel_axes(blob_nodes):
    """Mesh axes a program all-reduces over (from its all_reduce nodes)."""
    return sorted({n.ints[0] for n in blob_nodes if n.op == "all_reduce"})


def shard_jit(fun, mesh, input_shardings, partition_index, device=None, **opts):
    """``EXLA.shard_jit(fun, mesh, input_shardings: ...)`` for the partition this
    process owns.  The communicator for the tensor-parallel group must have been
    set up with `init_tensor_parallel_group` when the program contains a split
    contraction."""
    from . import backend as B
    from . import defn
    cache = {}

    def prepare(*local_args):
        """Partition and build for these arguments without running (so that the ranks can meet
        at a host barrier before the first run: kernels that wait on peers are bounded)."""
        flat, _ = defn._templates(local_args)
        key = tuple((t.type, t.shape) for t in flat)
        if key not in cache:
            blob, ospec, out_specs = partition(fun, mesh, input_shardings, list(local_args), partition_index)
            cache[key] = (defn.Program(blob), ospec, out_specs)
        return flat, cache[key]

    def run(*local_args):
        flat, (prog, ospec, _) = prepare(*local_args)
        dev = B._device_of(device)
        args = [B.backend_transfer(a, dev) for a in flat]
        outs = prog.run(args, dev)
        return defn._unflatten(ospec, iter(outs))

    run.cache = cache
    run.prepare = prepare
    return run


def torch_exchange():
    """An ``exchange`` for `init_tensor_parallel_group` on top of an initialised
    torch.distributed process group (the plumbing a one-process-per-GPU launch
    already has): every rank contributes ``(group_key, id or None)`` and picks
    the id of its own group."""
    import torch.distributed as dist

    def exchange(key, payload):
        objs = [None] * dist.get_world_size()
        dist.all_gather_object(objs, (key, payload))
        for k, p in objs:
            if k == key and p is not None:
                return p
        raise RuntimeError("no member of the tensor-parallel group published a communicator id")
    return exchange


def torch_gather():
    """A ``gather`` for `init_tensor_parallel_group` on top of torch.distributed:
    every rank contributes ``(group_key, rank_in_group, payload)`` and receives
    its group's payloads in rank order."""
    import torch.distributed as dist

    def gather(key, rank_in_group, payload):
        objs = [None] * dist.get_world_size()
        dist.all_gather_object(objs, (key, rank_in_group, payload))
        mine = sorted((r, p) for k, r, p in objs if k == key)
        return [p for _, p in mine]
    return gather


def init_tensor_parallel_group(mesh, axis, partition_index, device, exchange, gather=None, peer_elems=0):
    """Create the NCCL communicator of the partitions that differ only in their
    coordinate along ``axis``.  ``exchange(group_key, payload_or_None)`` is the
    host's way to hand the 128-byte id from the group's first member to the
    others (e.g. a torch.distributed broadcast or a key-value store).

    With ``gather(group_key, rank_in_group, payload) -> [payloads in rank order]``
    and ``peer_elems`` > 0 the group also maps a region of every member's GPU
    memory into every process (CUDA IPC), sized for matrices of ``peer_elems``
    16-bit elements; a row-parallel product followed by the sum over ranks then
    runs as one kernel over that memory instead of a product plus an NCCL call.
    Returns True when that path is enabled."""
    import ctypes as C
    from . import nif
    lib = nif.lib()
    coords = mesh.coords(partition_index)
    n = mesh.shape[axis]
    key = tuple(c for i, c in enumerate(coords) if i != axis)
    rank_in_group = coords[axis]
    if n == 1:
        return False
    if rank_in_group == 0:
        buf = C.create_string_buffer(nif.COMM_ID_BYTES)
        nif.check(lib.nxb200_comm_id(buf))
        ident = exchange(key, buf.raw)
    else:
        ident = exchange(key, None)
    nif.check(lib.nxb200_comm_init(device, rank_in_group, n, ident))
    if gather is None or peer_elems <= 0 or n > 8:
        return False
    blob = C.create_string_buffer(nif.COMM_PEER_BLOB_BYTES)
    nif.check(lib.nxb200_comm_peer_alloc(device, int(peer_elems), blob))
    blobs = gather(key, rank_in_group, blob.raw)
    if len(blobs) != n:
        raise RuntimeError(f"peer memory set-up gathered {len(blobs)} blobs for a group of {n}")
    enabled = C.c_int(0)
    nif.check(lib.nxb200_comm_peer_open(b"".join(blobs), C.byref(enabled)))
    # the members must agree, or some would wait in the fused kernel for the others' NCCL call
    votes = gather(key, rank_in_group, bool(enabled.value))
    if any(votes) and not all(votes):
        raise RuntimeError("peer memory was mapped on some ranks of the group only")
    return bool(enabled.value)
