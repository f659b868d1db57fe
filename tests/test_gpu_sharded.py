"""Sharded decoder block on two GPUs, one process per GPU: batch data-parallel, and
tensor-parallel linears with the sum over ranks done both ways - as an NCCL call after the
product and fused into the product kernel over peer memory.  Skipped on a single-GPU
machine; the partitioning logic also runs on CPU over gloo in test_sharding_cpu.py."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
import numpy as np
import torch, torch.distributed as dist
root = sys.argv[1]
sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "oracle")); sys.path.insert(0, os.path.join(root, "tests"))
import nx_oracle as O
from helpers import host_tensor
from nx_b200 import backend, configs, defn, nx, sharding
rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
backend.set_default_backend("b200", local)
block = configs.make_decoder_block(n_heads=8)
inputs = configs.decoder_inputs(batch=world, seq=128, hidden=512, inter=1024)   # `world` row tiles: one per rank
host = [host_tensor(a, t) for a, t in inputs]
blob, _ = defn.build_program(block, host)
(full, _, _), = O.run_program(blob, [h.data.raw for h in host], "xla_like")

def shard(a, sh, mesh):
    for dim, axes in sh.items():
        n = mesh.shape[axes[0]]
        c = mesh.coords(rank)[axes[0]]
        step = a.shape[dim] // n
        a = np.take(a, range(c * step, (c + 1) * step), axis=dim)
    return np.ascontiguousarray(a)

def close(got, want):
    err = np.abs(got.astype(np.float64) - want)
    return bool((err <= 1e-2 + 2e-2 * np.abs(want)).all())

# batch data-parallel: no collective, each rank owns one batch entry
mesh = sharding.Mesh("dp", (world,))
sh = [{0: [0]}] + [{}] * 9
f = sharding.shard_jit(block, mesh, sh, rank, device=local)
out = nx.to_numpy(f(*[nx.tensor(shard(a, s, mesh), t) for (a, t), s in zip(inputs, sh)]))
assert out.shape == (1, 128, 512)
assert close(out, full[rank:rank + 1]), "data-parallel shard differs from the oracle"

# tensor-parallel linears: one all-reduce after Wo and one after Wdown
mesh = sharding.Mesh("tp", (world,))
peer = sharding.init_tensor_parallel_group(mesh, 0, rank, local, sharding.torch_exchange(),
                                           gather=sharding.torch_gather(), peer_elems=world * 128 * 512)
assert peer, "distinct GPUs of one machine must be able to map each other's memory"
sh = [{}, {1: [0]}, {1: [0]}, {1: [0]}, {0: [0]}, {1: [0]}, {1: [0]}, {0: [0]}, {}, {}]
f = sharding.shard_jit(block, mesh, sh, rank, device=local)
args = [nx.tensor(shard(a, s, mesh), t) for (a, t), s in zip(inputs, sh)]
f.prepare(*args)
dist.barrier()
# the NCCL form first (product, then ncclAllReduce), then the product fused with the sum over peer memory
os.environ["NXB200_FUSED_ALLREDUCE"] = "never"
out_nccl = nx.to_numpy(f(*args))
assert sharding.fused_all_reduce_launches() == 0
os.environ["NXB200_FUSED_ALLREDUCE"] = "always"      # these products are far too small for the automatic choice
dist.barrier()
outs = [nx.to_numpy(f(*args)) for _ in range(3)]
assert sharding.fused_all_reduce_launches() == 6, sharding.fused_all_reduce_launches()
prog = list(f.cache.values())[0][0]
assert prog.describe().count("all_reduce") == 2
for out in [out_nccl] + outs:
    assert out.shape == (world, 128, 512)
    assert close(out, full), "tensor-parallel result differs from the oracle"
# repeated fused runs are bit-identical, and both ranks hold the same bits
assert all(np.array_equal(outs[0], o) for o in outs[1:])
t = torch.from_numpy(outs[0].astype(np.float32)).cuda()
peer_t = [torch.empty_like(t) for _ in range(world)]
dist.all_gather(peer_t, t)
assert all(torch.equal(peer_t[0], o) for o in peer_t[1:]), "ranks disagree on the reduced values"
dist.barrier()
print("rank", rank, "ok")
dist.destroy_process_group()
"""


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decoder_block_data_and_tensor_parallel(tmp_path, world):
    from nx_b200 import nif
    if nif.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script), ROOT]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == world
