"""Sharded decoder block on two GPUs (one process per GPU, NCCL all-reduce for the
tensor-parallel linears).  Skipped on a single-GPU machine; the same logic runs on
CPU over gloo in test_sharding_cpu.py."""
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
rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
backend.set_default_backend("b200", local)
block = configs.make_decoder_block(n_heads=8)
inputs = configs.decoder_inputs(batch=2, seq=128, hidden=512, inter=688)
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

# batch data-parallel: no collective, each rank owns half of the batch
mesh = sharding.Mesh("dp", (2,))
sh = [{0: [0]}] + [{}] * 9
f = sharding.shard_jit(block, mesh, sh, rank, device=local)
out = nx.to_numpy(f(*[nx.tensor(shard(a, s, mesh), t) for (a, t), s in zip(inputs, sh)]))
assert out.shape == (1, 128, 512)
assert close(out, full[rank:rank + 1]), "data-parallel shard differs from the oracle"

# tensor-parallel linears: one all-reduce after Wo and one after Wdown
mesh = sharding.Mesh("tp", (2,))
sharding.init_tensor_parallel_group(mesh, 0, rank, local, sharding.torch_exchange())
sh = [{}, {1: [0]}, {1: [0]}, {1: [0]}, {0: [0]}, {1: [0]}, {1: [0]}, {0: [0]}, {}, {}]
f = sharding.shard_jit(block, mesh, sh, rank, device=local)
out = nx.to_numpy(f(*[nx.tensor(shard(a, s, mesh), t) for (a, t), s in zip(inputs, sh)]))
prog = list(f.cache.values())[0][0]
assert prog.describe().count("all_reduce") == 2
assert out.shape == (2, 128, 512)
assert close(out, full), "tensor-parallel result differs from the oracle"
dist.barrier()
print("rank", rank, "ok")
dist.destroy_process_group()
"""


def test_decoder_block_dp2_and_tp2(tmp_path):
    from nx_b200 import nif
    if nif.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script), ROOT]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == 2
