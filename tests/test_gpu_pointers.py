"""Nx.to_pointer / Nx.from_pointer (exla/test/exla/backend_test.exs "to_pointer/from_pointer"): a device
address shared inside the process, and a CUDA IPC handle mapped by a second process."""
import os
import subprocess
import sys

import numpy as np
import pytest

from nx_b200 import backend, defn, nx

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def test_local_pointer_round_trip_shares_the_memory():
    x = nx.tensor(np.arange(12, dtype=np.float32).reshape(3, 4))
    p = backend.to_pointer(x)
    assert p.kind == "local" and p.data_size == 48 and p.address
    y = backend.from_pointer(p, "f32", (3, 4))
    assert np.array_equal(nx.to_numpy(y), nx.to_numpy(x))
    z = backend.from_pointer(p, "s32", (12,))                                   # the same bytes under another type
    assert np.array_equal(nx.to_numpy(z), np.arange(12, dtype=np.float32).view(np.int32))
    # a donated in-place update of x is visible through the borrowed view
    step = defn.jit(lambda c, n: nx.put_slice(c, [1, 0], n))
    x2 = step(nx.donatable(x), nx.tensor(np.full((1, 4), -1.0, np.float32)))
    want = np.arange(12, dtype=np.float32).reshape(3, 4)
    want[1] = -1.0
    assert np.array_equal(nx.to_numpy(x2), want) and np.array_equal(nx.to_numpy(y), want)
    backend.backend_deallocate(y)                                              # releases the view, not the memory
    assert np.array_equal(nx.to_numpy(x2), want)
    with pytest.raises(ValueError, match="invalid pointer data_size"):
        backend.from_pointer(p, "f32", (5, 4))
    with pytest.raises(ValueError, match="not device memory"):
        backend.from_pointer(backend.Pointer("local", address=4096, data_size=16), "f32", (4,))


CHILD = r"""
import sys
import numpy as np
sys.path.insert(0, sys.argv[1])
from nx_b200 import backend, nx
backend.set_default_backend("b200", 0)
x = nx.tensor(np.arange(1000, dtype=np.float32) * 0.5)
p = backend.to_pointer(x, mode="ipc")
print(p.handle.hex(), p.data_size, flush=True)
sys.stdin.readline()                      # keep the allocation alive until the parent is done
"""


def test_ipc_pointer_is_mapped_by_another_process():
    child = subprocess.Popen([sys.executable, "-c", CHILD, ROOT], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        line = child.stdout.readline().split()
        assert len(line) == 2, "the exporting process failed"
        p = backend.Pointer("ipc", address=0, handle=bytes.fromhex(line[0]), data_size=int(line[1]))
        t = backend.from_pointer(p, "f32", (1000,))
        assert np.array_equal(nx.to_numpy(t), np.arange(1000, dtype=np.float32) * 0.5)
        assert np.array_equal(nx.to_numpy(defn.jit(lambda a: a * 2.0)(t)), np.arange(1000, dtype=np.float32))
        backend.backend_deallocate(t)
    finally:
        child.stdin.write("\n")
        child.stdin.flush()
        child.wait(timeout=60)
