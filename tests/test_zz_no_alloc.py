"""The allocation-free matrix product (`nxb200_dot_bf16_static_scratch`).

Callers that have given the device's memory to another allocator, or that cannot
afford the stall of a device allocation in their serving loop, use this entry
point with buffers they own; its scratch is a fixed array inside the library.
The test drives it through the C ABI twice in a row on different data (the
array keeps the previous call's contents, so the second call proves nothing
stale is read) and checks both results bit for bit against the regular
`program_run` path, which runs the same tensor-core kernel, and against the
CPU oracle within the bf16 tolerance (rtol 2e-2, atol 1e-2).

This file sorts last on purpose: a run that stops at the first failure has
already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

import nx_oracle as O
from helpers import assert_close
from nx_b200 import backend, defn, nif, nx

pytestmark = pytest.mark.gpu


def _raw_pointer(t):
    p = C.c_void_p()
    nif.check(nif.lib().nxb200_buffer_device_pointer(t.data.handle, C.byref(p)))
    return p


def test_static_scratch_dot_matches_regular_path_twice():
    backend.set_default_backend("b200", 0)
    try:
        lib = nif.lib()
        stream = C.c_void_p()
        nif.check(lib.nxb200_device_stream(0, C.byref(stream)))
        rng = np.random.default_rng(7)
        regular = defn.jit(lambda x, y: nx.dot(x, y))
        for m, n, k in [(300, 520, 264), (128, 1024, 4096)]:
            a = nx.tensor(rng.normal(0, 1 / np.sqrt(k), (m, k)).astype(np.float32), "bf16")
            b = nx.tensor(rng.normal(0, 1, (k, n)).astype(np.float32), "bf16")
            want = nx.to_binary(regular(a, b))
            out = nx.tensor(np.zeros((m, n), np.float32), "bf16")      # caller-owned output buffer
            st = lib.nxb200_dot_bf16_static_scratch(0, _raw_pointer(a), _raw_pointer(b), _raw_pointer(out), m, n, k, stream)
            nif.check(st)
            assert nx.to_binary(out) == want, f"{m}x{n}x{k}: differs from the regular entry point"
            blob, _ = defn.build_program(lambda x, y: nx.dot(x, y), [defn.template((m, k), "bf16"), defn.template((k, n), "bf16")])
            (ref, _, _), = O.run_program(blob, [nx.to_binary(a), nx.to_binary(b)], "xla_like")
            assert_close(nx.to_numpy(out), ref, 2e-2, 1e-2, f"{m}x{n}x{k} against the oracle")
    finally:
        backend.set_default_backend(None)


def test_static_scratch_dot_rejects_what_does_not_fit():
    backend.set_default_backend("b200", 0)
    try:
        lib = nif.lib()
        a = nx.tensor(np.zeros((8, 8), np.float32), "bf16")
        p = _raw_pointer(a)
        # k*n beyond the 32 MiB array
        assert lib.nxb200_dot_bf16_static_scratch(0, p, p, p, 8, 8192, 4096, None) == nif.ERR_INVALID
        assert "scratch" in nif.last_error()
        # rows that would not start on 16-byte boundaries
        assert lib.nxb200_dot_bf16_static_scratch(0, p, p, p, 8, 8, 12, None) == nif.ERR_INVALID
        assert lib.nxb200_dot_bf16_static_scratch(0, None, p, p, 8, 8, 8, None) == nif.ERR_INVALID
        # a result pointer that is not 16-byte aligned is refused on the host; nothing is launched
        odd = C.c_void_p(p.value + 2)
        assert lib.nxb200_dot_bf16_static_scratch(0, p, p, odd, 8, 8, 8, None) == nif.ERR_INVALID
        assert "aligned" in nif.last_error()
        assert lib.nxb200_dot_bf16_static_scratch(0, p, odd, p, 8, 8, 8, None) == nif.ERR_INVALID
    finally:
        backend.set_default_backend(None)
