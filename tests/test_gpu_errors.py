"""Failure paths of the C ABI on a real device: every misuse answers with a
status code and a message, nothing is launched for it, and the device stays
usable.  Scenarios follow the reference's tests of its native layer
(exla/test/exla/backend_test.exs:48-50 use after free; exla/c_src/exla/exla.cc:462-475
second free; exla/test/exla/memory_tracking_test.exs the counters).
"""
import ctypes as C

import numpy as np
import pytest

from nx_b200 import backend, defn, nif, nx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    backend.set_default_backend("b200", 0)
    yield
    backend.set_default_backend(None)


def _alloc(shape, dtype_code=10):
    h = C.c_void_p()
    st = nif.lib().nxb200_buffer_alloc(0, dtype_code, nif.dims_array(shape), len(shape), C.byref(h))
    return st, h


def _stats():
    a, p, r = C.c_uint64(), C.c_uint64(), C.c_uint64()
    nif.check(nif.lib().nxb200_memory_stats(0, C.byref(a), C.byref(p), C.byref(r)))
    return a.value, p.value, r.value


def test_second_deallocate_is_reported_and_use_after_free_raises():
    lib = nif.lib()
    t = nx.tensor(np.arange(4, dtype=np.int32))
    h = t.data.handle
    assert lib.nxb200_buffer_deallocate(h) == nif.OK
    flag = C.c_int(0)
    nif.check(lib.nxb200_buffer_is_deallocated(h, C.byref(flag)))
    assert flag.value == 1
    assert lib.nxb200_buffer_deallocate(h) == nif.ERR_DEALLOCATED          # {:error, :already_deallocated}
    out = (C.c_char * 16)()
    assert lib.nxb200_buffer_to_host(h, out, 16) == nif.ERR_RUNTIME        # RuntimeError in the reference
    assert "deallocated" in nif.last_error()
    with pytest.raises(RuntimeError):
        nx.to_binary(t)
    # ... and as an argument of a program
    prog = defn.compile(lambda x: x + 1, [defn.template((4,), "s32")]).program
    with pytest.raises(RuntimeError):
        prog.run([t], 0)


def test_handles_are_checked():
    lib = nif.lib()
    bogus = C.create_string_buffer(256)
    assert lib.nxb200_buffer_deallocate(C.cast(bogus, C.c_void_p)) == nif.ERR_INVALID
    assert "not a buffer handle" in nif.last_error()
    assert lib.nxb200_program_release(C.cast(bogus, C.c_void_p)) == nif.ERR_INVALID
    assert lib.nxb200_buffer_deallocate(None) == nif.ERR_INVALID


def test_wrong_device_and_wrong_signature_are_refused_before_any_launch():
    lib = nif.lib()
    prog = defn.compile(lambda x: x * 2.0, [defn.template((8,), "f32")]).program
    x = nx.tensor(np.ones(8, np.float32))
    outs = (C.c_void_p * 1)()
    args = (C.c_void_p * 1)(x.data.handle)
    n = nif.device_count()
    assert lib.nxb200_program_run(prog.handle, n + 3, args, 1, outs, 1) == nif.ERR_INVALID     # no such device
    assert "out of range" in nif.last_error()
    if n > 1:
        assert lib.nxb200_program_run(prog.handle, 1, args, 1, outs, 1) == nif.ERR_INVALID     # tensor lives on device 0
        assert "lives on device 0" in nif.last_error()
    y = nx.tensor(np.ones(9, np.float32))
    args = (C.c_void_p * 1)(y.data.handle)
    assert lib.nxb200_program_run(prog.handle, 0, args, 1, outs, 1) == nif.ERR_INVALID         # shape of the argument
    assert "program was built for" in nif.last_error()
    assert lib.nxb200_program_run(prog.handle, 0, args, 0, outs, 1) == nif.ERR_INVALID         # argument count
    # the device still works
    assert np.array_equal(nx.to_numpy(prog.run([x], 0)[0]), np.full(8, 2.0, np.float32))


def test_binary_of_the_wrong_size_is_refused():
    lib = nif.lib()
    h = C.c_void_p()
    data = np.arange(6, dtype=np.float32)
    before = _stats()[0]
    st = lib.nxb200_buffer_from_host(0, 10, nif.dims_array((2, 4)), 2, data.ctypes.data, data.nbytes, C.byref(h))
    assert st == nif.ERR_INVALID and "tensor needs 32" in nif.last_error()
    assert _stats()[0] == before                                       # nothing stays allocated


def test_allocation_larger_than_the_device_reports_out_of_memory():
    before = _stats()
    st, h = _alloc((1 << 20, 1 << 20))                                 # 4 TiB of f32
    assert st == nif.ERR_OOM
    assert "allocation" in nif.last_error()
    assert _stats()[0] == before[0]
    # the failure did not poison the context
    t = nx.tensor(np.arange(8, dtype=np.float32))
    assert np.array_equal(nx.to_numpy(t + 1.0), np.arange(8, dtype=np.float32) + 1.0)


def test_memory_counters_follow_allocation_and_release():
    """exla/test/exla/memory_tracking_test.exs: allocated follows place_on_device / deallocate byte for
    byte, the peak keeps the maximum, reset_peak brings it back to what is allocated now."""
    lib = nif.lib()
    nif.check(lib.nxb200_memory_reset_peak(0))
    base_alloc, base_peak, _ = _stats()
    assert base_peak == base_alloc
    a = nx.from_binary(np.array([1, 2, 3, 4], np.int32).tobytes(), "s32", (4,))
    alloc, peak, reserved = _stats()
    assert alloc == base_alloc + 16 and peak == base_peak + 16 and reserved >= alloc
    b = nx.from_binary(np.array([5, 6, 7, 8], np.int32).tobytes(), "s32", (4,))
    alloc, peak, _ = _stats()
    assert alloc == base_alloc + 32 and peak == base_peak + 32
    backend.backend_deallocate(a)
    alloc, peak, _ = _stats()
    assert alloc == base_alloc + 16 and peak == base_peak + 32
    nif.check(lib.nxb200_memory_reset_peak(0))
    alloc, peak, _ = _stats()
    assert peak == alloc == base_alloc + 16
    backend.backend_deallocate(b)
    assert _stats()[0] == base_alloc


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """Every kernel's waits are bounded.  The self-test runs the bounded wait on a flag that nothing
    sets, with a limit of two milliseconds: the wait gives up, the kernel returns, the host reads
    NXB_ERR_TIMEOUT, and the next program runs normally."""
    lib = nif.lib()
    assert lib.nxb200_selftest_bounded_wait(0, 2000) == nif.ERR_TIMEOUT
    assert "gave up waiting" in nif.last_error()
    assert lib.nxb200_device_synchronize(0) == nif.OK                  # the status was consumed
    x = nx.tensor(np.arange(16, dtype=np.float32))
    assert np.array_equal(nx.to_numpy(nx.sum(x)), np.float32(120.0))
    assert lib.nxb200_selftest_bounded_wait(0, 0) == nif.ERR_INVALID


def test_released_memory_is_not_reused_under_a_download_in_flight():
    """read_async, release, then a new tensor of the same size class: the download must see the old data."""
    import torch
    lib = nif.lib()
    n = 8 << 20
    src = np.arange(n, dtype=np.int32)
    t = nx.tensor(src)
    pinned = torch.empty(n, dtype=torch.int32, pin_memory=True)
    nif.check(lib.nxb200_buffer_read_async(t.data.handle, pinned.data_ptr(), n * 4))
    h, t.data.handle = t.data.handle, None
    nif.check(lib.nxb200_buffer_release(h))
    other = nx.tensor(np.full(n, -1, np.int32))                       # likely the very same block
    nif.check(lib.nxb200_device_synchronize(0))
    assert np.array_equal(pinned.numpy(), src)
    backend.backend_deallocate(other)


def test_asynchronous_upload_from_pageable_memory():
    """nxb200_buffer_from_host_async: the call returns at once, the library's uploader thread streams the
    (unpinned) source through its staging buffers and calls back when it has read the last byte; the
    tensor can be used immediately, the device's work is ordered after the copies
    (exla/c_src/exla/exla_client.cc:118-151)."""
    import threading
    from nx_b200 import types as T
    from nx_b200.nx import Tensor
    lib = nif.lib()
    n = 24 << 20                                                      # 96 MiB of f32: two dozen staging chunks
    src = np.arange(n, dtype=np.float32)
    done, seen = threading.Event(), []

    def on_done(ctx):
        seen.append(ctx)
        done.set()
    cb = nif.UPLOAD_DONE(on_done)
    h = C.c_void_p()
    nif.check(lib.nxb200_buffer_from_host_async(0, 10, nif.dims_array((n,)), 1, src.ctypes.data, src.nbytes, cb, 1234, C.byref(h)))
    t = Tensor(backend.DeviceBuffer(h.value, 0), T.F32, (n,))
    y = t * 2.0 + 1.0                                                 # queued behind the upload, no explicit wait
    assert done.wait(30), "the completion callback never fired"
    assert seen == [1234]
    assert np.array_equal(nx.to_numpy(y), src * 2.0 + 1.0)
    assert np.array_equal(nx.to_numpy(t), src)
    # several uploads in flight, released without ever being read
    hs = []
    small = np.ones(1 << 20, np.float32)
    for _ in range(4):
        h2 = C.c_void_p()
        nif.check(lib.nxb200_buffer_from_host_async(0, 10, nif.dims_array((1 << 20,)), 1, small.ctypes.data, small.nbytes, nif.UPLOAD_DONE(0), None, C.byref(h2)))
        hs.append(h2)
    for h2 in hs:
        nif.check(lib.nxb200_buffer_release(h2))
    # a binary of the wrong size is refused before anything is queued
    bad = C.c_void_p()
    assert lib.nxb200_buffer_from_host_async(0, 10, nif.dims_array((8,)), 1, src.ctypes.data, 16, cb, None, C.byref(bad)) == nif.ERR_INVALID
