"""ctypes binding of libnxb200.so — the stand-in for the Erlang NIF shim.

Mirrors exla/lib/exla/nif.ex:5-21: the shared library is loaded once from the
package's own directory and every call maps a non-zero status to an exception
carrying the runtime's message (exla/c_src/exla/exla.cc:280-292).  There is no
fallback: if the library is missing or a call fails, the error propagates.
"""
from __future__ import annotations

import ctypes as C
import os

_LIB = None
LIB_NAME = "libnxb200.so"
MAX_RANK = 8
COMM_ID_BYTES = 128
COMM_PEER_BLOB_BYTES = 80

OK, ERR_INVALID, ERR_RUNTIME, ERR_DEALLOCATED, ERR_OOM, ERR_UNSUPPORTED, ERR_NO_DEVICE, ERR_TIMEOUT = \
    0, -1, -2, -3, -4, -5, -6, -7


class AlreadyDeallocated(RuntimeError):
    """{:error, :already_deallocated} (exla/c_src/exla/exla.cc:462-475)."""


class Unsupported(NotImplementedError):
    pass


def lib_path():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


def lib():
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(the backend has no other execution path)")
        _LIB = C.CDLL(path, mode=C.RTLD_GLOBAL)
        _declare(_LIB)
        check(_LIB.nxb200_init())
    return _LIB


UPLOAD_DONE = C.CFUNCTYPE(None, C.c_void_p)      # void (*nxb200_upload_done)(void *ctx)


def _declare(l):
    vp, i32, sz = C.c_void_p, C.c_int, C.c_size_t
    p = C.POINTER
    l.nxb200_last_error.restype = sz
    l.nxb200_last_error.argtypes = [C.c_char_p, sz]
    sigs = {
        "nxb200_init": [],
        "nxb200_device_count": [p(i32)],
        "nxb200_buffer_from_host": [i32, i32, p(C.c_int64), i32, vp, sz, p(vp)],
        "nxb200_buffer_alloc": [i32, i32, p(C.c_int64), i32, p(vp)],
        "nxb200_buffer_from_host_async": [i32, i32, p(C.c_int64), i32, vp, sz, UPLOAD_DONE, vp, p(vp)],
        "nxb200_buffer_to_host": [vp, vp, sz],
        "nxb200_buffer_write_async": [vp, vp, sz],
        "nxb200_buffer_read_async": [vp, vp, sz],
        "nxb200_buffer_copy_to_device": [vp, i32, p(vp)],
        "nxb200_buffer_info": [vp, p(i32), p(C.c_int64), p(i32), p(i32)],
        "nxb200_buffer_device_pointer": [vp, p(vp)],
        "nxb200_buffer_deallocate": [vp],
        "nxb200_buffer_is_deallocated": [vp, p(i32)],
        "nxb200_buffer_release": [vp],
        "nxb200_program_build": [vp, sz, p(vp)],
        "nxb200_program_io": [vp, p(i32), p(i32)],
        "nxb200_program_output_info": [vp, i32, p(i32), p(C.c_int64), p(i32)],
        "nxb200_program_run": [vp, i32, p(vp), i32, p(vp), i32],
        "nxb200_program_run_into": [vp, i32, p(vp), i32, p(vp), i32],
        "nxb200_program_release": [vp],
        "nxb200_program_launch_count": [vp, p(i32)],
        "nxb200_program_build_times": [vp, p(C.c_double), p(C.c_double)],
        "nxb200_device_synchronize": [i32],
        "nxb200_timer_begin": [i32],
        "nxb200_timer_end": [i32, p(C.c_float)],
        "nxb200_device_stream": [i32, p(vp)],
        "nxb200_selftest_bounded_wait": [i32, C.c_uint32],
        "nxb200_memory_stats": [i32, p(C.c_uint64), p(C.c_uint64), p(C.c_uint64)],
        "nxb200_memory_reset_peak": [i32],
        "nxb200_buffer_from_pointer": [i32, i32, C.POINTER(C.c_int64), i32, vp, C.POINTER(vp)],
        "nxb200_buffer_ipc_export": [vp, C.c_char_p],
        "nxb200_buffer_from_ipc": [i32, i32, C.POINTER(C.c_int64), i32, C.c_char_p, C.POINTER(vp)],
        "nxb200_comm_id": [C.c_char_p],
        "nxb200_comm_init": [i32, i32, i32, C.c_char_p],
        "nxb200_comm_all_reduce_sum": [vp],
        "nxb200_comm_peer_alloc": [i32, C.c_uint64, C.c_char_p],
        "nxb200_comm_peer_open": [C.c_char_p, C.POINTER(C.c_int)],
        "nxb200_comm_fused_launches": [C.POINTER(C.c_uint64)],
        "nxb200_comm_destroy": [],
        "nxb200_dot_bf16_static_scratch": [i32, vp, vp, vp, C.c_int64, C.c_int64, C.c_int64, vp],
    }
    for name, args in sigs.items():
        f = getattr(l, name)
        f.restype = i32
        f.argtypes = args
    l.nxb200_program_describe.restype = sz
    l.nxb200_program_describe.argtypes = [vp, C.c_char_p, sz]
    l.nxb200_program_kernel_source.restype = sz
    l.nxb200_program_kernel_source.argtypes = [vp, i32, C.c_char_p, sz]


def last_error():
    buf = C.create_string_buffer(4096)
    _LIB.nxb200_last_error(buf, len(buf))
    return buf.value.decode("utf-8", "replace")


def check(status):
    if status == OK:
        return
    msg = last_error()
    if status == ERR_INVALID:
        raise ValueError(msg)
    if status == ERR_DEALLOCATED:
        raise AlreadyDeallocated(msg)
    if status == ERR_UNSUPPORTED:
        raise Unsupported(msg)
    if status == ERR_OOM:
        raise MemoryError(msg)
    if status == ERR_TIMEOUT:
        raise TimeoutError(msg)
    raise RuntimeError(msg)


def device_count():
    n = C.c_int(0)
    check(lib().nxb200_device_count(C.byref(n)))
    return n.value


def dims_array(shape):
    return (C.c_int64 * MAX_RANK)(*shape)
