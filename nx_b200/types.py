"""Nx element types and the promotion rules the hot path depends on.

A type is a ``(kind, bits)`` tuple exactly like the reference's ``{kind, bits}``
(nx/lib/nx/type.ex:27-48): kind is one of ``"u" "s" "f" "bf"``.  Complex and
8-bit float types are outside the hot path and are rejected.
"""
from __future__ import annotations

import math

U8, U16, U32, U64 = ("u", 8), ("u", 16), ("u", 32), ("u", 64)
S8, S16, S32, S64 = ("s", 8), ("s", 16), ("s", 32), ("s", 64)
F16, BF16, F32, F64 = ("f", 16), ("bf", 16), ("f", 32), ("f", 64)

# wire codes shared with include/nxb200.h (nxb200_dtype)
DTYPE_CODES = {U8: 0, U16: 1, U32: 2, U64: 3, S8: 4, S16: 5, S32: 6, S64: 7,
               F16: 8, BF16: 9, F32: 10, F64: 11}
CODE_DTYPES = {v: k for k, v in DTYPE_CODES.items()}

_SHORT = {"u8": U8, "u16": U16, "u32": U32, "u64": U64, "s8": S8, "s16": S16,
          "s32": S32, "s64": S64, "f16": F16, "bf16": BF16, "f32": F32, "f64": F64}


def normalize(t):
    """nx/lib/nx/type.ex:190-230 (normalize!): accept tuple or short name."""
    if isinstance(t, str):
        if t not in _SHORT:
            raise ValueError(f"invalid numerical type: {t!r}")
        return _SHORT[t]
    t = tuple(t)
    if t not in DTYPE_CODES:
        raise ValueError(f"invalid numerical type: {t!r}")
    return t


def short(t):
    return f"{t[0]}{t[1]}"


def itemsize(t):
    return t[1] // 8


def is_integer(t):
    return t[0] in ("u", "s")


def is_float(t):
    return t[0] in ("f", "bf")


_ORDER = {"u": 0, "s": 1, "bf": 2, "f": 3}


def merge(a, b):
    """nx/lib/nx/type.ex:463-473."""
    if a[0] == b[0]:
        return (a[0], max(a[1], b[1]))
    lo, hi = (a, b) if _ORDER[a[0]] < _ORDER[b[0]] else (b, a)
    if lo[0] == "u" and hi[0] == "s":
        return ("s", max(min(lo[1] * 2, 64), hi[1]))
    return hi


def _unsigned_size(n):
    for bits in (8, 16, 32):
        if n < (1 << bits):
            return bits
    return 64


def _signed_size(n):
    for bits in (8, 16, 32):
        if -(1 << (bits - 1)) <= n < (1 << (bits - 1)):
            return bits
    return 64


def merge_number(t, number):
    """nx/lib/nx/type.ex:536-566 (merge_number)."""
    is_int = isinstance(number, int) and not isinstance(number, bool)
    if t[0] == "u" and is_int and number >= 0:
        return ("u", max(_unsigned_size(number), t[1]))
    if t[0] == "u" and is_int:
        return merge_number(("s", min(t[1] * 2, 64)), number)
    if t[0] == "s" and is_int:
        return ("s", max(_signed_size(number), t[1]))
    if t[0] in ("bf", "f"):
        return t
    return F32


def infer(number):
    """nx/lib/nx/type.ex:173-177."""
    if isinstance(number, bool):
        return U8
    if isinstance(number, int):
        return S32
    return F32


def to_floating(t):
    """nx/lib/nx/type.ex (to_floating): integers become f32, floats stay."""
    return t if is_float(t) else F32


def to_aggregate(t):
    """nx/lib/nx/type.ex:329-333."""
    if t == U64:
        return S64
    if t[0] == "u":
        return U32
    if t == S64:
        return S64
    if t[0] == "s":
        return S32
    return t


def min_value(t):
    """Lowest value of a type: -inf for floats (what reduce_max starts from,
    exla/lib/exla/lib.ex:158-171)."""
    if is_float(t):
        return -math.inf
    return 0 if t[0] == "u" else -(1 << (t[1] - 1))


def max_value(t):
    if is_float(t):
        return math.inf
    return (1 << t[1]) - 1 if t[0] == "u" else (1 << (t[1] - 1)) - 1
