"""nx_b200 — host side of a B200-native Nx backend and defn compiler.

``nx_b200.nx``       the slice of the Nx API above the hot path (type/shape inference)
``nx_b200.expr``     the defn expression graph and its wire format
``nx_b200.defn``     the Nx.Defn.Compiler callbacks, jit/compile, program cache
``nx_b200.backend``  the Nx.Backend callbacks (device storage + eager ops)
``nx_b200.nif``      binding of the C ABI in include/nxb200.h
"""
from . import types, expr, nx, backend, defn  # noqa: F401

__all__ = ["types", "expr", "nx", "backend", "defn"]
