"""logos_b200 -- B200 (sm_100a) attention engine for the LOGOS model's attention path.

The product is the C-ABI shared library `liblogos_attn.so` (see include/logos_attn.h).
This package is the thin host side used by tests and the benchmark: a ctypes binding
(`logos_b200.lib`), torch-tensor front ends (`logos_b200.engine`) and the (batch x head)
sharding helpers (`logos_b200.sharding`).
"""
from .lib import LogosError, load_library, Params  # noqa: F401

__all__ = ["LogosError", "load_library", "Params"]
