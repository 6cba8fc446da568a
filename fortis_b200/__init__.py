"""fortis_b200: B200-native gather -> NN forward -> scatter step behind the FORTIS operator surface.

The product is the C-ABI library `libfortis_b200.so` (CUDA for sm_100a; sources in fortis_b200/csrc, interface in
include/fortis_b200.h).  This package only loads it through ctypes and plays the role of the Fortran / C host in
tests and benchmarks.  There is no CPU fallback: loading fails loudly when the library has not been built
(`python -m fortis_b200.build`).
"""
from .lib import load, lib_path, FortisError  # noqa: F401
from .model import write_blob, mlp_layers, conv_layers  # noqa: F401
from .host import Host  # noqa: F401
