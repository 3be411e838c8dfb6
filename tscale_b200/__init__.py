"""B200 (sm_100a) implementation of TScale's quantized attention path.

The product is the shared library libtsa_b200.so (C ABI: include/tsa.h); this package binds it for
Python callers.  Importing the package loads the library and raises if it has not been built.
"""
from . import abi

abi.lib()

from . import ops  # noqa: E402,F401
