"""strixite_b200: a B200-native (sm_100a) implementation of strixite's quantized mixture-of-experts FFN path.

The product is libstrixite_b200.so (hand-written CUDA behind a C ABI, include/strixite_b200.h). This package is the
Python host side over it: `kernels` mirrors the reference's kernel functions, `layer` its per-layer driver. Importing
the package loads the library and raises if it is missing - there is no CPU or PyTorch fallback.
"""
from ._lib import LIB_PATH, StrixError, lib  # noqa: F401
from . import kernels  # noqa: F401
from . import layer  # noqa: F401
from .kernels import Act, MoeMath, QMixStack, QWeight  # noqa: F401
from .layer import MoeLayer  # noqa: F401

__version__ = lib.strix_version().decode()
