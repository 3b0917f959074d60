"""B200-native (sm_100a) decode path for AWQ W4 g128 Llama-2 models in the llama_cu_awq packed format.

The product is the CUDA shared library behind include/q4b200.h; this package is its thin host-side
mirror of the reference's op wrappers, used by the tests and the benchmark.
"""
from . import _lib  # noqa: F401
from ._lib import Q4Error, lib  # noqa: F401
