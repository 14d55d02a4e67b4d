"""motifcl_b200: a B200 (sm_100a) implementation of MotifCL's counter-synapse linear path.

The product is the CUDA library lib/libmotifcl_cuda.so behind the C ABI of
include/motifcl_cuda.h; this package is its Python face.
"""
from ._lib import LIB_PATH, MotifclCudaError, build_library, declared_symbols, lib  # noqa: F401
from . import codec, synth  # noqa: F401


def __getattr__(name):
    # torch-dependent parts are imported on first use so that the codec and the loader work
    # in processes that never touch a GPU.
    if name == "Context":
        from .runtime import Context
        return Context
    if name == "CounterStateLinear":
        from .counter import CounterStateLinear
        return CounterStateLinear
    raise AttributeError(name)
