"""B200-native (sm_100a) implementation of the MORTAR carved block-sparse ternary SwiGLU MLP.

Layout: ``csrc/`` holds the CUDA kernels and the C ABI (declared in ``include/mortar_b200.h``
at the repository root), ``format.py`` the matrix formats and converters, ``ops.py`` the
torch-facing operators, ``torch_ops.py`` the same as registered custom ops plus the
``morph_stk::dds``-signature shim, ``modules.py`` the mirrors of the reference module API, ``synth.py``
seeded synthetic layers for tests and benchmarks, ``build.py`` the nvcc build.
"""
from . import _lib  # noqa: F401
from .format import MortarMatrix, StreamMatrix, ternary_quantize  # noqa: F401
from . import ops, synth  # noqa: F401
from . import torch_ops  # noqa: F401  (registers the mortar_b200:: custom ops)
from .modules import MortarLinear, SwiGLUMortar  # noqa: F401

__all__ = ["MortarMatrix", "StreamMatrix", "MortarLinear", "SwiGLUMortar", "ops", "synth",
           "ternary_quantize"]
