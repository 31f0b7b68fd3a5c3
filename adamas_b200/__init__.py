"""adamas_b200: the per-step decode hot path of Adamas sparse attention (code append, distance
estimate, top-k, sparse paged decode attention) as hand-written sm_100a CUDA behind a C ABI.

``adamas_b200._kernels`` has the surface of the reference's ``adamas._kernels`` extension and
``adamas_b200.utils`` that of ``adamas.utils``.  Importing the package loads
``libadamas_b200.so``; it raises if the library has not been built.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from . import _kernels, utils
from ._kernels import hadamard_transform

__version__ = "0.1.0"
__all__ = ["_kernels", "utils", "hadamard_transform"]
