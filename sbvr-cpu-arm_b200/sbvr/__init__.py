"""SBVR on B200: same import surface as the reference package (`sbvr/__init__.py:1`):
`sbvr.sbvr`, `sbvr._sbvr_serialized`, `sbvr.load`, `sbvr.mm_T`, plus `sbvr.linear` for fp16
activations.  Importing it loads the CUDA library; there is no CPU implementation."""
import torch

from .core import sbvr, _sbvr_serialized, load, mm_T, linear, row_deq_mm_T  # noqa: F401
from . import _lib, sbvr_cuda  # noqa: F401
from .sbvr_cuda import _sbvr_mm_T, _sbvr_row_deq_mm_T, _sbvr_cuda_init  # noqa: F401  (reference sbvr/__init__.py:2)

# files written by `save` pickle this class by name (reference sbvr/__init__.py:8)
torch.serialization.add_safe_globals([_sbvr_serialized])
