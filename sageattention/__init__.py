"""Drop-in name: ``from sageattention import sageattn`` resolves to the B200 implementation
(the reference exports the same names from ``sageattention/__init__.py:1-4``)."""
from .core import sageattn, sageattn_qk_int8_pv_fp16_cuda

__all__ = ["sageattn", "sageattn_qk_int8_pv_fp16_cuda"]
__version__ = "0.1.0"
