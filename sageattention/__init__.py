"""Drop-in name: ``from sageattention import sageattn`` resolves to the B200 implementation
(the reference exports the same names from ``sageattention/__init__.py:1-4``)."""
from sageattention_rdna3_b200 import __version__, sageattn, sageattn_qk_int8_pv_fp16_cuda
from sageattention_rdna3_b200 import core

__all__ = ["sageattn", "sageattn_qk_int8_pv_fp16_cuda"]
