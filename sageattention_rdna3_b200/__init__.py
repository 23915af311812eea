"""B200-native INT8 SageAttention: ``sageattn`` of LuXuxue/sageattention-rdna3 on sm_100a kernels."""
from .core import check_status, sageattn, sageattn_qk_int8_pv_fp16_cuda

__version__ = "0.1.0"
__all__ = ["sageattn", "sageattn_qk_int8_pv_fp16_cuda", "check_status"]
