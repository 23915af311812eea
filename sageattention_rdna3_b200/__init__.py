"""B200-native INT8 SageAttention: ``sageattn`` of LuXuxue/sageattention-rdna3 on sm_100a kernels."""
from .core import check_status, sageattn, sageattn_qk_int8_pv_fp16_cuda
from .host_pipeline import sageattn_host
from .context_parallel import sageattn_context_parallel
from .kv_cache import QuantizedKV, quantize_kv, sageattn_quantized_kv

__version__ = "0.1.0"
__all__ = ["sageattn", "sageattn_qk_int8_pv_fp16_cuda", "sageattn_host", "check_status", "QuantizedKV",
           "quantize_kv", "sageattn_quantized_kv", "sageattn_context_parallel"]
