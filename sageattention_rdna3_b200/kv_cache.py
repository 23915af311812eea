"""Keys and values that are quantised once and attended to many times.

``sageattn`` quantises Q and K on every call (``sageattention/core.py:191-198``); the operator
boundary already separates that step from the attention launch (``csrc/pybind_gfx11.cpp:19-35``).
When K and V do not change between calls - cross-attention to a text encoder over the steps of a
diffusion sampler, a prefix that many queries share - the K half of the work (the mean, the INT8
tensor and its scales, the fp16 copy of a bf16 V) can be kept:

    kv = quantize_kv(k, v, tensor_layout="HND", smooth_k=True)
    for q in queries:
        o = sageattn_quantized_kv(q, kv, is_causal=False)

The result is bit-identical to ``sageattn(q, k, v, ..., kernel="int8")``: the same kernels run on
the same values, only fewer of them per call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

import torch

from . import _native
from .core import _LAYOUT_CODE, _aligned, _status_word


@dataclass
class QuantizedKV:
    """What the attention launch needs of K and V."""
    k_int8: torch.Tensor            # [B,Hkv,Skv,D] int8
    k_scale: torch.Tensor           # [B,Hkv,ceil(Skv/16)] fp32
    v16: torch.Tensor               # fp16 V; [B,Hkv,Skv,D] for bf16 inputs, the caller's tensor for fp16
    v_layout: int                   # layout code of v16
    k_mean: Optional[torch.Tensor]  # [B,Hkv,D] in the input dtype when smooth_k, else None
    tensor_layout: str
    dtype: torch.dtype              # dtype of the k, v (and expected q) tensors

    @property
    def kv_len(self) -> int:
        return self.k_int8.size(2)

    @property
    def num_kv_heads(self) -> int:
        return self.k_int8.size(1)


def quantize_kv(k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND", smooth_k: bool = False) -> QuantizedKV:
    """The K/V half of ``sageattn``'s INT8 path: [K mean] and one quantisation launch.

    The int8 keys, their scales and the mean are snapshots.  The values are a snapshot only for bf16
    inputs (an fp16 copy is made); for fp16 inputs ``v16`` IS the caller's ``v``, not a copy: writing
    into ``v`` afterwards changes what later ``sageattn_quantized_kv`` calls read while the keys stay
    as they were.  Pass ``v.clone()`` if the tensor will be reused."""
    assert k.is_cuda and v.is_cuda and k.device == v.device, "k, v must be CUDA tensors on one device."
    assert k.dtype == v.dtype and k.dtype in (torch.float16, torch.bfloat16), "k, v must both be fp16 or bf16."
    assert tensor_layout in _LAYOUT_CODE, f"tensor_layout must be 'HND' or 'NHD', got {tensor_layout!r}."
    assert k.dim() == 4 and k.shape == v.shape, "k and v must be 4-D tensors of the same shape."
    assert k.size(-1) in (64, 128), f"head_dim must be 64 or 128, got {k.size(-1)}."
    assert k.stride(-1) == 1 and v.stride(-1) == 1, "Last dim of kv must be contiguous."
    ops = _native.load_ops()
    layout = _LAYOUT_CODE[tensor_layout]
    if not _aligned(k):
        k = k.contiguous()
    if not _aligned(v):
        v = v.contiguous()
    seq_dim = 2 if tensor_layout == "HND" else 1
    k_mean = ops.mean_seq(k, layout) if (smooth_k and k.size(seq_dim) > 0) else None
    mean_arg = k_mean if k_mean is not None else torch.empty(0, device=k.device, dtype=k.dtype)
    no_q = k.narrow(seq_dim, 0, 0)          # an empty query: only the K (and V) blocks of the launch exist
    if k.dtype == torch.bfloat16:
        _, _, k_int8, k_scale, v16 = ops.prep_qkv(no_q, k, v, mean_arg, layout, 1.0)
        v_layout = _LAYOUT_CODE["HND"]
    else:
        _, _, k_int8, k_scale = ops.quant_qk_int8(no_q, k, mean_arg, layout, 1.0)
        v16, v_layout = v, layout
    return QuantizedKV(k_int8, k_scale, v16, v_layout, k_mean, tensor_layout, k.dtype)


def sageattn_quantized_kv(q: torch.Tensor, kv: QuantizedKV, is_causal: bool = False,
                          sm_scale: Optional[float] = None, return_lse: bool = False
                          ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """``sageattn`` (INT8 kernel) against keys and values prepared by :func:`quantize_kv`.

    q: fp16 / bf16 in ``kv.tensor_layout``, same dtype as the cached k, v.  Returns O shaped like q, and
    with ``return_lse`` the log-sum-exp ``[B,Hq,Sq]`` (referring to the original keys: the smooth_k
    shift is added back)."""
    assert q.is_cuda and q.device == kv.k_int8.device, "q must be on the device of the cached keys."
    assert q.dtype == kv.dtype, f"q must be {kv.dtype}, like the cached keys."
    assert q.dim() == 4 and q.stride(-1) == 1, "q must be a 4-D tensor with a contiguous last dim."
    headdim = q.size(-1)
    assert headdim == kv.k_int8.size(3), "head_dim of q and of the cached keys differ."
    assert q.stride(0) % 8 == 0 and q.stride(1) % 8 == 0 and q.stride(2) % 8 == 0, (
        f"q strides must be multiples of 8 elements (16-byte write-back); got {q.stride()}."
    )
    tensor_layout = kv.tensor_layout
    layout = _LAYOUT_CODE[tensor_layout]
    seq_dim, head_idx = (2, 1) if tensor_layout == "HND" else (1, 2)
    B, Hq, q_len = q.size(0), q.size(head_idx), q.size(seq_dim)
    assert B == kv.k_int8.size(0) and Hq % max(kv.num_kv_heads, 1) == 0, (
        "batch sizes must match and num_qo_heads must be a multiple of num_kv_heads."
    )
    if sm_scale is None:
        sm_scale = headdim ** -0.5
    if q.data_ptr() % 16 != 0:
        q = q.clone(memory_format=torch.contiguous_format)
    ops = _native.load_ops()
    o = torch.empty_like(q)
    lse = torch.full((B, Hq, q_len), float("-inf"), dtype=torch.float32, device=q.device) if return_lse else None
    if q_len == 0 or B == 0 or Hq == 0:
        pass
    elif kv.kv_len == 0:
        o.zero_()
    else:
        shape = list(q.shape)
        shape[seq_dim], shape[head_idx] = 0, kv.num_kv_heads
        no_k = q.new_empty(shape)           # an empty key: only the Q blocks of the launch exist
        q_int8, q_scale, _, _ = ops.quant_qk_int8(q, no_k, q.new_empty(0), layout, sm_scale)
        ops.qk_int8_sv_f16_attn(q_int8, kv.k_int8, kv.v16, o, q_scale, kv.k_scale, layout, int(is_causal), sm_scale,
                                value_layout=kv.v_layout, status=_status_word(q.device), lse=lse)
        if return_lse and kv.k_mean is not None:
            km = kv.k_mean.float().repeat_interleave(Hq // kv.num_kv_heads, dim=1)
            eq = "bhsd,bhd->bhs" if tensor_layout == "HND" else "bshd,bhd->bhs"
            lse += torch.einsum(eq, q.float(), km) * sm_scale
    return (o, lse) if return_lse else o
