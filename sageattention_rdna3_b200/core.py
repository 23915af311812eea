"""``sageattn`` for NVIDIA B200: the Python entry point of LuXuxue/sageattention-rdna3
(``sageattention/core.py:40-233``) in front of hand-written sm_100a kernels.

Same call, same defaults, same assertions as the reference.  What is gone: the Triton default and
the ``SAGEATTN_BACKEND`` switch (``core.py:8,68-76``) and the transposed V scratch
(``core.py:173-180``).  A call runs either the INT8 path - [K mean] -> quantise Q/K (+ fp16 copy of a
bf16 V) -> fused attention - or, for the short sequences the reference sends there
(``core.py:113-163``), the un-quantised kernel.  There is no CPU or PyTorch fallback; without the
compiled extension the call raises.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional, Tuple, Union

import torch

from . import _native

_BACKEND = "native"          # the reference's scripts read this name (core.py:8)
_LAYOUT_CODE = {"NHD": 0, "HND": 1}   # csrc/attn_gfx11.cu:32-33

_status_words: Dict[int, torch.Tensor] = {}
_status_mirrors: Dict[int, tuple] = {}
_STATUS_MESSAGE = ("sageattn: the attention kernel reported device status {code} "
                   "(1 = shared memory misaligned, 2+16*k = bounded wait k timed out)")


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that the attention kernel sets if it had to give up on a wait."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(idx)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = word
    return word


def _status_mirror(device: torch.device):
    """A word in pinned host memory that a failing attention kernel of the device writes its code to
    as well (tensor, numpy view; registered with ``sage_set_status_mirror``).  Every ``sageattn``
    call looks at it before it launches: a kernel that gave up is reported by the next call on that
    device, without any synchronisation and at no cost to calls that succeed.
    ``SAGEATTN_B200_STATUS_MIRROR=0`` switches it off."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    pair = _status_mirrors.get(idx)
    if pair is None:
        host = torch.zeros(1, dtype=torch.int32).pin_memory()
        pair = (host, host.numpy())
        _status_mirrors[idx] = pair
        with torch.cuda.device(idx):
            rc = _native.load_abi().sage_set_status_mirror(host.data_ptr())
        if rc != 0:
            raise RuntimeError("sage_set_status_mirror failed: " + _native.load_abi().sage_last_error().decode())
    return pair


_MIRROR_ON = os.environ.get("SAGEATTN_B200_STATUS_MIRROR", "1") != "0"


def check_status(device: Union[torch.device, int, str, None] = None) -> None:
    """Synchronise and raise if a kernel on ``device`` reported an internal error since the last check."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    elif isinstance(device, int):
        device = torch.device("cuda", device)
    elif isinstance(device, str):
        device = torch.device(device)
    word = _status_word(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        if _MIRROR_ON:
            _status_mirror(device)[1][0] = 0
        raise RuntimeError(_STATUS_MESSAGE.format(code=code))


def _aligned(t: torch.Tensor) -> bool:
    s0, s1, s2, _ = t.stride()
    return (s0 | s1 | s2) % 8 == 0 and t.data_ptr() % 16 == 0


# Largest kv length that goes to the un-quantised kernel, per case of the reference's dispatch
# (sageattention/core.py:113-139); the same environment variables override them.  The values are the
# reference's: on a B200 the un-quantised kernel is at least as fast as the INT8 path everywhere
# below them (head_dim 64: faster at every length measured, the exponential unit and not the tensor
# pipe limits both kernels there; head_dim 128: level at kv = 2048, INT8 ahead by 1.2x at 8192), so
# every call takes the branch the reference takes for its shape.
_DIRECT_DEFAULTS = {
    "SAGEATTN_DIRECT_THRESHOLD_D64": {"HND": 2048, "NHD": 3072},
    "SAGEATTN_DIRECT_THRESHOLD_D64_CAUSAL": 6144,
    "SAGEATTN_DIRECT_THRESHOLD_D64_CROSS": 6144,
    "SAGEATTN_DIRECT_THRESHOLD_D128": 2048,
    "SAGEATTN_DIRECT_THRESHOLD_D128_CROSS": 4096,
}


def _threshold(name: str, tensor_layout: str = "HND") -> int:
    default = _DIRECT_DEFAULTS[name]
    if isinstance(default, dict):
        default = default[tensor_layout]
    return int(os.environ.get(name, str(default)) or default)


def use_direct_kernel(headdim: int, tensor_layout: str, is_causal: bool, q_len: int, kv_len: int) -> bool:
    """The reference's choice between the un-quantised and the INT8 kernels
    (``sageattention/core.py:113-139``): by head_dim, causal / cross / self attention and kv length.
    ``SAGEATTN_KERNEL=int8`` or ``=direct`` in the environment overrides it for every call."""
    forced = os.environ.get("SAGEATTN_KERNEL", "")
    if forced:
        assert forced in ("int8", "direct"), f"SAGEATTN_KERNEL must be 'int8' or 'direct', got {forced!r}."
        return forced == "direct"
    if headdim == 64:
        if is_causal:
            return kv_len <= _threshold("SAGEATTN_DIRECT_THRESHOLD_D64_CAUSAL")
        if q_len < kv_len:
            return kv_len <= _threshold("SAGEATTN_DIRECT_THRESHOLD_D64_CROSS")
        return kv_len <= _threshold("SAGEATTN_DIRECT_THRESHOLD_D64", tensor_layout)
    if q_len * 2 < kv_len:
        return kv_len <= _threshold("SAGEATTN_DIRECT_THRESHOLD_D128_CROSS")
    return kv_len <= _threshold("SAGEATTN_DIRECT_THRESHOLD_D128")


def sageattn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    tensor_layout: str = "HND",
    is_causal: bool = False,
    sm_scale: Optional[float] = None,
    return_lse: bool = False,
    smooth_k: bool = False,
    **kwargs: Any,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """INT8-QK / FP16-PV attention.  Signature and checks of ``sageattention/core.py:40-63``.

    q: ``[B,Hq,Sq,D]`` ("HND") or ``[B,Sq,Hq,D]`` ("NHD"); k, v likewise with Hkv, Skv
    (Hq a multiple of Hkv).  D in {64, 128}; fp16 / bf16, or fp32 which is computed in fp16 and
    returned in fp32 (``core.py:78-83,200-201``).  ``smooth_k`` subtracts the per-channel mean of K
    before quantisation (``core.py:186-190``; default False as in the native path).  Unknown keyword
    arguments are ignored, as in the reference.

    Short sequences go to the un-quantised kernel (fp16 / bf16 Q.K^T, no quantisation launches), as
    in the reference (``core.py:113-163``), below the kv lengths of ``_DIRECT_DEFAULTS``;
    ``kernel="int8"`` or ``kernel="direct"`` (keyword, or ``SAGEATTN_KERNEL`` in the environment)
    forces one of the two.  ``smooth_k`` only
    applies to the INT8 kernel, as in the reference.

    ``return_lse=True`` also returns ``lse`` ``[B,Hq,Sq]`` fp32, the natural-log sum of
    ``exp(sm_scale * q.k)`` over the visible keys of each row, as computed by the kernel from the
    quantised scores (with ``smooth_k`` the kernel works on centred keys and ``sm_scale * q.mean(k)``
    is added back, so the value refers to the caller's keys).  The reference returns zeros there as
    a placeholder (``core.py:203-211``); ``SAGEATTN_B200_LSE_ZEROS=1`` restores that.

    Errors on the device.  Every wait inside the kernels is bounded; a kernel that has to give up
    writes a code to a per-device status word and returns, leaving the output partly unwritten.  The
    call itself never synchronises, so it cannot raise for its own launch: the failure is raised by
    the NEXT ``sageattn`` call on that device (a failing kernel also writes its code to a word in
    pinned host memory), by ``check_status()`` (synchronises), or at once with
    ``SAGEATTN_B200_CHECK_STATUS=1`` (synchronises every call).  The reference has no such state.

    Two keywords beyond the reference's, used by the multi-GPU paths: ``out`` (a tensor with the
    shape, dtype and device of ``q``; fp16 / bf16 inputs only) receives the result instead of a new
    tensor, and ``scatter_to`` (device addresses of further copies of ``out``, normally in other
    GPUs' memory, see :mod:`.peer_gather`) makes the kernel write them as well.
    """
    dtype = q.dtype
    assert q.is_cuda, "Input tensors must be on CUDA/HIP device."
    assert dtype in [torch.float16, torch.bfloat16, torch.float32], (
        "Input tensors must be fp16, bf16, or fp32."
    )
    assert q.device == k.device == v.device, "All tensors must be on the same device."
    assert q.dtype == k.dtype == v.dtype, "All tensors must have the same dtype."
    assert tensor_layout in _LAYOUT_CODE, f"tensor_layout must be 'HND' or 'NHD', got {tensor_layout!r}."
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must be 4-D tensors."

    q_shape, k_shape, q_stride = q.shape, k.shape, q.stride()    # read once: each call costs ~0.3 us
    headdim = q_shape[3]
    assert headdim in [64, 128], f"head_dim must be 64 or 128, got {headdim}."
    assert q_stride[3] == 1 and k.stride(3) == 1 and v.stride(3) == 1, (
        "Last dim of qkv must be contiguous."
    )
    if sm_scale is None:
        sm_scale = headdim ** -0.5

    input_dtype = dtype
    if dtype == torch.float32:
        q, k, v = q.to(torch.float16), k.to(torch.float16), v.to(torch.float16)
        dtype = torch.float16
        q_stride = q.stride()

    # core.py:91-95: the output inherits q's strides and is written with 16-byte vector stores.
    assert q_stride[0] % 8 == 0 and q_stride[1] % 8 == 0 and q_stride[2] % 8 == 0, (
        "native backend requires q strides that are multiples of 8 halfs "
        "(16B aligned write-back). "
        f"Got strides={q.stride()}. Use contiguous tensors."
    )
    ops = _native.load_ops()
    layout = _LAYOUT_CODE[tensor_layout]
    seq_dim, head_dim_idx = (2, 1) if tensor_layout == "HND" else (1, 2)
    q_len, kv_len = q_shape[seq_dim], k_shape[seq_dim]
    assert k_shape == v.shape, "k and v must have the same shape."
    assert q_shape[0] == k_shape[0] and q_shape[head_dim_idx] % max(k_shape[head_dim_idx], 1) == 0, (
        "batch sizes must match and num_qo_heads must be a multiple of num_kv_heads."
    )
    # 16-byte vector loads and TMA need aligned bases and strides; the reference leaves that to
    # the caller for k and v, here a misaligned view is copied once.
    if q.data_ptr() % 16 != 0:
        q = q.clone(memory_format=torch.contiguous_format)
    if not _aligned(k):
        k = k.contiguous()
    if not _aligned(v):
        v = v.contiguous()

    o = None
    lse = None
    out_arg, scatter_to = kwargs.get("out"), kwargs.get("scatter_to")
    if out_arg is not None:
        assert input_dtype != torch.float32, "out= is for fp16 / bf16 inputs."
        assert out_arg.shape == q.shape and out_arg.dtype == q.dtype and out_arg.device == q.device, (
            "out must have the shape, dtype and device of q."
        )
    assert not scatter_to or out_arg is not None, "scatter_to needs out=."
    want_lse = return_lse and os.environ.get("SAGEATTN_B200_LSE_ZEROS", "0") != "1"
    if return_lse:
        lse_shape = (q_shape[0], q_shape[head_dim_idx], q_len)
        if want_lse:
            lse = torch.full(lse_shape, float("-inf"), dtype=torch.float32, device=q.device)
        else:
            lse = torch.zeros(lse_shape, dtype=torch.float32, device=q.device)
    if q_len == 0 or q_shape[0] == 0 or q_shape[head_dim_idx] == 0:
        o = torch.empty_like(q) if out_arg is None else out_arg
    elif kv_len == 0:
        # l == 0 for every row -> 0 (csrc/attn_gfx11.cu:771)
        assert not scatter_to, "scatter_to needs at least one key."
        o = torch.zeros_like(q) if out_arg is None else out_arg.zero_()
    else:
        # core.py:141-198 in one operator call: the un-quantised branch (V as fp16, fp16_attn / bf16_attn)
        # or the INT8 branch ([K mean,] quantise Q / K and convert a bf16 V in one launch, attention).
        direct = _pick_direct(kwargs.get("kernel"), headdim, tensor_layout, is_causal, q_len, kv_len)
        smooth = bool(smooth_k) and not direct          # the un-quantised branch has no use for the mean
        if _MIRROR_ON:
            _, seen = _status_mirror(q.device)
            if seen[0] != 0:                            # an earlier call on this device gave up
                code = int(seen[0])
                seen[0] = 0
                _status_word(q.device).zero_()
                raise RuntimeError(_STATUS_MESSAGE.format(code=code) + "; reported by the call after the one that failed")
        out = ops.sageattn_fwd(q, k, v, layout, int(is_causal), sm_scale, int(smooth), int(direct),
                               _status_word(q.device), lse if want_lse else None, out_arg,
                               [int(a) for a in scatter_to] if scatter_to else None)
        o = out[0]
        if want_lse and smooth:
            # the kernel saw k - mean: every score of a row was lowered by sm_scale * q.mean
            rep = q_shape[head_dim_idx] // k_shape[head_dim_idx]
            km = out[1].float().repeat_interleave(rep, dim=1)                   # [B,Hq,D]
            eq = "bhsd,bhd->bhs" if tensor_layout == "HND" else "bshd,bhd->bhs"
            lse += torch.einsum(eq, q.float(), km) * sm_scale
        if os.environ.get("SAGEATTN_B200_CHECK_STATUS", "0") == "1":
            check_status(q.device)

    if input_dtype == torch.float32:
        o = o.to(torch.float32)

    if return_lse:
        return o, lse
    return o


def _pick_direct(forced: Optional[str], headdim: int, tensor_layout: str, is_causal: bool, q_len: int,
                 kv_len: int) -> bool:
    if forced is not None:
        assert forced in ("int8", "direct"), f"kernel must be 'int8' or 'direct', got {forced!r}."
        return forced == "direct"
    return use_direct_kernel(headdim, tensor_layout, is_causal, q_len, kv_len)


def sageattn_qk_int8_pv_fp16_cuda(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    tensor_layout: str = "HND",
    is_causal: bool = False,
    sm_scale: Optional[float] = None,
    return_lse: bool = False,
    **kwargs: Any,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Alias kept for callers of upstream SageAttention (``sageattention/core.py:216-233``)."""
    return sageattn(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale,
                    return_lse=return_lse, **kwargs)
