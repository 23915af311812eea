"""Shared test helpers: seeded inputs, and thin ctypes callers of the C ABI (include/sage_b200.h)
that take torch CUDA tensors.  The GPU parity tests go through these, i.e. through the same
exported symbols a foreign-language binding would use."""
from __future__ import annotations

import ctypes

import torch

from sageattention_rdna3_b200 import _native
from sageattention_rdna3_b200._native import SageStrided

LAYOUT = {"NHD": 0, "HND": 1}


def randn(shape, seed, dtype, device="cpu", scale=1.0, offset=0.0):
    """N(0,1) from a CPU generator (same bits on every machine), then cast and moved."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32) * scale + offset
    return x.to(dtype).to(device)


def dims(t, layout):
    return (t.size(0), t.size(1), t.size(2), t.size(3)) if layout == "HND" else (t.size(0), t.size(2), t.size(1), t.size(3))


def strided(t, layout):
    if layout == "HND":
        return SageStrided(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    return SageStrided(t.data_ptr(), t.stride(0), t.stride(2), t.stride(1))


def dtype_code(t):
    return {torch.float16: 0, torch.bfloat16: 1}[t.dtype]


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: rc={rc}: {_native.load_abi().sage_last_error().decode()}")


def abi_mean_seq(k, layout):
    lib = _native.load_abi()
    B, H, S, D = dims(k, layout)
    out = torch.empty(B, H, D, dtype=k.dtype, device=k.device)
    ks = strided(k, layout)
    _check(lib.sage_mean_seq(ctypes.byref(ks), dtype_code(k), B, H, S, D, out.data_ptr(), _stream()), "sage_mean_seq")
    return out


def abi_quant(q, k, k_mean, layout, sm_scale, v=None):
    lib = _native.load_abi()
    B, Hq, Sq, D = dims(q, layout)
    _, Hkv, Skv, _ = dims(k, layout)
    dev = q.device
    q_i8 = torch.empty(B, Hq, Sq, D, dtype=torch.int8, device=dev)
    k_i8 = torch.empty(B, Hkv, Skv, D, dtype=torch.int8, device=dev)
    q_scale = torch.empty(B, Hq, (Sq + 31) // 32, dtype=torch.float32, device=dev)
    k_scale = torch.empty(B, Hkv, (Skv + 15) // 16, dtype=torch.float32, device=dev)
    qs, ks = strided(q, layout), strided(k, layout)
    v16, vs_ref, v16_ptr = None, None, None
    if v is not None:
        v16 = torch.empty(B, Hkv, Skv, D, dtype=torch.float16, device=dev)
        vs = strided(v, layout)
        vs_ref, v16_ptr = ctypes.byref(vs), v16.data_ptr()
    mean_ptr = k_mean.data_ptr() if (k_mean is not None and k_mean.numel() > 0) else None
    _check(lib.sage_quant_qk_int8(ctypes.byref(qs), ctypes.byref(ks), mean_ptr, vs_ref, v16_ptr, dtype_code(q),
                                  B, Hq, Hkv, Sq, Skv, D, float(sm_scale), q_i8.data_ptr(), q_scale.data_ptr(),
                                  k_i8.data_ptr(), k_scale.data_ptr(), _stream()), "sage_quant_qk_int8")
    return q_i8, q_scale, k_i8, k_scale, v16


def abi_prep_smooth(q, k, layout, sm_scale, v=None):
    """sage_prep_smooth_qkv: (q_i8, q_scale, k_i8, k_scale, k_mean, v16 or None)."""
    lib = _native.load_abi()
    B, Hq, Sq, D = dims(q, layout)
    _, Hkv, Skv, _ = dims(k, layout)
    dev = q.device
    q_i8 = torch.empty(B, Hq, Sq, D, dtype=torch.int8, device=dev)
    k_i8 = torch.empty(B, Hkv, Skv, D, dtype=torch.int8, device=dev)
    q_scale = torch.empty(B, Hq, (Sq + 31) // 32, dtype=torch.float32, device=dev)
    k_scale = torch.empty(B, Hkv, (Skv + 15) // 16, dtype=torch.float32, device=dev)
    k_mean = torch.empty(B, Hkv, D, dtype=k.dtype, device=dev)
    qs, ks = strided(q, layout), strided(k, layout)
    v16, vs_ref, v16_ptr = None, None, None
    if v is not None:
        v16 = torch.empty(B, Hkv, Skv, D, dtype=torch.float16, device=dev)
        vs = strided(v, layout)
        vs_ref, v16_ptr = ctypes.byref(vs), v16.data_ptr()
    _check(lib.sage_prep_smooth_qkv(ctypes.byref(qs), ctypes.byref(ks), vs_ref, v16_ptr, dtype_code(q), B, Hq, Hkv, Sq,
                                    Skv, D, float(sm_scale), q_i8.data_ptr(), q_scale.data_ptr(), k_i8.data_ptr(),
                                    k_scale.data_ptr(), k_mean.data_ptr(), _stream()), "sage_prep_smooth_qkv")
    return q_i8, q_scale, k_i8, k_scale, k_mean, v16


def abi_v_to_f16(v, layout):
    lib = _native.load_abi()
    B, H, S, D = dims(v, layout)
    out = torch.empty(B, H, S, D, dtype=torch.float16, device=v.device)
    vs = strided(v, layout)
    _check(lib.sage_v_to_f16(ctypes.byref(vs), dtype_code(v), B, H, S, D, out.data_ptr(), _stream()), "sage_v_to_f16")
    return out


def abi_attn(q_i8, k_i8, v16, v_layout, q_scale, k_scale, out_dtype, out_layout, is_causal, dump=False):
    """Returns (o, s_dump or None, status int). ``o`` is allocated in ``out_layout``."""
    lib = _native.load_abi()
    B, Hq, Sq, D = q_i8.shape
    Hkv, Skv = k_i8.shape[1], k_i8.shape[2]
    dev = q_i8.device
    shape = (B, Hq, Sq, D) if out_layout == "HND" else (B, Sq, Hq, D)
    o = torch.full(shape, float("nan"), dtype=out_dtype, device=dev)
    os_ = strided(o, out_layout)
    vs = strided(v16, v_layout)
    s_dump = torch.full((B, Hq, Sq, Skv), -(2 ** 31), dtype=torch.int32, device=dev) if dump else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(lib.sage_qk_int8_sv_f16_attn(q_i8.data_ptr(), k_i8.data_ptr(), ctypes.byref(vs), o.data_ptr(),
                                        os_.stride_b, os_.stride_h, os_.stride_s, q_scale.data_ptr(),
                                        k_scale.data_ptr(), dtype_code(o), B, Hq, Hkv, Sq, Skv, D, int(is_causal),
                                        s_dump.data_ptr() if dump else None, status.data_ptr(), _stream()),
           "sage_qk_int8_sv_f16_attn")
    torch.cuda.synchronize()
    return o, s_dump, int(status.item())


def set_streamk(mode):
    """Launch schedule of the attention kernels: -1 cost model, 0 plain, 1 persistent (sage_set_streamk)."""
    assert _native.load_abi().sage_set_streamk(int(mode)) == 0
