"""Loading of the native code: the ``torch.ops.sageattention`` operators (``_C.so``) and, for
tests and tools that want the raw entry points, the C ABI (``libsage_b200.so``) through ctypes.

There is no fallback of any kind: if the shared objects are missing or do not load, every entry
point raises.  Build them with ``python -m sageattention_rdna3_b200.build`` (nvcc, no GPU needed).
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Optional

import torch

PKG_DIR = Path(__file__).resolve().parent
ABI_PATH = PKG_DIR / "libsage_b200.so"
OPS_PATH = PKG_DIR / "_C.so"

_ops = None
_abi = None
_import_error: Optional[BaseException] = None

SAGE_DTYPE_F16 = 0
SAGE_DTYPE_BF16 = 1


class SageStrided(ctypes.Structure):
    """``sage_strided_t`` of include/sage_b200.h."""
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64),
                ("stride_s", ctypes.c_int64)]


def _missing(what: str, err: Optional[BaseException] = None) -> RuntimeError:
    return RuntimeError(
        f"sageattention_rdna3_b200: the native extension ({what}) is not available; there is no "
        "CPU or PyTorch fallback. Build it in-tree with\n    python -m sageattention_rdna3_b200.build\n"
        "(needs nvcc with sm_100a support; the kernels run on NVIDIA B200 only)."
        + (f"\nOriginal error: {err!r}" if err is not None else ""))


def load_abi() -> ctypes.CDLL:
    """The C ABI as a ctypes library with argument types set."""
    global _abi
    if _abi is not None:
        return _abi
    if not ABI_PATH.exists():
        raise _missing(ABI_PATH.name)
    try:
        lib = ctypes.CDLL(str(ABI_PATH), mode=ctypes.RTLD_GLOBAL)
    except OSError as e:  # pragma: no cover - depends on the machine
        raise _missing(ABI_PATH.name, e) from e
    vp, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    sp = ctypes.POINTER(SageStrided)
    lib.sage_abi_version.restype = i
    lib.sage_abi_version.argtypes = []
    lib.sage_last_error.restype = ctypes.c_char_p
    lib.sage_last_error.argtypes = []
    lib.sage_test_set_wait_limit_us.restype = i
    lib.sage_test_set_wait_limit_us.argtypes = [ctypes.c_longlong]
    lib.sage_set_status_mirror.restype = i
    lib.sage_set_status_mirror.argtypes = [vp]
    lib.sage_set_streamk.restype = i
    lib.sage_set_streamk.argtypes = [i]
    lib.sage_test_drop_v_load.restype = i
    lib.sage_test_drop_v_load.argtypes = [i]
    lib.sage_mean_seq.restype = i
    lib.sage_mean_seq.argtypes = [sp, i, i, i, i, i, vp, vp]
    lib.sage_quant_qk_int8.restype = i
    lib.sage_quant_qk_int8.argtypes = [sp, sp, vp, sp, vp, i, i, i, i, i, i, i, f, vp, vp, vp, vp, vp]
    lib.sage_fold_attn_partial.restype = i
    lib.sage_fold_attn_partial.argtypes = [sp, vp, i64, i64, sp, i, vp, i, i, i, i, i, vp]
    lib.sage_prep_smooth_preferred.restype = i
    lib.sage_prep_smooth_preferred.argtypes = [i, i]
    lib.sage_prep_smooth_qkv.restype = i
    lib.sage_prep_smooth_qkv.argtypes = [sp, sp, sp, vp, i, i, i, i, i, i, i, f, vp, vp, vp, vp, vp, vp]
    lib.sage_quant_qk_int8_smooth_static.restype = i
    lib.sage_quant_qk_int8_smooth_static.argtypes = [sp, sp, i, i, i, i, i, i, i, f, vp, vp, vp, vp, vp]
    lib.sage_v_to_f16.restype = i
    lib.sage_v_to_f16.argtypes = [sp, i, i, i, i, i, vp, vp]
    lib.sage_qk_int8_sv_f16_attn.restype = i
    lib.sage_qk_int8_sv_f16_attn.argtypes = [vp, vp, sp, vp, i64, i64, i64, vp, vp, i, i, i, i, i, i, i, i, vp, vp, vp]
    lib.sage_qk_int8_sv_f16_attn_lse.restype = i
    lib.sage_qk_int8_sv_f16_attn_lse.argtypes = [vp, vp, sp, vp, i64, i64, i64, vp, vp, i, i, i, i, i, i, i, i, vp, vp,
                                                 vp, vp]
    lib.sage_attn_workspace_bytes.restype = i64
    lib.sage_attn_workspace_bytes.argtypes = [i, i, i, i, i, i]
    lib.sage_qk_int8_sv_f16_attn_ws.restype = i
    lib.sage_qk_int8_sv_f16_attn_ws.argtypes = [vp, vp, sp, vp, i64, i64, i64, vp, vp, i, i, i, i, i, i, i, i, vp, vp,
                                                vp, vp, i64, vp]
    lib.sage_qk_int8_sv_f16_attn_scatter.restype = i
    lib.sage_qk_int8_sv_f16_attn_scatter.argtypes = [vp, vp, sp, vp, i64, i64, i64, vp, vp, i, i, i, i, i, i, i, i, vp,
                                                     vp, i, ctypes.POINTER(vp), vp]
    lib.sage_direct_attn_scatter.restype = i
    lib.sage_direct_attn_scatter.argtypes = [sp, sp, sp, vp, i64, i64, i64, i, i, i, i, i, i, i, i, ctypes.c_float, vp, vp,
                                             i, ctypes.POINTER(vp), vp]
    lib.sage_peer_export.restype = i
    lib.sage_peer_export.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(i64)]
    lib.sage_peer_open.restype = i
    lib.sage_peer_open.argtypes = [ctypes.c_char_p, i64, ctypes.POINTER(vp)]
    lib.sage_peer_close.restype = i
    lib.sage_peer_close.argtypes = [vp, i64]
    lib.sage_direct_attn_ws.restype = i
    lib.sage_direct_attn_ws.argtypes = [sp, sp, sp, vp, i64, i64, i64, i, i, i, i, i, i, i, i, ctypes.c_float, vp, vp,
                                        vp, i64, vp]
    lib.sage_direct_attn.restype = i
    lib.sage_direct_attn.argtypes = [sp, sp, sp, vp, i64, i64, i64, i, i, i, i, i, i, i, i, ctypes.c_float, vp, vp, vp]
    _abi = lib
    return lib


def load_ops():
    """``torch.ops.sageattention`` with the B200 operators registered."""
    global _ops, _import_error
    if _ops is not None:
        return _ops
    if not OPS_PATH.exists() or not ABI_PATH.exists():
        raise _missing(f"{OPS_PATH.name} / {ABI_PATH.name}")
    try:
        load_abi()                       # resolve libsage_b200.so first (also found through $ORIGIN)
        torch.ops.load_library(str(OPS_PATH))
    except Exception as e:  # pragma: no cover - depends on the machine
        _import_error = e
        raise _missing(OPS_PATH.name, e) from e
    _ops = torch.ops.sageattention
    return _ops


def native_available() -> bool:
    try:
        load_ops()
        return True
    except RuntimeError:
        return False
