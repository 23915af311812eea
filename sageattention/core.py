"""``sageattention.core`` of the drop-in: the names the reference's scripts and tests read from
``sageattention/core.py`` (``:8-17`` module flags, ``:40`` ``sageattn``, ``:216`` the alias).

``GFX11_NATIVE_ENABLED`` is true when the compiled B200 libraries are present (the reference sets
it when its ``_qattn_gfx11`` extension imports, ``core.py:11-17``; its test file skips every case
when it is false, ``test_sageattn_rdna3.py:64-77``).  ``_BACKEND`` is always "native": the Triton
back-end and the ``SAGEATTN_BACKEND`` switch do not exist here.
"""
from sageattention_rdna3_b200 import _native
from sageattention_rdna3_b200.core import (_BACKEND, check_status, sageattn, sageattn_qk_int8_pv_fp16_cuda,
                                           use_direct_kernel)

GFX11_NATIVE_ENABLED = _native.ABI_PATH.exists() and _native.OPS_PATH.exists()
_import_error = None if GFX11_NATIVE_ENABLED else _native._missing("libsage_b200.so / _C.so")


def _get_native_ops():
    """``torch.ops.sageattention`` with the B200 operators registered (``core.py:22-37``); raises
    when the libraries are not built."""
    return _native.load_ops()


__all__ = ["sageattn", "sageattn_qk_int8_pv_fp16_cuda", "GFX11_NATIVE_ENABLED", "_BACKEND", "check_status",
           "use_direct_kernel"]
