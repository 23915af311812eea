"""The allocation-free smooth-K quantisation entry point (sage_quant_qk_int8_smooth_static).

Some hosts cannot allocate device memory at call time (everything was sized at start-up, or the
host's allocator is not theirs to use, or cudaMalloc's device-wide synchronisation is unaffordable).
For them the library keeps the one intermediate of smooth-K quantisation, the mean of K, in a
fixed buffer of its own.  The results must be the ones the allocating entry points give, bit for
bit, call after call: the buffer is shared and keeps stale contents between calls.

This file sorts last on purpose: a run that stops at the first failure has already run every
other test.  It passes both on its own in a fresh process and after the rest of the suite.
"""
import ctypes

import pytest
import torch

import helpers as H
from sageattention_rdna3_b200 import _native

MAX_ELEMS = 65536      # SAGE_STATIC_KMEAN_MAX_ELEMS in include/sage_b200.h


def _static_quant(q, k, layout, sm_scale):
    lib = _native.load_abi()
    B, Hq, Sq, D = H.dims(q, layout)
    _, Hkv, Skv, _ = H.dims(k, layout)
    dev = q.device
    q_i8 = torch.empty(B, Hq, Sq, D, dtype=torch.int8, device=dev)
    k_i8 = torch.empty(B, Hkv, Skv, D, dtype=torch.int8, device=dev)
    q_scale = torch.empty(B, Hq, (Sq + 31) // 32, dtype=torch.float32, device=dev)
    k_scale = torch.empty(B, Hkv, (Skv + 15) // 16, dtype=torch.float32, device=dev)
    qs, ks = H.strided(q, layout), H.strided(k, layout)
    rc = lib.sage_quant_qk_int8_smooth_static(ctypes.byref(qs), ctypes.byref(ks), H.dtype_code(q), B, Hq, Hkv, Sq,
                                              Skv, D, float(sm_scale), q_i8.data_ptr(), q_scale.data_ptr(),
                                              k_i8.data_ptr(), k_scale.data_ptr(),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.sage_last_error().decode()
    return q_i8, q_scale, k_i8, k_scale


@pytest.mark.gpu
@pytest.mark.parametrize("index", [0, 1])
def test_static_entry_point_matches_allocating_path_twice_in_a_row(index):
    if index >= torch.cuda.device_count():
        pytest.skip("the buffer's address is looked up per device: the second device needs a second GPU")
    dev = torch.device("cuda", index)
    torch.cuda.set_device(dev)
    calls = [
        # B, Hq, Hkv, Sq, Skv, D, dtype, layout, K offset
        (2, 8, 4, 700, 700, 128, torch.bfloat16, "HND", 3.0),     # fills 1024 elements of the buffer
        (1, 2, 2, 333, 1000, 64, torch.float16, "NHD", -1.5),     # smaller, other dtype: stale bytes remain behind it
    ]
    for n, (B, Hq, Hkv, Sq, Skv, D, dtype, layout, off) in enumerate(calls):
        shp = (lambda h, s: (B, h, s, D)) if layout == "HND" else (lambda h, s: (B, s, h, D))
        q = H.randn(shp(Hq, Sq), 10 + n, dtype).to(dev)
        k = H.randn(shp(Hkv, Skv), 20 + n, dtype, offset=off).to(dev)
        sm = D ** -0.5
        want = H.abi_quant(q, k, H.abi_mean_seq(k, layout), layout, sm)[:4]
        got = _static_quant(q, k, layout, sm)
        torch.cuda.synchronize()
        if n > 0:
            # The property in the name: after the first call on the device (which looks the buffer's
            # address up) a call must leave the device's free memory and torch's allocator untouched.
            # _static_quant allocates the OUTPUTS, so call the entry point once more on the same ones.
            lib = _native.load_abi()
            qs, ks = H.strided(q, layout), H.strided(k, layout)
            free_before, allocated_before = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev)
            rc = lib.sage_quant_qk_int8_smooth_static(
                ctypes.byref(qs), ctypes.byref(ks), H.dtype_code(q), B, Hq, Hkv, Sq, Skv, D, float(sm),
                got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), got[3].data_ptr(),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            assert rc == 0
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call changed the device's free memory"
            assert torch.cuda.memory_allocated(dev) == allocated_before
        for name, a, b in zip(("q_i8", "q_scale", "k_i8", "k_scale"), got, want):
            if a.dtype == torch.float32:
                assert torch.equal(a.view(torch.int32), b.view(torch.int32)), f"call {n}: {name} differs"
            else:
                assert torch.equal(a, b), f"call {n}: {name} differs"


def test_static_entry_point_refuses_what_does_not_fit():
    """The size check comes before any CUDA call, so it can be exercised without a GPU."""
    lib = _native.load_abi()
    fake = H.SageStrided(0x1000, 1 << 20, 1 << 10, 128)
    B, Hkv, D = 8, 128, 128                                   # 131072 elements > 65536
    assert B * Hkv * D > MAX_ELEMS
    rc = lib.sage_quant_qk_int8_smooth_static(ctypes.byref(fake), ctypes.byref(fake), 1, B, Hkv, Hkv, 64, 64, D,
                                              ctypes.c_float(0.1), 0x2000, 0x3000, 0x4000, 0x5000, None)
    assert rc == 1
    msg = lib.sage_last_error().decode()
    assert "exceeds" in msg and str(MAX_ELEMS) in msg
    rc = lib.sage_quant_qk_int8_smooth_static(ctypes.byref(fake), ctypes.byref(fake), 1, 1, 2, 2, 64, 0, D,
                                              ctypes.c_float(0.1), 0x2000, 0x3000, 0x4000, 0x5000, None)
    assert rc == 1
