"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares, and
rejects bad arguments before touching CUDA (no compute call is made here)."""
import ctypes
import os
import re

import pytest
import torch

from sageattention_rdna3_b200 import _native
from sageattention_rdna3_b200._native import SageStrided

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sage_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sage_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    assert declared_symbols() == sorted(["sage_abi_version", "sage_last_error", "sage_mean_seq",
                                         "sage_quant_qk_int8", "sage_v_to_f16", "sage_qk_int8_sv_f16_attn",
                                         "sage_qk_int8_sv_f16_attn_lse", "sage_direct_attn", "sage_attn_workspace_bytes",
                                         "sage_qk_int8_sv_f16_attn_ws", "sage_direct_attn_ws",
                                         "sage_quant_qk_int8_smooth_static", "sage_test_set_wait_limit_us",
                                         "sage_test_drop_v_load", "sage_set_streamk", "sage_prep_smooth_qkv", "sage_prep_smooth_preferred", "sage_fold_attn_partial", "sage_set_status_mirror",
                                         "sage_qk_int8_sv_f16_attn_scatter", "sage_direct_attn_scatter", "sage_peer_export", "sage_peer_open",
                                         "sage_peer_close"])


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_native.ABI_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/sage_b200.h but not exported"


def test_abi_version_matches_header():
    lib = _native.load_abi()
    want = int(re.search(r"#define SAGE_ABI_VERSION (\d+)", open(HEADER).read()).group(1))
    assert lib.sage_abi_version() == want


def test_torch_ops_are_registered():
    ops = _native.load_ops()
    for name in ("mean_seq", "quant_qk_int8", "prep_qkv", "v_to_f16", "qk_int8_sv_f16_attn"):
        assert hasattr(ops, name)
    schema = str(torch.ops.sageattention.quant_qk_int8.default._schema)
    assert "Tensor query, Tensor key, Tensor key_mean, int tensor_layout, float sm_scale" in schema


def _fake(ptr=0x1000, sb=64 * 16 * 2, sh=64 * 16, ss=64):
    return SageStrided(ptr, sb, sh, ss)


def test_invalid_arguments_are_rejected_without_cuda():
    lib = _native.load_abi()
    k = _fake()
    out = ctypes.c_void_p(0x2000)
    # head_dim 96
    assert lib.sage_mean_seq(ctypes.byref(k), 0, 1, 2, 16, 96, out, None) == 1
    assert b"head_dim" in lib.sage_last_error()
    # dtype code 7
    assert lib.sage_mean_seq(ctypes.byref(k), 7, 1, 2, 16, 64, out, None) == 1
    # null output
    assert lib.sage_mean_seq(ctypes.byref(k), 0, 1, 2, 16, 64, None, None) == 1
    # misaligned base pointer, stride not a multiple of 8
    bad = _fake(ptr=0x1008)
    assert lib.sage_mean_seq(ctypes.byref(bad), 0, 1, 2, 16, 64, out, None) == 1
    bad = _fake(ss=68)
    assert lib.sage_mean_seq(ctypes.byref(bad), 0, 1, 2, 16, 64, out, None) == 1
    assert b"16-byte" in lib.sage_last_error()
    # attention: Hq not a multiple of Hkv
    v = _fake()
    rc = lib.sage_qk_int8_sv_f16_attn(0x1000, 0x1000, ctypes.byref(v), 0x3000, 1024, 512, 64, 0x4000, 0x5000, 0,
                                      1, 3, 2, 16, 16, 64, 0, None, None, None)
    assert rc == 1 and b"multiple" in lib.sage_last_error()
    # quant: missing outputs
    rc = lib.sage_quant_qk_int8(ctypes.byref(k), ctypes.byref(k), None, None, None, 0, 1, 2, 2, 16, 16, 64,
                                ctypes.c_float(0.125), None, None, None, None, None)
    assert rc == 1
    # scatter: too many peers, a null peer list, a misaligned peer, a peer that is the output itself
    args = (0x1000, 0x1000, ctypes.byref(v), 0x3000, 1024, 512, 64, 0x4000, 0x5000, 0, 1, 2, 2, 16, 16, 64, 0, None, None)
    assert lib.sage_qk_int8_sv_f16_attn_scatter(*args, 16, None, None) == 1 and b"n_peers" in lib.sage_last_error()
    assert lib.sage_qk_int8_sv_f16_attn_scatter(*args, 1, None, None) == 1
    for bad_peer in (0x7008, 0x3000, 0):
        peers = (ctypes.c_void_p * 1)(bad_peer)
        assert lib.sage_qk_int8_sv_f16_attn_scatter(*args, 1, peers, None) == 1, hex(bad_peer)
        assert b"peer buffer 0" in lib.sage_last_error()
    # peer mapping: null arguments
    off = ctypes.c_int64(0)
    assert lib.sage_peer_export(None, ctypes.create_string_buffer(64), ctypes.byref(off)) == 1
    assert lib.sage_peer_open(None, 0, ctypes.byref(ctypes.c_void_p(0))) == 1
    assert lib.sage_peer_open(bytes(64), -16, ctypes.byref(ctypes.c_void_p(0))) == 1
    assert lib.sage_peer_close(None, 0) == 1


def test_graft_entry_build_runs():
    """The build entry point compiles (or finds up to date) both libraries and checks them."""
    import __graft_entry__
    __graft_entry__.build()
