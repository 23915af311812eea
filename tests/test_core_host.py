"""CPU-side checks of the Python entry point and of the shard planner."""
import inspect

import pytest
import torch

import sageattention
from sageattention_rdna3_b200 import core, sageattn, sageattn_qk_int8_pv_fp16_cuda
from sageattention_rdna3_b200.shard import Shard, from_units, plan_shards, shard_inputs, to_units


def test_drop_in_names_and_signature():
    assert sageattention.sageattn is sageattn
    assert sageattention.__all__ == ["sageattn", "sageattn_qk_int8_pv_fp16_cuda"]
    sig = inspect.signature(sageattn)
    names = list(sig.parameters)
    assert names[:7] == ["q", "k", "v", "tensor_layout", "is_causal", "sm_scale", "return_lse"]
    assert sig.parameters["tensor_layout"].default == "HND"
    assert sig.parameters["is_causal"].default is False
    assert sig.parameters["sm_scale"].default is None
    assert sig.parameters["smooth_k"].default is False
    assert sig.parameters["kwargs"].kind is inspect.Parameter.VAR_KEYWORD
    assert list(inspect.signature(sageattn_qk_int8_pv_fp16_cuda).parameters)[:7] == names[:7]
    assert core._BACKEND == "native"


def test_cpu_tensors_are_refused():
    """No CPU fallback: the reference's first assertion (core.py:51) stands."""
    q = torch.zeros(1, 1, 16, 64, dtype=torch.float16)
    with pytest.raises(AssertionError, match="CUDA"):
        sageattn(q, q, q)


@pytest.mark.parametrize("B,Hq,Hkv,world", [(2, 32, 32, 1), (2, 32, 32, 8), (4, 32, 8, 8), (1, 24, 24, 8),
                                           (1, 24, 24, 5), (1, 2, 2, 4), (3, 6, 3, 2)])
def test_plan_shards_covers_all_units_once(B, Hq, Hkv, world):
    shards = plan_shards(B, Hq, Hkv, world)
    assert len(shards) == world and shards[0].unit_start == 0 and shards[-1].unit_stop == B * Hkv
    for a, b in zip(shards, shards[1:]):
        assert a.unit_stop == b.unit_start
    sizes = [s.n_units for s in shards]
    assert max(sizes) - min(sizes) <= 1 and sum(sizes) == B * Hkv


def test_plan_shards_baseline_configs():
    assert [s.n_units for s in plan_shards(2, 32, 32, 8)] == [8] * 8          # B=2 H=32
    assert [s.n_units for s in plan_shards(4, 32, 8, 8)] == [4] * 8           # B=4 Hq=32 Hkv=8 (4 q heads per unit)
    assert [s.n_units for s in plan_shards(1, 24, 24, 8)] == [3] * 8          # B=1 H=24
    assert [s.n_units for s in plan_shards(1, 24, 24, 4)] == [6] * 4
    with pytest.raises(ValueError):
        plan_shards(1, 6, 4, 2)


@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_units_roundtrip_keeps_gqa_groups_together(layout):
    B, Hq, Hkv, S, D = 2, 6, 3, 5, 8
    q_hnd = torch.arange(B * Hq * S * D, dtype=torch.float32).reshape(B, Hq, S, D)
    k_hnd = torch.arange(B * Hkv * S * D, dtype=torch.float32).reshape(B, Hkv, S, D)
    q = q_hnd if layout == "HND" else q_hnd.permute(0, 2, 1, 3).contiguous()
    k = k_hnd if layout == "HND" else k_hnd.permute(0, 2, 1, 3).contiguous()
    u = to_units(q, layout, Hkv)
    assert u.shape == (B * Hkv, Hq // Hkv, S, D)
    # unit b*Hkv + hkv holds query heads hkv*rep .. hkv*rep+rep-1 of batch b
    assert torch.equal(u[1 * Hkv + 2], q_hnd[1, 4:6])
    assert torch.equal(from_units(u, B, Hq, layout), q)
    ql, kl, vl = shard_inputs(q, k, k, layout, Shard(1, 2, 5))
    assert ql.shape == (3, 2, S, D) and kl.shape == (3, 1, S, D)
    assert torch.equal(kl[:, 0], k_hnd.reshape(B * Hkv, S, D)[2:5])


def test_kernel_dispatch_table_of_the_reference(monkeypatch):
    """``use_direct_kernel`` reproduces ``sageattention/core.py:113-139`` case by case."""
    from sageattention_rdna3_b200.core import use_direct_kernel as ud
    for name in ("SAGEATTN_KERNEL", "SAGEATTN_DIRECT_THRESHOLD_D64", "SAGEATTN_DIRECT_THRESHOLD_D64_CAUSAL",
                 "SAGEATTN_DIRECT_THRESHOLD_D64_CROSS", "SAGEATTN_DIRECT_THRESHOLD_D128",
                 "SAGEATTN_DIRECT_THRESHOLD_D128_CROSS"):
        monkeypatch.delenv(name, raising=False)
    # head_dim 64, self attention: 2048 in HND, 3072 in NHD (core.py:121-124,132)
    assert ud(64, "HND", False, 2048, 2048) and not ud(64, "HND", False, 2049, 2049)
    assert ud(64, "NHD", False, 3072, 3072) and not ud(64, "NHD", False, 3073, 3073)
    # causal: 6144 (core.py:125-126); cross (q shorter than kv): 6144 (core.py:127-129)
    assert ud(64, "HND", True, 6144, 6144) and not ud(64, "HND", True, 6145, 6145)
    assert ud(64, "NHD", False, 3072, 4096) and not ud(64, "NHD", False, 100, 6145)
    # head_dim 128: 2048, and 4096 when q is less than half of kv (core.py:133-139)
    assert ud(128, "HND", False, 2048, 2048) and not ud(128, "HND", True, 2049, 2049)
    assert ud(128, "HND", False, 512, 4096) and not ud(128, "HND", False, 2048, 4096)
    assert not ud(128, "NHD", False, 512, 4097)
    # the five benchmark configurations: the smallest -> un-quantised, the others -> INT8
    assert ud(64, "HND", False, 1024, 1024)
    assert not ud(64, "NHD", False, 4096, 4096) and not ud(128, "HND", True, 8192, 8192)
    assert not ud(128, "HND", True, 4096, 4096) and not ud(128, "NHD", False, 32768, 32768)
    # overrides
    monkeypatch.setenv("SAGEATTN_DIRECT_THRESHOLD_D128", "0")
    assert not ud(128, "HND", False, 64, 64)
    monkeypatch.setenv("SAGEATTN_KERNEL", "direct")
    assert ud(128, "HND", False, 8192, 8192)


def test_direct_emulation_against_fp32_sdpa():
    from oracle import sage_oracle as so
    g = torch.Generator().manual_seed(0)
    for dtype, causal, layout in ((torch.float16, False, "HND"), (torch.bfloat16, True, "NHD")):
        shape = (1, 3, 150, 64) if layout == "HND" else (1, 150, 3, 64)
        q, k, v = (torch.randn(shape, generator=g).to(dtype) for _ in range(3))
        o = so.direct_attn_emulated(q, k, v, tensor_layout=layout, is_causal=causal)
        ref = so.sdpa_fp32(q, k, v, tensor_layout=layout, is_causal=causal)
        acc = so.accuracy(o.float(), ref)
        assert o.dtype == dtype and acc["cos"] > 0.9999 and acc["max_abs"] < 2e-2, acc


def test_peer_mappings_are_opened_once_per_allocation_and_closed_by_the_last_user():
    """peer_gather keeps one CUDA-IPC mapping per exported allocation and process: buffers that share
    an allocation share the mapping, and it is closed when the last of them lets go."""
    import ctypes
    from sageattention_rdna3_b200 import peer_gather as pg

    class FakeLib:
        def __init__(self):
            self.opened, self.closed, self.fail = [], [], False

        def sage_peer_open(self, handle, offset, out):
            if self.fail:
                return 2
            assert offset == 0                      # the mapping is of the allocation, offsets are added by the caller
            self.opened.append(handle)
            ctypes.cast(out, ctypes.POINTER(ctypes.c_void_p))[0] = 0x10000000 + 0x1000000 * len(self.opened)
            return 0

        def sage_peer_close(self, addr, offset):
            self.closed.append(addr.value)
            return 0

        def sage_last_error(self):
            return b"fake failure"

    lib = FakeLib()
    pg._OPEN.clear()
    a = pg._open(lib, b"A" * 64, 256)
    b = pg._open(lib, b"A" * 64, 4096)              # another buffer in the same allocation
    c = pg._open(lib, b"B" * 64, 0)
    assert (a, b, c) == (0x11000000 + 256, 0x11000000 + 4096, 0x12000000)
    assert lib.opened == [b"A" * 64, b"B" * 64]
    pg._close(lib, b"A" * 64)
    assert lib.closed == []                          # still used by the second buffer
    pg._close(lib, b"A" * 64)
    pg._close(lib, b"B" * 64)
    assert lib.closed == [0x11000000, 0x12000000] and pg._OPEN == {}
    pg._close(lib, b"A" * 64)                        # closing what is not open is a no-op
    lib.fail = True
    assert isinstance(pg._open(lib, b"C" * 64, 0), str) and pg._OPEN == {}
