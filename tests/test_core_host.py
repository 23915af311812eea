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
    assert [s.n_units for s in plan_shards(2, 32, 32, 8)] == [8] * 8          # config 3
    assert [s.n_units for s in plan_shards(4, 32, 8, 8)] == [4] * 8           # config 4 (4 q heads per unit)
    assert [s.n_units for s in plan_shards(1, 24, 24, 8)] == [3] * 8          # config 5
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
