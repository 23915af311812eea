"""Failure detection on the device, without faulting or hanging the GPU.

Every barrier wait in the attention kernel is bounded.  The test shortens the bound and uses the
library's test hook to make one wait run out for real (the TMA producer never loads V of the first
KV tile, so the MMA warp's wait for it cannot be satisfied).  The kernel must then return by
itself, report through the status word, and leave the CUDA context usable for the next call.
"""
import pytest
import torch

import helpers as H
from oracle import sage_oracle as so

pytestmark = pytest.mark.gpu


def _case(dev):
    q, k, v = (H.randn((1, 1, 256, 128), s, torch.float16) for s in (0, 1, 2))
    sm = 128 ** -0.5
    q_i8, q_scale, k_i8, k_scale, _ = H.abi_quant(q.to(dev), k.to(dev), None, "HND", sm)
    return (q, k, v), (q_i8, k_i8, v.to(dev), q_scale, k_scale)


def test_wait_that_cannot_complete_gives_a_status_not_a_hang(monkeypatch):
    dev = torch.device("cuda", 0)
    (q, k, v), (q_i8, k_i8, vd, q_scale, k_scale) = _case(dev)
    monkeypatch.setenv("SAGE_WAIT_LIMIT_US", "20000")        # 20 ms instead of about a second
    monkeypatch.setenv("SAGE_TEST_DROP_V_LOAD", "1")
    _, _, status = H.abi_attn(q_i8, k_i8, vd, "HND", q_scale, k_scale, torch.float16, "HND", False)
    # 2 + 16 * 6: the wait for a V tile (barrier id 6) gave up
    assert status == 2 + 16 * 6
    monkeypatch.delenv("SAGE_TEST_DROP_V_LOAD")
    monkeypatch.delenv("SAGE_WAIT_LIMIT_US")
    # the context is intact and the next launch is correct
    o, _, status = H.abi_attn(q_i8, k_i8, vd, "HND", q_scale, k_scale, torch.float16, "HND", False)
    assert status == 0
    rq = so.quant_qk_int8(q, k, None, 128 ** -0.5)
    o_ref = so.attention(rq[0], rq[2], v, rq[1], rq[3], False, torch.float16)
    acc = so.accuracy(o.float().cpu(), o_ref.float())
    assert acc["cos"] >= 0.999 and acc["rel_l1"] <= 1e-2, acc


def test_public_api_raises_on_device_status(monkeypatch):
    from sageattention_rdna3_b200 import check_status, sageattn
    dev = torch.device("cuda", 0)
    q, k, v = (H.randn((1, 1, 256, 128), s, torch.float16).to(dev) for s in (0, 1, 2))
    monkeypatch.setenv("SAGE_WAIT_LIMIT_US", "20000")
    monkeypatch.setenv("SAGE_TEST_DROP_V_LOAD", "1")
    sageattn(q, k, v)
    with pytest.raises(RuntimeError, match="device status"):
        check_status(dev)
    monkeypatch.delenv("SAGE_TEST_DROP_V_LOAD")
    monkeypatch.delenv("SAGE_WAIT_LIMIT_US")
    sageattn(q, k, v)
    check_status(dev)                                        # cleared, and the new call was clean
