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


@pytest.fixture
def hooks():
    """The library's test hooks, always switched back off."""
    from sageattention_rdna3_b200 import _native
    lib = _native.load_abi()
    yield lib
    lib.sage_test_drop_v_load(0)
    lib.sage_test_set_wait_limit_us(0)


def test_wait_that_cannot_complete_gives_a_status_not_a_hang(hooks):
    dev = torch.device("cuda", 0)
    (q, k, v), (q_i8, k_i8, vd, q_scale, k_scale) = _case(dev)
    hooks.sage_test_set_wait_limit_us(20000)                 # 20 ms instead of about a second
    hooks.sage_test_drop_v_load(1)
    _, _, status = H.abi_attn(q_i8, k_i8, vd, "HND", q_scale, k_scale, torch.float16, "HND", False)
    # 2 + 16 * 6: the wait for a V tile (barrier id 6) gave up
    assert status == 2 + 16 * 6
    hooks.sage_test_drop_v_load(0)
    hooks.sage_test_set_wait_limit_us(0)
    # the context is intact and the next launch is correct
    o, _, status = H.abi_attn(q_i8, k_i8, vd, "HND", q_scale, k_scale, torch.float16, "HND", False)
    assert status == 0
    rq = so.quant_qk_int8(q, k, None, 128 ** -0.5)
    o_ref = so.attention(rq[0], rq[2], v, rq[1], rq[3], False, torch.float16)
    acc = so.accuracy(o.float().cpu(), o_ref.float())
    assert acc["cos"] >= 0.999 and acc["rel_l1"] <= 1e-2, acc


def test_dropped_load_is_ignored_without_a_shortened_bound(hooks):
    """The hook that breaks a launch only works together with the shortened bound: set alone it
    must not cost a launch a second per wave."""
    dev = torch.device("cuda", 0)
    _, (q_i8, k_i8, vd, q_scale, k_scale) = _case(dev)
    hooks.sage_test_drop_v_load(1)
    _, _, status = H.abi_attn(q_i8, k_i8, vd, "HND", q_scale, k_scale, torch.float16, "HND", False)
    assert status == 0


def test_later_ctas_leave_at_once_when_the_status_word_is_set(hooks):
    """Many CTAs (several waves), every one of which would time out: the launch must take about one
    bound, not one per wave - CTAs that start after the first report see the word and return."""
    import time
    dev = torch.device("cuda", 0)
    q, k, v = (H.randn((1, 16, 8192, 128), s, torch.float16) for s in (0, 1, 2))      # 1024 CTAs: 3.5 waves
    q_i8, q_scale, k_i8, k_scale, _ = H.abi_quant(q.to(dev), k.to(dev), None, "HND", 128 ** -0.5)
    vd = v.to(dev)
    hooks.sage_test_set_wait_limit_us(50000)                 # 50 ms
    hooks.sage_test_drop_v_load(1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _, _, status = H.abi_attn(q_i8, k_i8, vd, "HND", q_scale, k_scale, torch.float16, "HND", False)
    dt = time.perf_counter() - t0
    assert status % 16 == 2, status      # some bounded wait gave up (which one reports first is a race)
    assert dt < 0.15, f"a failing launch of 3.5 waves took {dt * 1e3:.0f} ms with a 50 ms bound"


def test_public_api_raises_on_device_status(hooks):
    from sageattention_rdna3_b200 import check_status, sageattn
    dev = torch.device("cuda", 0)
    q, k, v = (H.randn((1, 1, 256, 128), s, torch.float16).to(dev) for s in (0, 1, 2))
    hooks.sage_test_set_wait_limit_us(20000)
    hooks.sage_test_drop_v_load(1)
    sageattn(q, k, v, kernel="int8")
    with pytest.raises(RuntimeError, match="device status"):
        check_status(dev)
    hooks.sage_test_drop_v_load(0)
    hooks.sage_test_set_wait_limit_us(0)
    sageattn(q, k, v, kernel="int8")
    check_status(dev)                                        # cleared, and the new call was clean


def test_next_call_reports_the_failure_of_the_previous_one(hooks):
    """Without any explicit check: the status word is mirrored to pinned host memory after every
    call, and the next ``sageattn`` on the device looks at the mirror before it launches."""
    from sageattention_rdna3_b200 import check_status, sageattn
    dev = torch.device("cuda", 0)
    q, k, v = (H.randn((1, 1, 256, 128), s, torch.float16).to(dev) for s in (0, 1, 2))
    hooks.sage_test_set_wait_limit_us(20000)
    hooks.sage_test_drop_v_load(1)
    sageattn(q, k, v, kernel="int8")
    hooks.sage_test_drop_v_load(0)
    hooks.sage_test_set_wait_limit_us(0)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status"):
        sageattn(q, k, v, kernel="int8")
    o = sageattn(q, k, v, kernel="int8")                     # the raise cleared the word
    check_status(dev)
    assert torch.isfinite(o.float()).all()
