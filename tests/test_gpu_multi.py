"""Two ranks on two GPUs (NCCL): each computes its (batch, kv-head) units with the CUDA kernels,
the all-gather must reproduce the single-GPU result - bit for bit with the one-tile-per-CTA launch
(SAGE_STREAMK=0), to fp32 rounding of the merge when the scheduler may pick persistent CTAs (a rank
with half of the units cuts its work into different spans).  Skipped with fewer than 2 GPUs."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(layout, B=2):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import randn
    Hq, Hkv, S, D = 6, 3, 700, 128
    shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
    return randn(shp(Hq), 0, torch.bfloat16), randn(shp(Hkv), 1, torch.bfloat16, offset=1.0), randn(shp(Hkv), 2, torch.bfloat16)


def _worker(rank, world, port, layout, streamk, out_dir):
    sys.path.insert(0, ROOT)
    if streamk is not None:
        os.environ["SAGE_STREAMK"] = streamk
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sageattention_rdna3_b200 import check_status
        from sageattention_rdna3_b200.shard import sageattn_sharded
        q, k, v = (t.cuda(rank) for t in _inputs(layout))
        out = sageattn_sharded(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True)
        check_status(rank)
        torch.save(out.cpu(), os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("streamk", ["0", None])
@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_two_gpus_reproduce_one(tmp_path, monkeypatch, layout, streamk):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_worker, args=(2, _free_port(), layout, streamk, str(tmp_path)), nprocs=2, join=True)
    from sageattention_rdna3_b200 import sageattn
    if streamk is not None:
        monkeypatch.setenv("SAGE_STREAMK", streamk)
    q, k, v = (t.cuda(0) for t in _inputs(layout))
    want = sageattn(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True).cpu()
    for r in range(2):
        got = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        if streamk == "0":
            assert torch.equal(got, want), f"rank {r}"
        else:
            assert (got.float() - want.float()).abs().max().item() <= 2 ** -5, f"rank {r}"


def _cp_worker(rank, world, port, layout, causal, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sageattention_rdna3_b200 import check_status
        from sageattention_rdna3_b200.context_parallel import sageattn_context_parallel
        s_dim = 2 if layout == "HND" else 1
        q, k, v = (t.chunk(world, dim=s_dim)[rank].contiguous().cuda(rank) for t in _cp_inputs(layout))
        out = sageattn_context_parallel(q, k, v, tensor_layout=layout, is_causal=causal, smooth_k=True, kernel="int8")
        check_status(rank)
        torch.save(out.cpu(), os.path.join(out_dir, f"cp{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _cp_inputs(layout):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import randn
    B, Hq, Hkv, S, D = 1, 4, 2, 2048, 128
    shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
    return randn(shp(Hq), 0, torch.bfloat16), randn(shp(Hkv), 1, torch.bfloat16, offset=1.0), randn(shp(Hkv), 2, torch.bfloat16)


@pytest.mark.parametrize("layout,causal", [("HND", True), ("NHD", False)])
def test_context_parallel_ring_on_two_gpus(tmp_path, layout, causal):
    """Sequence shards on two GPUs, KV passed round the ring over NCCL, partials merged with the
    kernel's log-sum-exp: equal to one-GPU attention to the accuracy of the INT8 path."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_cp_worker, args=(2, _free_port(), layout, causal, str(tmp_path)), nprocs=2, join=True)
    sys.path.insert(0, ROOT)
    from oracle import sage_oracle as so
    from sageattention_rdna3_b200 import sageattn
    q, k, v = _cp_inputs(layout)
    want = sageattn(q.cuda(0), k.cuda(0), v.cuda(0), tensor_layout=layout, is_causal=causal, smooth_k=True,
                    kernel="int8").cpu()
    s_dim = 2 if layout == "HND" else 1
    got = torch.cat([torch.load(os.path.join(str(tmp_path), f"cp{r}.pt")) for r in range(2)], dim=s_dim)
    acc = so.accuracy(got.float(), want.float())
    # two INT8 runs with different quantisation groups and K means: each is ~1.1e-2 (rel L1) from fp32
    assert acc["cos"] >= 0.9999 and acc["rel_l1"] <= 2e-2, acc
    ref = so.sdpa_fp32(q, k, v, tensor_layout=layout, is_causal=causal)
    acc2 = so.accuracy(got.float(), ref)
    assert acc2["cos"] > 0.98 and acc2["max_abs"] < 0.35, acc2


def _fused_worker(rank, world, port, layout, B, kernel, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["SAGE_STREAMK"] = "0"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sageattention_rdna3_b200 import check_status
        from sageattention_rdna3_b200.peer_gather import PeerOutput
        from sageattention_rdna3_b200.shard import plan_shards, sageattn_sharded
        q, k, v = (t.cuda(rank) for t in _inputs(layout, B))
        Hq, Hkv, S, D = 6, 3, 700, 128
        sizes = [s.n_units for s in plan_shards(B, Hq, Hkv, world)]
        # two sets of buffers (small ones share an allocation of the caching allocator: one mapping serves both)
        peers = [PeerOutput(sizes, (Hq // Hkv, S, D), torch.bfloat16, torch.device("cuda", rank)) for _ in range(2)]
        try:
            for p in peers:
                p.full.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            outs = []
            for i in range(4):      # the buffers are used alternately and reused
                outs.append(sageattn_sharded(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True, gather="fused",
                                             peer_output=peers[i & 1], kernel=kernel))
            check_status(rank)
            assert torch.equal(outs[2], outs[3])
            torch.save(outs[3].cpu(), os.path.join(out_dir, f"fused{rank}.pt"))
        finally:
            for p in peers:
                p.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout,B,kernel", [("HND", 2, "int8"), ("NHD", 2, "int8"), ("HND", 1, "int8"), ("NHD", 1, "direct")])
def test_fused_gather_on_two_gpus(tmp_path, monkeypatch, layout, B, kernel):
    """The attention kernels write their slabs into both GPUs' copies of the output (peer stores from
    the epilogue); after the one-element all-reduce every rank holds the single-GPU result, bit for
    bit.  3 + 3 units, or 2 + 1 (slabs of different sizes); a sequence length that is not a multiple
    of the tile."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_fused_worker, args=(2, _free_port(), layout, B, kernel, str(tmp_path)), nprocs=2, join=True)
    from sageattention_rdna3_b200 import sageattn
    monkeypatch.setenv("SAGE_STREAMK", "0")
    q, k, v = (t.cuda(0) for t in _inputs(layout, B))
    want = sageattn(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True, kernel=kernel).cpu()
    for r in range(2):
        got = torch.load(os.path.join(str(tmp_path), f"fused{r}.pt"))
        assert torch.equal(got, want), f"rank {r}"
