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


def _inputs(layout):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import randn
    B, Hq, Hkv, S, D = 2, 6, 3, 700, 128
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
