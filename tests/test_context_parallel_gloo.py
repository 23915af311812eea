"""Ring (context-parallel) attention on two gloo ranks, CPU only: the oracle stands in for the CUDA
kernels, so this checks the ring schedule, the causal shard rules and the log-sum-exp merge."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_attn(q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None, smooth_k=False, return_lse=False):
    from oracle import sage_oracle as so
    return so.sageattn_emulated(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale,
                                smooth_k=smooth_k, return_lse=return_lse)


def _inputs(layout):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import randn
    B, Hq, Hkv, S, D = 1, 4, 2, 192, 64
    shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
    return randn(shp(Hq), 0, torch.float16), randn(shp(Hkv), 1, torch.float16, offset=0.5), randn(shp(Hkv), 2, torch.float16)


def _worker(rank, world, port, layout, causal, out_dir, zigzag=False):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import sage_oracle as so
        from sageattention_rdna3_b200.context_parallel import sageattn_context_parallel, zigzag_shard
        s_dim = 2 if layout == "HND" else 1
        if zigzag:
            q, k, v = (zigzag_shard(t, rank, world, s_dim).contiguous() for t in _inputs(layout))
        else:
            q, k, v = (t.chunk(world, dim=s_dim)[rank].contiguous() for t in _inputs(layout))
        out = sageattn_context_parallel(q, k, v, tensor_layout=layout, is_causal=causal, smooth_k=True,
                                        attn_fn=_oracle_attn, fold_fn=so.fold_partial, zigzag=zigzag)
        torch.save(out, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout,causal", [("HND", False), ("HND", True), ("NHD", True)])
def test_ring_of_two_matches_full_attention(tmp_path, layout, causal):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), layout, causal, str(tmp_path)), nprocs=world, join=True)
    from oracle import sage_oracle as so
    q, k, v = _inputs(layout)
    ref = so.sdpa_fp32(q, k, v, tensor_layout=layout, is_causal=causal)
    s_dim = 2 if layout == "HND" else 1
    got = torch.cat([torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)], dim=s_dim)
    acc = so.accuracy(got.float(), ref)
    # the accuracy of the INT8 path itself against fp32 (every shard is quantised on its own)
    assert acc["cos"] > 0.9995 and acc["max_abs"] < 0.05, acc


@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_zigzag_ring_of_two_matches_full_attention(tmp_path, layout):
    from sageattention_rdna3_b200.context_parallel import zigzag_unshard
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), layout, True, str(tmp_path), True), nprocs=world, join=True)
    from oracle import sage_oracle as so
    q, k, v = _inputs(layout)
    ref = so.sdpa_fp32(q, k, v, tensor_layout=layout, is_causal=True)
    s_dim = 2 if layout == "HND" else 1
    got = zigzag_unshard([torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)], s_dim)
    acc = so.accuracy(got.float(), ref)
    assert acc["cos"] > 0.9995 and acc["max_abs"] < 0.05, acc


@pytest.mark.parametrize("world,zigzag,causal", [(4, True, True), (3, False, True), (4, False, False)])
def test_ring_walked_in_one_process(world, zigzag, causal):
    """Every rank of a ring walked in this process (``all_shards``): the schedule and the shard rules
    for more than two ranks, with the oracle as the attention and the fold."""
    from oracle import sage_oracle as so
    from sageattention_rdna3_b200.context_parallel import sageattn_context_parallel, zigzag_shard, zigzag_unshard
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import randn
    B, Hq, Hkv, S, D = 1, 2, 1, 48 * world, 64
    q, k, v = randn((B, Hq, S, D), 0, torch.float16), randn((B, Hkv, S, D), 1, torch.float16), randn((B, Hkv, S, D), 2, torch.float16)
    cut = (lambda t, r: zigzag_shard(t, r, world, 2).contiguous()) if zigzag else (lambda t, r: t.chunk(world, dim=2)[r].contiguous())
    shards = [(cut(k, r), cut(v, r)) for r in range(world)]
    outs = [sageattn_context_parallel(cut(q, r), *shards[r], is_causal=causal, attn_fn=_oracle_attn, fold_fn=so.fold_partial,
                                      zigzag=zigzag, all_shards=shards, rank=r) for r in range(world)]
    got = zigzag_unshard(outs, 2) if zigzag else torch.cat(outs, dim=2)
    acc = so.accuracy(got.float(), so.sdpa_fp32(q, k, v, is_causal=causal))
    assert acc["cos"] > 0.9995 and acc["max_abs"] < 0.05, acc


def test_fold_of_partials_is_exact_for_fp32_partials():
    """The fold on exact partial results reproduces softmax attention over the union of keys."""
    from oracle import sage_oracle as so
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 2, 16, 8, generator=g) for _ in range(3))
    s = torch.einsum("bhsd,bhtd->bhst", q, k)
    full = torch.softmax(s, -1) @ v
    o, lse = torch.empty(1, 2, 16, 8), torch.empty(1, 2, 16)
    for i, (lo, hi) in enumerate(((0, 5), (5, 6), (6, 16))):
        so.fold_partial(o, lse, torch.softmax(s[..., lo:hi], -1) @ v[:, :, lo:hi], torch.logsumexp(s[..., lo:hi], -1), "HND", i == 0)
    assert torch.allclose(o, full, atol=1e-5) and torch.allclose(lse, torch.logsumexp(s, -1), atol=1e-5)
