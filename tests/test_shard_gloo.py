"""The multi-rank path on CPU: two gloo ranks shard (batch, kv-head) units, each computes its own
with the CPU oracle standing in for the GPU kernels, and the all-gather must reproduce the
single-process result exactly."""
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


def _oracle_attn(q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None, smooth_k=False, kernel="int8"):
    from oracle import sage_oracle as so
    if kernel == "direct":
        return so.direct_attn_emulated(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale)
    return so.sageattn_emulated(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale,
                                smooth_k=smooth_k)


def _worker(rank, world, port, layout, B, Hq, Hkv, kernel, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    torch.set_num_threads(2)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import randn
        from sageattention_rdna3_b200.shard import sageattn_sharded
        S, D = 48, 64
        shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
        q, k, v = randn(shp(Hq), 0, torch.float16), randn(shp(Hkv), 1, torch.float16), randn(shp(Hkv), 2, torch.float16)
        kw = {} if kernel == "auto" else {"kernel": kernel}      # "auto": S = 48 resolves to the un-quantised kernel
        out = sageattn_sharded(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True, attn_fn=_oracle_attn, **kw)
        local, shard = sageattn_sharded(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True,
                                        attn_fn=_oracle_attn, gather=False, **kw)
        # rank-local form: the rank passes only its own units and the head counts of the whole problem
        from sageattention_rdna3_b200.shard import shard_inputs
        ql, kl, vl = shard_inputs(q, k, v, layout, shard)
        kw_local = dict(kw) if kw else {"kernel": "direct"}
        out_local = sageattn_sharded(ql, kl, vl, tensor_layout=layout, is_causal=True, smooth_k=True,
                                     attn_fn=_oracle_attn, global_heads=(B, Hq, Hkv), **kw_local)
        assert torch.equal(out_local, out), "rank-local inputs give a different gathered output"
        torch.save({"out": out, "n_local": shard.n_units, "local_shape": tuple(local.shape)},
                   os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout,B,Hq,Hkv,kernel", [("HND", 1, 4, 2, "int8"), ("NHD", 1, 6, 3, "int8"),
                                                    ("NHD", 2, 4, 1, "auto")])
def test_two_ranks_reproduce_single_process(tmp_path, layout, B, Hq, Hkv, kernel):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, layout, B, Hq, Hkv, kernel, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import randn
    S, D = 48, 64
    shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
    q, k, v = randn(shp(Hq), 0, torch.float16), randn(shp(Hkv), 1, torch.float16), randn(shp(Hkv), 2, torch.float16)
    want = _oracle_attn(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True,
                        kernel="direct" if kernel == "auto" else kernel)
    units = 0
    for r in range(world):
        got = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        assert got["out"].shape == want.shape
        assert torch.equal(got["out"], want), f"rank {r}: gathered output differs"
        units += got["n_local"]
    assert units == B * Hkv


class _FakePeerOutput:
    """Host-side stand-in for peer_gather.PeerOutput on CPU ranks: the same bookkeeping, with the
    peer stores of the kernel played by an all-gather of the slabs inside ``sync``."""

    def __init__(self, unit_sizes, unit_shape, dtype):
        self.unit_sizes = list(unit_sizes)
        self.rank = dist.get_rank()
        self.starts = [sum(self.unit_sizes[:r]) for r in range(len(self.unit_sizes))]
        self.full = torch.full((sum(self.unit_sizes),) + tuple(unit_shape), float("nan"), dtype=dtype)
        self.seen_scatter = None

    def local_slab(self):
        return self.full[self.starts[self.rank]:self.starts[self.rank] + self.unit_sizes[self.rank]]

    def scatter_addresses(self):
        return [0xDEAD0000 + 16 * r for r in range(len(self.unit_sizes)) if r != self.rank]

    def sync(self):
        slabs = [None] * len(self.unit_sizes)
        dist.all_gather_object(slabs, self.local_slab().clone())
        for r, s in enumerate(slabs):
            self.full[self.starts[r]:self.starts[r] + self.unit_sizes[r]] = s


def _fused_worker(rank, world, port, layout, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    torch.set_num_threads(2)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import randn
        from sageattention_rdna3_b200.shard import plan_shards, sageattn_sharded
        B, Hq, Hkv, S, D = 1, 6, 3, 48, 64            # 3 units over 2 ranks: unequal slabs
        shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
        q, k, v = randn(shp(Hq), 0, torch.float16), randn(shp(Hkv), 1, torch.float16), randn(shp(Hkv), 2, torch.float16)
        sizes = [s.n_units for s in plan_shards(B, Hq, Hkv, world)]
        peer = _FakePeerOutput(sizes, (Hq // Hkv, S, D), torch.float16)
        calls = []

        def attn(q_, k_, v_, out=None, scatter_to=None, **kw):
            calls.append((tuple(out.shape), list(scatter_to)))
            out.copy_(_oracle_attn(q_, k_, v_, **kw))
            return out

        got = sageattn_sharded(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True, attn_fn=attn,
                               gather="fused", peer_output=peer, kernel="int8")
        assert calls == [((sizes[rank], Hq // Hkv, S, D), peer.scatter_addresses())]
        with pytest.raises(ValueError):
            sageattn_sharded(q, k, v, tensor_layout=layout, is_causal=True, attn_fn=attn, gather="fused", kernel="int8")
        wrong = _FakePeerOutput(sizes, (Hq // Hkv, S + 1, D), torch.float16)
        with pytest.raises(ValueError):
            sageattn_sharded(q, k, v, tensor_layout=layout, is_causal=True, attn_fn=attn, gather="fused",
                             peer_output=wrong, kernel="int8")
        torch.save(got.clone(), os.path.join(result_dir, f"fused{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_fused_gather_bookkeeping_on_two_cpu_ranks(tmp_path, layout):
    """gather="fused": every rank computes into its slab of the full buffer and passes the peers'
    addresses on; the gathered result equals the single-process one; a missing or mismatching
    PeerOutput is refused."""
    world = 2
    mp.spawn(_fused_worker, args=(world, _free_port(), layout, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import randn
    B, Hq, Hkv, S, D = 1, 6, 3, 48, 64
    shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
    q, k, v = randn(shp(Hq), 0, torch.float16), randn(shp(Hkv), 1, torch.float16), randn(shp(Hkv), 2, torch.float16)
    want = _oracle_attn(q, k, v, tensor_layout=layout, is_causal=True, smooth_k=True, kernel="int8")
    for r in range(world):
        assert torch.equal(torch.load(os.path.join(str(tmp_path), f"fused{r}.pt")), want), f"rank {r}"
