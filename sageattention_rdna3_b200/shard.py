"""Multi-GPU sharding of ``sageattn`` over (batch, kv-head) units.

Every (batch, kv head) pair - with the ``Hq/Hkv`` query heads that read it (GQA,
``csrc/attn_gfx11.cu:464`` of the reference) - is an independent attention problem, so the path
shards with no exchange during compute.  The reference itself is single-GPU; this module is the
new piece: a planner (pure Python), slicing of the inputs into a rank's units, and an optional
final all-gather of the outputs (NCCL on GPUs; any ``torch.distributed`` backend works, the CPU
tests use gloo).  One process per GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch


@dataclass(frozen=True)
class Shard:
    rank: int
    unit_start: int      # first unit u = b * Hkv + hkv owned by the rank
    unit_stop: int       # one past the last

    @property
    def n_units(self) -> int:
        return self.unit_stop - self.unit_start


def plan_shards(batch: int, num_qo_heads: int, num_kv_heads: int, world_size: int) -> List[Shard]:
    """Contiguous, count-balanced ranges of units per rank (all units cost the same, causal or not).

    The first ``n % world`` ranks get one unit more.  Ranks may be left without work when there are
    fewer units than ranks.
    """
    if batch < 0 or num_kv_heads <= 0 or num_qo_heads % num_kv_heads != 0 or world_size <= 0:
        raise ValueError("plan_shards: need batch >= 0, Hkv > 0, Hq % Hkv == 0, world_size > 0")
    n = batch * num_kv_heads
    base, extra = divmod(n, world_size)
    shards, start = [], 0
    for r in range(world_size):
        size = base + (1 if r < extra else 0)
        shards.append(Shard(r, start, start + size))
        start += size
    return shards


def to_units(x: torch.Tensor, tensor_layout: str, num_kv_heads: int) -> torch.Tensor:
    """View ``x`` ([B,H,S,D] or [B,S,H,D]) as ``[B*Hkv, H/Hkv, S, D]`` (units first, HND inside)."""
    if tensor_layout == "NHD":
        x = x.permute(0, 2, 1, 3)
    B, H, S, D = x.shape
    rep = H // num_kv_heads
    return x.reshape(B * num_kv_heads, rep, S, D) if x.is_contiguous() else \
        x.unflatten(1, (num_kv_heads, rep)).flatten(0, 1)


def shard_inputs(q, k, v, tensor_layout: str, shard: Shard):
    """This rank's units as a batch of single-kv-head problems in HND layout:
    q ``[n, Hq/Hkv, Sq, D]``, k and v ``[n, 1, Skv, D]``."""
    hkv = k.size(1) if tensor_layout == "HND" else k.size(2)
    sl = slice(shard.unit_start, shard.unit_stop)
    return (to_units(q, tensor_layout, hkv)[sl].contiguous(), to_units(k, tensor_layout, hkv)[sl].contiguous(),
            to_units(v, tensor_layout, hkv)[sl].contiguous())


def from_units(o_units: torch.Tensor, batch: int, num_qo_heads: int, tensor_layout: str) -> torch.Tensor:
    """Inverse of :func:`to_units` for the output: ``[B*Hkv, rep, S, D]`` -> caller layout."""
    n, rep, S, D = o_units.shape
    o = o_units.reshape(batch, num_qo_heads, S, D)
    return o if tensor_layout == "HND" else o.permute(0, 2, 1, 3).contiguous()


def sageattn_sharded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                     is_causal: bool = False, sm_scale: Optional[float] = None, smooth_k: bool = False,
                     group=None, gather=True, attn_fn: Optional[Callable] = None,
                     global_heads: Optional[tuple] = None, peer_output=None, **kwargs):
    """Run this rank's share of ``sageattn(q, k, v)`` and optionally all-gather the outputs.

    Two ways to pass the inputs.  Global: every rank passes the same global ``q, k, v`` in
    ``tensor_layout`` (or at least its own units filled in).  Rank-local: with
    ``global_heads=(B, Hq, Hkv)`` of the whole problem, ``q, k, v`` are only this rank's units of
    :func:`plan_shards`, already in unit form - q ``[n, Hq/Hkv, Sq, D]``, k and v ``[n, 1, Skv, D]`` -
    so no rank ever holds another rank's data; ``tensor_layout`` then only names the layout of the
    gathered result.  Returns the full output in ``tensor_layout`` when ``gather`` is true,
    otherwise this rank's units ``[n, Hq/Hkv, Sq, D]`` and its :class:`Shard`.  ``attn_fn`` defaults to :func:`sageattn`; other
    keyword arguments go to it.  The choice between the INT8 and the un-quantised kernel is made
    here, from the caller's shapes and layout, so that every rank and the unsharded call agree.

    ``gather="fused"`` with ``peer_output`` (a :class:`.peer_gather.PeerOutput` built once for these
    shapes): the attention kernel writes this rank's slab into every rank's copy of the output while
    it computes, and the collective shrinks to a one-element all-reduce.  The result is a view of
    ``peer_output.full`` (valid until the next call that uses the same ``peer_output``).
    """
    import torch.distributed as dist
    if attn_fn is None:
        from .core import sageattn as attn_fn
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if global_heads is not None:
        B, hq, hkv = global_heads
        shards = plan_shards(B, hq, hkv, world)
        mine = shards[rank]
        if q.size(0) != mine.n_units or q.size(1) != hq // hkv or k.size(1) != 1:
            raise ValueError(f"rank {rank} owns {mine.n_units} units of {hq // hkv} query head(s): expected q "
                             f"[{mine.n_units}, {hq // hkv}, Sq, D] and k, v [{mine.n_units}, 1, Skv, D], got "
                             f"{tuple(q.shape)} and {tuple(k.shape)}")
        ql, kl, vl = q, k, v
        q_len, kv_len = q.size(2), k.size(2)
    else:
        B = q.size(0)
        hq = q.size(1) if tensor_layout == "HND" else q.size(2)
        hkv = k.size(1) if tensor_layout == "HND" else k.size(2)
        shards = plan_shards(B, hq, hkv, world)
        mine = shards[rank]
        ql, kl, vl = shard_inputs(q, k, v, tensor_layout, mine)
        s_dim = 2 if tensor_layout == "HND" else 1
        q_len, kv_len = q.size(s_dim), k.size(s_dim)
    if "kernel" not in kwargs:
        from .core import use_direct_kernel
        direct = use_direct_kernel(q.size(-1), tensor_layout, is_causal, q_len, kv_len)
        kwargs["kernel"] = "direct" if direct else "int8"
    if gather == "fused" and world > 1:
        if peer_output is None:
            raise ValueError('gather="fused" needs peer_output=PeerOutput(...)')
        rep = hq // hkv
        want = (B * hkv, rep, ql.size(2), ql.size(3))
        if tuple(peer_output.full.shape) != want or peer_output.full.dtype != ql.dtype or \
                peer_output.unit_sizes != [s.n_units for s in shards]:
            raise ValueError(f"peer_output was built for {tuple(peer_output.full.shape)} {peer_output.full.dtype} "
                             f"{peer_output.unit_sizes}, this call needs {want} {ql.dtype} {[s.n_units for s in shards]}")
        if mine.n_units > 0:
            attn_fn(ql, kl, vl, tensor_layout="HND", is_causal=is_causal, sm_scale=sm_scale, smooth_k=smooth_k,
                    out=peer_output.local_slab(), scatter_to=peer_output.scatter_addresses(), **kwargs)
        peer_output.sync()
        return from_units(peer_output.full, B, hq, tensor_layout)
    if mine.n_units > 0:
        o_local = attn_fn(ql, kl, vl, tensor_layout="HND", is_causal=is_causal, sm_scale=sm_scale, smooth_k=smooth_k,
                          **kwargs)
    else:
        o_local = ql.new_empty(ql.shape)
    if not gather:
        return o_local, mine
    if world == 1:
        return from_units(o_local, B, hq, tensor_layout)
    rep, Sq, D = hq // hkv, ql.size(2), ql.size(3)
    sizes = [s.n_units for s in shards]
    if len(set(sizes)) == 1:
        # equal slabs of [units, rep, Sq, D]: one all_gather_into_tensor straight into the result
        out = o_local.new_empty(B * hkv, rep, Sq, D)
        dist.all_gather_into_tensor(out, o_local.contiguous(), group=group)
    else:
        # unequal shares: pad every rank's slab to the largest, gather, drop the padding
        n_max = max(sizes)
        padded = o_local.new_zeros(n_max, rep, Sq, D)
        padded[:mine.n_units] = o_local
        gathered = o_local.new_empty(world * n_max, rep, Sq, D)
        dist.all_gather_into_tensor(gathered, padded, group=group)
        out = torch.cat([gathered[r * n_max:r * n_max + n] for r, n in enumerate(sizes)], dim=0)
    return from_units(out, B, hq, tensor_layout)
