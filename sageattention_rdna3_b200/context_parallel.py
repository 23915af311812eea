"""Sequence (context) parallel attention over the ranks of one node: a ring over KV shards.

The reference has no counterpart (its attention is single-GPU); this is what its placeholder
``return_lse`` (``sageattention/core.py:47,203-211``) exists for upstream.  Head sharding
(:mod:`.shard`) is the first choice because it needs no exchange; it runs out for the 3-4 head VAE
shapes and for sequences that do not fit one GPU.

Rank r of W holds rows [r*S/W, (r+1)*S/W) of q, k and v.  In step s it attends its queries to the KV
shard of rank (r - s) mod W while that shard travels on to rank r+1 (``batch_isend_irecv``, NCCL over
NVLink on GPUs), and folds the partial result into its accumulators with the log-sum-exp the kernel
returns:

    lse' = logaddexp(lse, lse_j);  o' = o * exp(lse - lse') + o_j * exp(lse_j - lse')

Under a causal mask shard j > r is skipped (every key is in the future), shard j == r is attended
causally and shards j < r in full; the work per rank then grows with r (no zig-zag re-ordering here).
Each shard is quantised on its own, so results agree with single-GPU ``sageattn`` to the accuracy of
the INT8 path, not bit for bit.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


def merge_partial(o: Optional[torch.Tensor], lse: Optional[torch.Tensor], o_j: torch.Tensor, lse_j: torch.Tensor,
                  tensor_layout: str):
    """Fold one partial result (o_j in the caller's layout, lse_j ``[B,H,S]``) into fp32 accumulators."""
    o_j = o_j.float()
    if o is None:
        return o_j, lse_j.clone()
    new = torch.logaddexp(lse, lse_j)
    w_old, w_new = torch.exp(lse - new), torch.exp(lse_j - new)
    # a row that has seen no key yet has lse = -inf on both sides: exp(nan) -> keep zeros
    w_old, w_new = torch.nan_to_num(w_old, nan=0.0), torch.nan_to_num(w_new, nan=0.0)
    if tensor_layout == "HND":
        w_old, w_new = w_old[..., None], w_new[..., None]                       # [B,H,S,1]
    else:
        w_old, w_new = w_old.transpose(1, 2)[..., None], w_new.transpose(1, 2)[..., None]   # [B,S,H,1]
    return o * w_old + o_j * w_new, new


def sageattn_context_parallel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                              is_causal: bool = False, sm_scale: Optional[float] = None, smooth_k: bool = False,
                              group=None, attn_fn: Optional[Callable] = None, **kwargs) -> torch.Tensor:
    """Attention of this rank's query rows to the keys and values of all ranks.

    q, k, v: this rank's sequence shard (equal lengths on all ranks), shaped as for ``sageattn``.
    ``attn_fn(q, k, v, tensor_layout=, is_causal=, sm_scale=, smooth_k=, return_lse=True, **kwargs)``
    must return ``(o, lse)``; it defaults to :func:`sageattn`.  Returns this rank's rows of the output.
    """
    import torch.distributed as dist
    if attn_fn is None:
        from .core import sageattn as attn_fn
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    o_acc, lse_acc = None, None
    k_cur, v_cur = k.contiguous(), v.contiguous()
    for step in range(world):
        src = (rank - step) % world                       # whose shard k_cur / v_cur is
        reqs, k_next, v_next = [], None, None
        if step + 1 < world:
            # pass the shard on while it is being used; the next one arrives in separate buffers
            k_next, v_next = torch.empty_like(k_cur), torch.empty_like(v_cur)
            to_rank = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
            from_rank = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
            ops = [dist.P2POp(dist.isend, k_cur, to_rank, group), dist.P2POp(dist.isend, v_cur, to_rank, group),
                   dist.P2POp(dist.irecv, k_next, from_rank, group), dist.P2POp(dist.irecv, v_next, from_rank, group)]
            reqs = dist.batch_isend_irecv(ops)
        if not (is_causal and src > rank):
            o_j, lse_j = attn_fn(q, k_cur, v_cur, tensor_layout=tensor_layout, is_causal=is_causal and src == rank,
                                 sm_scale=sm_scale, smooth_k=smooth_k, return_lse=True, **kwargs)
            o_acc, lse_acc = merge_partial(o_acc, lse_acc, o_j, lse_j, tensor_layout)
        for r in reqs:
            r.wait()
        if k_next is not None:
            k_cur, v_cur = k_next, v_next
    return o_acc.to(q.dtype)
