"""Sequence (context) parallel attention over the ranks of one node: a ring over KV shards.

The reference has no counterpart (its attention is single-GPU); this is what its placeholder
``return_lse`` (``sageattention/core.py:47,203-211``) exists for upstream.  Head sharding
(:mod:`.shard`) is the first choice because it needs no exchange; it runs out for the 3-4 head VAE
shapes and for sequences that do not fit one GPU.

Rank r of W holds a shard of the rows of q, k and v.  In step s it attends its queries to the KV
shard of rank (r - s) mod W while that shard travels on to rank r+1 (``batch_isend_irecv``, NCCL over
NVLink on GPUs), and folds the partial result into fp32 accumulators with the log-sum-exp the kernel
returns - one launch per fold (``sage_fold_attn_partial``):

    lse' = logaddexp(lse, lse_j);  o' = o * exp(lse - lse') + o_j * exp(lse_j - lse')

Which rows a rank holds:

* contiguous (default): rank r holds rows [r*S/W, (r+1)*S/W).  Under a causal mask shard j > r is
  skipped, shard j == r is attended causally and shards j < r in full: the work grows with r.
* zig-zag (``zigzag=True``, for causal masks): the sequence is cut into 2W chunks and rank r holds
  chunks r and 2W-1-r, in that order (:func:`zigzag_shard`).  Then every rank does the same amount of
  work in every step: its own shard causally; for a shard from a lower rank, all of its queries
  against the first chunk of that shard; for a shard from a higher rank, its second chunk of
  queries against both chunks of that shard.

Each shard is quantised on its own, so results agree with single-GPU ``sageattn`` to the accuracy of
the INT8 path, not bit for bit.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch


def zigzag_shard(x: torch.Tensor, rank: int, world: int, seq_dim: int) -> torch.Tensor:
    """Rows of ``x`` that rank ``rank`` holds under the zig-zag split: chunks ``rank`` and
    ``2*world-1-rank`` of ``2*world`` equal chunks, concatenated.  The length must divide evenly."""
    n = x.size(seq_dim)
    if n % (2 * world) != 0:
        raise ValueError(f"zig-zag sharding needs a sequence length divisible by {2 * world}, got {n}")
    c = n // (2 * world)
    return torch.cat([x.narrow(seq_dim, rank * c, c), x.narrow(seq_dim, (2 * world - 1 - rank) * c, c)], dim=seq_dim)


def zigzag_unshard(parts: Sequence[torch.Tensor], seq_dim: int) -> torch.Tensor:
    """Inverse of :func:`zigzag_shard` over the list of all ranks' shards."""
    world = len(parts)
    chunks: List[Optional[torch.Tensor]] = [None] * (2 * world)
    for r, p in enumerate(parts):
        c = p.size(seq_dim) // 2
        chunks[r] = p.narrow(seq_dim, 0, c)
        chunks[2 * world - 1 - r] = p.narrow(seq_dim, c, c)
    return torch.cat(chunks, dim=seq_dim)


def fold_partial_cuda(o_acc: torch.Tensor, lse_acc: torch.Tensor, o_j: torch.Tensor, lse_j: torch.Tensor,
                      tensor_layout: str, first: bool) -> None:
    """Fold ``(o_j, lse_j)`` into the fp32 accumulators in place: one CUDA launch."""
    from . import _native
    _native.load_ops().fold_partial(o_acc, lse_acc, o_j, lse_j.contiguous(), 1 if tensor_layout == "HND" else 0, int(first))


def _ring_steps(rank: int, world: int, is_causal: bool, zigzag: bool):
    """For every step of the ring: (source rank of the KV shard, which of my query rows take part,
    which rows of the shard are visible, whether the call is causal).  Row selections are None (all),
    "first" or "second" (half of the local rows)."""
    for step in range(world):
        src = (rank - step) % world
        if not is_causal:
            yield src, None, None, False
        elif src == rank:
            yield src, None, None, True
        elif zigzag:
            yield (src, None, "first", False) if src < rank else (src, "second", None, False)
        elif src < rank:
            yield src, None, None, False
        else:
            yield src, "skip", None, False


def _half(x: torch.Tensor, which: Optional[str], seq_dim: int) -> torch.Tensor:
    if which is None:
        return x
    n = x.size(seq_dim) // 2
    return x.narrow(seq_dim, 0, n) if which == "first" else x.narrow(seq_dim, n, x.size(seq_dim) - n)


def sageattn_context_parallel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                              is_causal: bool = False, sm_scale: Optional[float] = None, smooth_k: bool = False,
                              group=None, attn_fn: Optional[Callable] = None, zigzag: bool = False,
                              fold_fn: Optional[Callable] = None,
                              all_shards: Optional[Sequence[Tuple[torch.Tensor, torch.Tensor]]] = None,
                              rank: Optional[int] = None, **kwargs) -> torch.Tensor:
    """Attention of this rank's query rows to the keys and values of all ranks.

    q, k, v: this rank's sequence shard (equal lengths on all ranks; with ``zigzag`` the two chunks of
    :func:`zigzag_shard`), shaped as for ``sageattn``.
    ``attn_fn(q, k, v, tensor_layout=, is_causal=, sm_scale=, smooth_k=, return_lse=True, **kwargs)``
    must return ``(o, lse)``; it defaults to :func:`sageattn`.  ``fold_fn(o_acc, lse_acc, o_j, lse_j,
    tensor_layout, first)`` folds in place; it defaults to the CUDA kernel (:func:`fold_partial_cuda`).
    Returns this rank's rows of the output.

    ``all_shards`` (the list of every rank's ``(k, v)``) together with ``rank`` runs the same steps
    with no communication - a rank of a ring walked inside one process, for tests on one GPU.
    """
    import torch.distributed as dist
    if attn_fn is None:
        from .core import sageattn as attn_fn
    if fold_fn is None:
        fold_fn = fold_partial_cuda
    if all_shards is not None:
        world = len(all_shards)
        assert rank is not None and 0 <= rank < world, "all_shards needs the rank to walk"
    else:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    seq_dim, head_dim_idx = (2, 1) if tensor_layout == "HND" else (1, 2)
    o_acc = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    lse_acc = torch.empty((q.size(0), q.size(head_dim_idx), q.size(seq_dim)), dtype=torch.float32, device=q.device)
    started = False
    k_cur, v_cur = k.contiguous(), v.contiguous()
    for step, (src, q_rows, kv_rows, causal_call) in enumerate(_ring_steps(rank, world, is_causal, zigzag)):
        reqs, k_next, v_next = [], None, None
        if all_shards is not None:
            k_cur, v_cur = all_shards[src]
        elif step + 1 < world:
            # pass the shard on while it is being used; the next one arrives in separate buffers
            k_next, v_next = torch.empty_like(k_cur), torch.empty_like(v_cur)
            to_rank = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
            from_rank = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
            ops = [dist.P2POp(dist.isend, k_cur, to_rank, group), dist.P2POp(dist.isend, v_cur, to_rank, group),
                   dist.P2POp(dist.irecv, k_next, from_rank, group), dist.P2POp(dist.irecv, v_next, from_rank, group)]
            reqs = dist.batch_isend_irecv(ops)
        if q_rows != "skip":
            o_j, lse_j = attn_fn(_half(q, q_rows, seq_dim), _half(k_cur, kv_rows, seq_dim), _half(v_cur, kv_rows, seq_dim),
                                 tensor_layout=tensor_layout, is_causal=causal_call, sm_scale=sm_scale,
                                 smooth_k=smooth_k, return_lse=True, **kwargs)
            # the first fold of a ring is the rank's own shard and always covers all of its rows
            fold_fn(_half(o_acc, q_rows, seq_dim), _half(lse_acc, q_rows, 2), o_j, lse_j, tensor_layout, not started)
            started = True
        for r in reqs:
            r.wait()
        if k_next is not None:
            k_cur, v_cur = k_next, v_next
    return o_acc.to(q.dtype)
