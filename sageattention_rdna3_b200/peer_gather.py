"""The gathered output of a sharded call, kept on every GPU of the node and written by the attention
kernels themselves.

With (batch, kv-head) units sharded over GPUs (:mod:`.shard`) every rank ends up with a slab of the
output, and a caller that needs all of it on every rank pays for an all-gather afterwards: at 8 GPUs
that collective takes longer than the attention it follows.  Here every rank holds the full output
buffer, maps the buffers of the other ranks into its address space (CUDA IPC, one process per GPU,
one node) and hands their addresses to the attention kernel, whose epilogue writes every finished
tile into its own slab of all of them with ordinary stores (``sage_qk_int8_sv_f16_attn_scatter``):
the transfer runs under the computation, tile by tile, over NVLink.  What is left after the launch
is a one-element all-reduce, which tells every rank that the others' launches - and with them
their stores - have completed.

The reference has no counterpart (it is single-GPU).  No rank reads another GPU's memory; no
library kernel is given a peer address.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import _native


# One mapping per exported allocation and process, however many buffers live inside it (small
# buffers of PyTorch's allocator share an allocation): handle -> [mapped base address, users].
_OPEN = {}


def _open(lib, handle: bytes, offset: int):
    """Address of the peer's buffer in this process, or an error string."""
    if handle in _OPEN:
        _OPEN[handle][1] += 1
        return _OPEN[handle][0] + offset
    addr = ctypes.c_void_p(0)
    rc = lib.sage_peer_open(handle, 0, ctypes.byref(addr))
    if rc != 0:
        return f"sage_peer_open failed ({rc}): {lib.sage_last_error().decode()}"
    _OPEN[handle] = [int(addr.value), 1]
    return int(addr.value) + offset


def _close(lib, handle: bytes) -> None:
    entry = _OPEN.get(handle)
    if entry is None:
        return
    entry[1] -= 1
    if entry[1] == 0:
        del _OPEN[handle]
        _check(lib.sage_peer_close(ctypes.c_void_p(entry[0]), 0), "sage_peer_close")


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {_native.load_abi().sage_last_error().decode()}")


class PeerOutput:
    """``full``: this rank's copy of the gathered output, ``[n_units_total, *unit_shape]``.

    ``unit_sizes[r]`` is the number of units rank ``r`` owns (:func:`.shard.plan_shards`); rank r's slab
    is ``full[sum(unit_sizes[:r]) : sum(unit_sizes[:r+1])]`` in every copy.  Construction is
    collective over ``group``.  The buffers stay mapped until :meth:`close`.
    """

    def __init__(self, unit_sizes: Sequence[int], unit_shape: Sequence[int], dtype: torch.dtype,
                 device: torch.device, group=None):
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert len(unit_sizes) == self.world, "one unit count per rank"
        self.unit_sizes = [int(n) for n in unit_sizes]
        self.starts = [sum(self.unit_sizes[:r]) for r in range(self.world)]
        self.unit_shape = tuple(int(d) for d in unit_shape)
        self.unit_bytes = torch.empty((), dtype=dtype).element_size()
        for d in self.unit_shape:
            self.unit_bytes *= d
        self.full = torch.empty((sum(self.unit_sizes),) + self.unit_shape, dtype=dtype, device=device)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        lib = _native.load_abi()
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_int64(0)
        with torch.cuda.device(device):
            _check(lib.sage_peer_export(ctypes.c_void_p(self.full.data_ptr()), handle, ctypes.byref(offset)),
                   "sage_peer_export")
            mine = (bytes(handle.raw), int(offset.value), tuple(self.full.shape), str(dtype))
            everyone: List[Optional[tuple]] = [None] * self.world
            dist.all_gather_object(everyone, mine, group=group)
            self._mapped = {}            # rank -> (address of that rank's `full`, handle of its allocation)
            problem = None
            for r, (h, off, shape, dt) in enumerate(everyone):
                if r == self.rank:
                    continue
                if shape != tuple(self.full.shape) or dt != str(dtype):
                    problem = f"rank {r} built a different output buffer: {shape} {dt}"
                    break
                addr = _open(lib, h, off)
                if isinstance(addr, str):
                    problem = f"rank {r}'s buffer: {addr}"
                    break
                self._mapped[r] = (addr, h)
            # all ranks succeed or all ranks raise: nobody is left waiting in a collective
            reports: List[Optional[str]] = [None] * self.world
            dist.all_gather_object(reports, problem, group=group)
            bad = [f"rank {r}: {v}" for r, v in enumerate(reports) if v]
            if bad:
                for _, h in self._mapped.values():
                    _close(lib, h)
                self._mapped = {}
                raise RuntimeError("PeerOutput could not be set up: " + "; ".join(bad))

    def local_slab(self, rank: Optional[int] = None) -> torch.Tensor:
        """This rank's units inside its own copy (a view: the kernel's ``out``)."""
        r = self.rank if rank is None else rank
        return self.full[self.starts[r]:self.starts[r] + self.unit_sizes[r]]

    def scatter_addresses(self) -> List[int]:
        """Where this rank's slab starts in every OTHER rank's copy, nearest higher rank first: the
        kernel writes a tile to the peers in this order, and no two ranks start with the same one."""
        off = self.starts[self.rank] * self.unit_bytes
        order = sorted(self._mapped, key=lambda r: (r - self.rank) % self.world)
        return [self._mapped[r][0] + off for r in order]

    def sync(self) -> None:
        """Stream-ordered: returns at once; work queued after it on the current stream sees every
        rank's slab in ``full`` (every rank's launch precedes its contribution to the all-reduce)."""
        import torch.distributed as dist
        dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        import torch.distributed as dist
        torch.cuda.synchronize(self.full.device)
        dist.barrier(group=self.group)          # nobody is still writing into a buffer that is about to go
        lib = _native.load_abi()
        with torch.cuda.device(self.full.device):
            for _, h in self._mapped.values():
                _close(lib, h)
        self._mapped = {}
