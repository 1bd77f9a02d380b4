"""Symmetric tensor factories: the three ways the reference hands out cross-rank memory
(moonep/buffer.py:182-410 -- an all-rank view of per-rank chunks, the same plus an NVSwitch
multicast alias, and one owner's allocation mapped by everyone), built on ``SymmetricHeap``.

All three are collective over ``group``, must be destroyed collectively (``destroy()``) before
the process group goes away, and fall back to ordinary device memory when no process group is
in use (single process).
"""

from __future__ import annotations

import ctypes as C
import math
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _native
from ..geometry import align_up
from .symm import (HANDLE_FABRIC, SymmetricHeap, _all_gather_bytes, exchange_fds,
                   resolve_handle_kind, tensor_from_ptr, vmm_granularity)


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _multi(group) -> bool:
    return dist.is_initialized() and dist.get_world_size(group) > 1


@dataclass
class DistTensor:
    """``all``: ``[R * rows, *shape[1:]]`` with rank r's chunk at rows ``[r*rows, (r+1)*rows)``, readable
    and writable from every rank; ``local``: this rank's ``[shape[0], ...]`` part; ``multicast``:
    alias of one chunk whose stores land in every rank's chunk (or None); ``rows``: dim 0 of a
    chunk after padding to the allocation granularity."""
    all: torch.Tensor
    local: torch.Tensor
    multicast: torch.Tensor | None
    rows: int
    heap: SymmetricHeap | None

    def of_rank(self, r: int) -> torch.Tensor:
        return self.all[r * self.rows:r * self.rows + self.local.shape[0]]

    def destroy(self) -> None:
        self.all = self.local = self.multicast = None
        if self.heap is not None:
            torch.cuda.synchronize()
            if _multi(getattr(self, "_group", None)):
                dist.barrier(group=getattr(self, "_group", None))
            self.heap.close()
            self.heap = None


def create_dist_tensor(shape, dtype: torch.dtype, group=None, multicast: bool = False) -> DistTensor:
    """One ``shape``-sized chunk per rank, all chunks mapped back to back on every rank.  With
    ``multicast=True`` the chunks are also bound to an NVSwitch multicast object when the platform
    offers one (``DistTensor.multicast`` stays None otherwise: callers fall back to peer stores)."""
    shape = tuple(int(s) for s in shape)
    dev = torch.device("cuda", torch.cuda.current_device())
    if not _multi(group):
        t = torch.zeros(shape, dtype=dtype, device=dev)
        return DistTensor(t, t, None, shape[0], None)
    es = torch.tensor([], dtype=dtype).element_size()
    row_bytes = es * _numel(shape[1:])
    payload = shape[0] * row_bytes

    def padded_rows(gran: int) -> int:       # smallest dim 0 >= shape[0] whose chunk is a multiple of gran
        step = gran // math.gcd(gran, row_bytes)
        return (shape[0] + step - 1) // step * step

    gran = vmm_granularity(dev.index)
    rows = padded_rows(gran)
    if multicast:
        # a multicast object wants its (often much larger) granularity; a small tensor is not
        # blown up for it and simply does without the alias
        mg = C.c_size_t(0)
        kind = resolve_handle_kind(dev.index, group)
        lib = _native.load()
        ok = lib.mep_multicast_granularity(dev.index, dist.get_world_size(group), kind, rows * row_bytes, C.byref(mg)) == 0
        big = padded_rows(max(gran, mg.value)) if ok and mg.value else 0
        want = 1 if big and big * row_bytes <= max(4 * payload, 64 << 20) else 0
        flags = _all_gather_bytes(bytes([want]), group)
        multicast = all(f == b"\x01" for f in flags)
        if multicast:
            rows = big
    heap = SymmetricHeap.create(rows * row_bytes, group=group, multicast=multicast)
    if heap.chunk_bytes % row_bytes:
        heap.close()
        raise RuntimeError(f"symmetric chunk of {heap.chunk_bytes} bytes is not a whole number of {row_bytes}-byte rows")
    rows = heap.chunk_bytes // row_bytes
    whole = heap.whole().view(dtype).view(heap.world * rows, *shape[1:])
    local = whole[heap.rank * rows:heap.rank * rows + shape[0]]
    mc = None
    if heap.mc_base:
        mc = tensor_from_ptr(heap.mc_base, heap.chunk_bytes, dev).view(dtype).view(rows, *shape[1:])[:shape[0]]
    out = DistTensor(whole, local, mc, rows, heap)
    out._group = group
    return out


class SingleOwnerTensor:
    """``tensor``: ``shape`` elements that live in ``owner``'s memory and are mapped read-write
    by every rank of the group."""

    def __init__(self, tensor, owner, heap=None, mapping=None, group=None):
        self.tensor, self.owner = tensor, owner
        self._heap, self._mapping, self._group = heap, mapping, group

    def destroy(self) -> None:
        self.tensor = None
        if self._heap is None and self._mapping is None:
            return
        torch.cuda.synchronize()
        if _multi(self._group):
            dist.barrier(group=self._group)        # nobody unmaps while a peer may still touch the memory
        if self._mapping is not None:
            _native.load().mep_unmap_all(self._mapping)
            self._mapping = None
        if self._heap is not None:
            self._heap.close()
            self._heap = None


def create_single_owner_tensor(shape, dtype: torch.dtype, owner: int = 0, group=None) -> SingleOwnerTensor:
    """Only ``owner`` allocates; its chunk is exported (fd or fabric handle, same policy as the
    heap) and every other rank imports and maps just that chunk."""
    shape = tuple(int(s) for s in shape)
    dev = torch.device("cuda", torch.cuda.current_device())
    if not _multi(group):
        return SingleOwnerTensor(torch.zeros(shape, dtype=dtype, device=dev), 0)
    lib = _native.load()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    assert 0 <= owner < world, f"owner {owner} is not a rank of the group (size {world})"
    es = torch.tensor([], dtype=dtype).element_size()
    kind = resolve_handle_kind(dev.index, group)
    nbytes = align_up(max(1, _numel(shape)) * es, vmm_granularity(dev.index))
    chunk, mapping, base = C.c_void_p(), C.c_void_p(), C.c_ulonglong(0)
    share = (C.c_ubyte * 64)()
    heap = None
    if rank == owner:
        _native.check(lib.mep_chunk_create(dev.index, nbytes, kind, C.byref(chunk), share), "chunk create")
    if kind == HANDLE_FABRIC:
        blob = _all_gather_bytes(bytes(share) if rank == owner else b"", group)[owner]
        recv = (C.c_ubyte * 64).from_buffer_copy(blob)
    else:
        # all-to-all of descriptors: only the owner's matters, the others send a placeholder
        send_fd = (int.from_bytes(bytes(share[:4]), "little", signed=True) if rank == owner
                   else os.open(os.devnull, os.O_RDONLY))
        try:
            fds = exchange_fds(send_fd, group)
        finally:
            lib.mep_close_fd(send_fd)
        for i, fd in enumerate(fds):
            if i != owner or rank == owner:
                lib.mep_close_fd(fd)
        recv = (C.c_ubyte * 64)()
        if rank != owner:
            C.memmove(recv, int(fds[owner]).to_bytes(4, "little", signed=True), 4)
    try:
        if rank == owner:
            table = (C.c_ubyte * 64)(0xFF, 0xFF, 0xFF, 0xFF)      # fd -1: the own entry carries no descriptor
            _native.check(lib.mep_map_all(dev.index, 1, 0, chunk, table, C.byref(mapping), C.byref(base)), "map own chunk")
        else:
            _native.check(lib.mep_map_remote_one(dev.index, kind, nbytes, recv, C.byref(mapping), C.byref(base)),
                          "map the owner's chunk")     # consumes the descriptor
    except Exception:
        if rank == owner:
            lib.mep_chunk_release(chunk)
        raise
    if rank == owner:
        heap = SymmetricHeap()          # carries the owned chunk so that close() releases it
        heap.world, heap.rank, heap.device, heap.chunk_bytes = 1, 0, dev, nbytes
        heap._chunk, heap._mapping, heap.base = chunk, mapping, base.value
        mapping_for_self = None
    else:
        mapping_for_self = mapping
    raw = tensor_from_ptr(base.value, nbytes, dev)
    if rank == owner:
        raw.zero_()
        torch.cuda.synchronize()
    dist.barrier(group=group)
    t = raw[:_numel(shape) * es].view(dtype).view(*shape)
    return SingleOwnerTensor(t, owner, heap=heap, mapping=mapping_for_self, group=group)
