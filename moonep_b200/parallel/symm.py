"""Symmetric memory: one chunk per rank, all chunks mapped contiguously on every rank.

``SymmetricHeap.create`` is the multi-process path (CUDA VMM + fd / fabric handle
exchange, native code in csrc/host/symm_heap.cc and ipc_exchange.cc; reference
behaviour: moonep/buffer.py:25-410).  ``SymmetricHeap.local`` is the single-process path
used when one process hosts all R ranks on one GPU (tests, CPU-less emulation of the
multi-rank logic): the "mapping" is one ordinary allocation of ``R * chunk`` bytes.

Handle type policy (``MOONEP_MEM_HANDLE_TYPE`` = auto | fabric | fd): ``auto`` picks fabric
handles only if every rank of the group can export them, else POSIX fds passed over unix
sockets.
"""

from __future__ import annotations

import ctypes as C
import logging
import os
import shutil
import tempfile

import torch
import torch.distributed as dist

from .. import _native
from ..geometry import align_up

logger = logging.getLogger(__name__)

HANDLE_FD, HANDLE_FABRIC = 0, 1
IPC_TIMEOUT_MS = 120_000


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """Non-owning uint8 tensor over raw device memory, labelled with ``device`` (peer
    chunks are physically remote but addressed from this device)."""
    storage = torch._C._construct_storage_from_data_pointer(ptr, device, nbytes)
    return torch.empty(0, dtype=torch.uint8, device=device).set_(storage, 0, (nbytes,), (1,))


def _all_gather_bytes(payload: bytes, group) -> list[bytes]:
    world = dist.get_world_size(group)
    out = [None] * world
    dist.all_gather_object(out, payload, group=group)
    return out


def resolve_handle_kind(device_index: int, group) -> int:
    mode = os.environ.get("MOONEP_MEM_HANDLE_TYPE", "auto").lower()
    if mode not in ("auto", "fabric", "fd"):
        raise ValueError(f"MOONEP_MEM_HANDLE_TYPE must be auto|fabric|fd, got {mode!r}")
    if mode == "fd":
        return HANDLE_FD
    lib = _native.load()
    ok = C.c_int(0)
    _native.check(lib.mep_fabric_supported(device_index, C.byref(ok)), "fabric probe")
    flags = _all_gather_bytes(bytes([ok.value]), group)
    everyone = all(f == b"\x01" for f in flags)
    if mode == "fabric":
        if not everyone:
            raise RuntimeError("MOONEP_MEM_HANDLE_TYPE=fabric but not every rank can export fabric handles")
        return HANDLE_FABRIC
    return HANDLE_FABRIC if everyone else HANDLE_FD


def vmm_granularity(device_index: int, kind: int | None = None) -> int:
    """Recommended mapping granularity; with ``kind=None`` the max over fd and fabric."""
    lib = _native.load()
    kinds = (HANDLE_FD, HANDLE_FABRIC) if kind is None else (kind,)
    best = 0
    for k in kinds:
        g = C.c_size_t(0)
        if lib.mep_vmm_granularity(device_index, k, C.byref(g)) == 0:
            best = max(best, g.value)
    if best == 0:
        raise _native.MoonEPNativeError("could not query the VMM granularity")
    return best


def pad_to_granularity(nbytes: int, device_index: int) -> int:
    return align_up(nbytes, vmm_granularity(device_index))


def pad_dim0_for_alignment(shape, dtype: torch.dtype, device_index: int | None = None) -> int:
    """Smallest dim-0 >= shape[0] whose chunk size is a multiple of the VMM granularity."""
    device_index = torch.cuda.current_device() if device_index is None else device_index
    gran = vmm_granularity(device_index)
    row = int(torch.tensor([], dtype=dtype).element_size())
    for s in shape[1:]:
        row *= int(s)
    n = int(shape[0])
    while (n * row) % gran:
        n += 1
        if n > shape[0] + gran:
            raise ValueError("cannot align dim 0 to the VMM granularity")
    return n


def exchange_fds(my_fd: int, group) -> list[int]:
    """All-to-all of file descriptors inside one node (SCM_RIGHTS over unix sockets)."""
    lib = _native.load()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [tempfile.mkdtemp(prefix="mep_ipc_") if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    path = box[0]
    ep = C.c_void_p()
    fds = (C.c_int * world)()
    try:
        _native.check(lib.mep_ipc_open(path.encode(), rank, world, C.byref(ep)), "ipc open")
        dist.barrier(group=group)            # every socket is bound
        _native.check(lib.mep_ipc_send_all(ep, my_fd), "ipc send")
        _native.check(lib.mep_ipc_recv_all(ep, fds, IPC_TIMEOUT_MS), "ipc recv")
        dist.barrier(group=group)            # everyone received everything
    finally:
        if ep:
            lib.mep_ipc_close(ep)
        if rank == 0:
            shutil.rmtree(path, ignore_errors=True)
    return list(fds)


class SymmetricHeap:
    """R chunks of ``chunk_bytes`` each; rank r's chunk starts at ``base + r*chunk_bytes``."""

    def __init__(self):
        self.base = 0
        self.chunk_bytes = 0
        self.world = 1
        self.rank = 0
        self.device = None
        self.mc_base = 0
        self._whole = None        # uint8 tensor over all chunks
        self._mapping = None
        self._chunk = None
        self._mc = None
        self._local_storage = None
        self.closed = False

    # -- single process, all ranks on one device
    @classmethod
    def local(cls, world: int, chunk_bytes: int, device) -> "SymmetricHeap":
        h = cls()
        h.world, h.rank, h.device = world, 0, torch.device(device)
        h.chunk_bytes = align_up(chunk_bytes, 1024)
        h._local_storage = torch.zeros(world * h.chunk_bytes, dtype=torch.uint8, device=h.device)
        h._whole = h._local_storage
        h.base = h._whole.data_ptr()
        return h

    # -- one process per rank
    @classmethod
    def create(cls, chunk_bytes: int, group=None, multicast: bool = False) -> "SymmetricHeap":
        lib = _native.load()
        h = cls()
        h.world, h.rank = dist.get_world_size(group), dist.get_rank(group)
        dev = torch.cuda.current_device()
        h.device = torch.device("cuda", dev)
        kind = resolve_handle_kind(dev, group)
        gran = vmm_granularity(dev)
        if multicast:
            mg = C.c_size_t(0)
            if lib.mep_multicast_granularity(dev, h.world, kind, align_up(chunk_bytes, gran), C.byref(mg)) == 0:
                gran = max(gran, mg.value)
        h.chunk_bytes = align_up(chunk_bytes, gran)
        sizes = _all_gather_bytes(h.chunk_bytes.to_bytes(8, "little"), group)
        if any(s != sizes[0] for s in sizes):
            raise RuntimeError("symmetric heap: ranks disagree on the chunk size "
                               f"({[int.from_bytes(s, 'little') for s in sizes]})")
        chunk = C.c_void_p()
        share = (C.c_ubyte * 64)()
        _native.check(lib.mep_chunk_create(dev, h.chunk_bytes, kind, C.byref(chunk), share), "chunk create")  # argtypes: size_t
        h._chunk = chunk
        my_fd = -1
        try:
            table = (C.c_ubyte * (64 * h.world))()
            # fd handles: mep_map_all consumes (closes) every descriptor of the table, including the copy
            # of this rank's own descriptor that the exchange delivered back in entry [rank]
            if kind == HANDLE_FABRIC:
                blobs = _all_gather_bytes(bytes(share), group)
                for i, b in enumerate(blobs):
                    if len(b) != 64:
                        raise RuntimeError(f"rank {i} sent a fabric handle of {len(b)} bytes, expected 64")
                    C.memmove(C.addressof(table) + 64 * i, b, 64)
            else:
                my_fd = int.from_bytes(bytes(share[:4]), "little", signed=True)
                fds = exchange_fds(my_fd, group)
                for i, fd in enumerate(fds):
                    C.memmove(C.addressof(table) + 64 * i, int(fd).to_bytes(4, "little", signed=True), 4)
            mapping = C.c_void_p()
            base = C.c_ulonglong(0)
            _native.check(lib.mep_map_all(dev, h.world, h.rank, chunk, table, C.byref(mapping), C.byref(base)), "map_all")
            h._mapping, h.base = mapping, base.value
        except Exception:
            lib.mep_chunk_release(chunk)
            h._chunk = None
            raise
        finally:
            if my_fd >= 0:
                lib.mep_close_fd(my_fd)
        h._whole = tensor_from_ptr(h.base, h.world * h.chunk_bytes, h.device)
        h.local_bytes().zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        if multicast:
            h._try_multicast(kind, group)
        return h

    def _try_multicast(self, kind: int, group) -> None:
        """Bind the chunks to an NVSwitch multicast object (optional; failures fall back to
        plain peer stores and are logged, unlike the reference's hard assert, buffer.py:308)."""
        lib = _native.load()
        dev = self.device.index
        ok = C.c_int(0)
        lib.mep_multicast_supported(dev, C.byref(ok))
        flags = _all_gather_bytes(bytes([1 if ok.value else 0]), group)
        if not all(f == b"\x01" for f in flags) or self.world < 2:
            return
        mc = C.c_void_p()
        share = (C.c_ubyte * 64)()
        rc = 0
        if self.rank == 0:
            rc = lib.mep_mc_create(dev, self.world, self.chunk_bytes, kind, C.byref(mc), share)
        oks = _all_gather_bytes(bytes([1 if rc == 0 else 0]), group)
        if oks[0] != b"\x01":
            logger.warning("multicast object creation failed on the root; using peer stores")
            return
        if kind == HANDLE_FABRIC:
            blob = _all_gather_bytes(bytes(share), group)[0]
            if self.rank != 0:
                buf = (C.c_ubyte * 64).from_buffer_copy(blob)
                rc = lib.mep_mc_import(dev, self.chunk_bytes, kind, buf, C.byref(mc))
        else:
            # all-to-all of descriptors; only the root's matters, the others send a placeholder
            send_fd = (int.from_bytes(bytes(share[:4]), "little", signed=True) if self.rank == 0
                       else os.open(os.devnull, os.O_RDONLY))
            try:
                fds = exchange_fds(send_fd, group)
            finally:
                lib.mep_close_fd(send_fd)
            for i, fd in enumerate(fds):
                if i != 0 or self.rank == 0:
                    lib.mep_close_fd(fd)
            if self.rank != 0:
                buf = (C.c_ubyte * 64)()
                C.memmove(buf, int(fds[0]).to_bytes(4, "little", signed=True), 4)
                rc = lib.mep_mc_import(dev, self.chunk_bytes, kind, buf, C.byref(mc))   # closes the fd
        good = rc == 0 and lib.mep_mc_add_device(mc) == 0
        oks = _all_gather_bytes(bytes([1 if good else 0]), group)      # doubles as the barrier before binding
        if not all(o == b"\x01" for o in oks):
            if mc:
                lib.mep_mc_destroy(mc)
            logger.warning("multicast setup failed on some rank; using peer stores")
            return
        va = C.c_ulonglong(0)
        good = lib.mep_mc_bind_map(mc, self._chunk, C.byref(va)) == 0
        oks = _all_gather_bytes(bytes([1 if good else 0]), group)
        self._mc = mc
        if all(o == b"\x01" for o in oks):
            self.mc_base = va.value
        else:
            logger.warning("multicast bind failed on some rank; using peer stores")

    # -- views
    def whole(self) -> torch.Tensor:
        return self._whole

    def chunk(self, rank: int) -> torch.Tensor:
        return self._whole[rank * self.chunk_bytes:(rank + 1) * self.chunk_bytes]

    def local_bytes(self, rank: int | None = None) -> torch.Tensor:
        return self.chunk(self.rank if rank is None else rank)

    def view(self, rank: int, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.tensor([], dtype=dtype).element_size()
        return self.chunk(rank)[offset:offset + nbytes].view(dtype).view(*shape)

    def strided_view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """``[R, *shape]`` view of the same sub-buffer on every rank (rank stride = chunk)."""
        es = torch.tensor([], dtype=dtype).element_size()
        assert offset % es == 0 and self.chunk_bytes % es == 0
        flat = self._whole.view(dtype)
        strides, acc = [], 1
        for s in reversed(shape):
            strides.append(acc)
            acc *= int(s)
        strides = [self.chunk_bytes // es] + list(reversed(strides))
        return flat.as_strided((self.world, *shape), strides, offset // es)

    def close(self) -> None:
        """Release mappings. Caller has synchronised the device and (multi-process)
        barriered; views must not be used afterwards."""
        if self.closed:
            return
        self.closed = True
        self._whole = None
        self._local_storage = None
        if self._mapping is not None or self._chunk is not None or self._mc is not None:
            lib = _native.load()
            if self._mc is not None:
                lib.mep_mc_destroy(self._mc)
                self._mc = None
            if self._mapping is not None:
                lib.mep_unmap_all(self._mapping)
                self._mapping = None
            if self._chunk is not None:
                lib.mep_chunk_release(self._chunk)
                self._chunk = None
