"""Expert weight / gradient pools in symmetric memory.

The communication API takes, per projection (gate, up, down), a local tensor
``[epn, rows, cols]`` and an all-rank view ``[R, epn, rows, cols]`` of every rank's spare
slots; the expert GEMM wants ``[2*epn, rows, cols]`` = local experts followed by this
rank's slots (contract: README.md:45-68 of the reference, which leaves building these
views to the integrating framework; its tests assemble them by hand,
tests/test_e2e.py:50-57).  ``ExpertPools`` allocates ``[local | slots]`` per projection in
one symmetric chunk and hands out all three views, for weights (payload dtype) and, for
training, for gradients (fp32: local grad | reduce slots).

The slots are scratch that only lives from a layer's prefetch to its last GEMM (and from its
weight-gradient GEMM to its reduction), so a model needs them ONCE, not once per layer
(README.md:56 of the reference: the prefetch pool is process-global and shared by all layers).
``SharedSlots`` owns one set of slots; an ``ExpertPools(shared=...)`` then keeps only its own
experts and gradients in private device memory and builds its ``[local | slots]`` compute views by
mapping the shared slots a second time behind them (CUDA virtual-memory aliasing), so the grouped
GEMM still sees one contiguous operand.  A layer whose slots are shared has to prefetch again in
its backward pass (``ExpertParallelMoE`` does).
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _native
from .geometry import align_up
from .parallel.symm import SymmetricHeap, tensor_from_ptr

NAMES = ("gate", "up", "down")


def pool_layout(epn: int, shapes: dict, dtype, with_grads: bool):
    """Byte offsets inside one rank's chunk: per projection ``[local epn | slots epn]`` of the
    payload dtype, then (training) the same in fp32 for the gradients.  Returns
    ``(weight_offsets, grad_offsets, bytes_per_rank)``."""
    es = torch.tensor([], dtype=dtype).element_size()
    off = 0
    woff, goff = {}, {}
    for n in NAMES:
        r, c = shapes[n]
        woff[n] = off
        off = align_up(off + 2 * epn * r * c * es, 1024)
    if with_grads:
        for n in NAMES:
            r, c = shapes[n]
            goff[n] = off
            off = align_up(off + 2 * epn * r * c * 4, 1024)
    return woff, goff, off


def describe_layout(epn: int, shapes: dict, dtype=torch.bfloat16, with_grads: bool = True, world: int = 8) -> str:
    """Text diagram of the pools of one rank and of the three views the API takes (the
    counterpart of the reference's weight_buffer / grad_buffer figures,
    figure/generate_buffer_figures.py there).  Needs no GPU."""
    woff, goff, total = pool_layout(epn, shapes, dtype, with_grads)
    es = torch.tensor([], dtype=dtype).element_size()
    dn = str(dtype).replace("torch.", "")
    mib = lambda b: f"{b / 2**20:9.1f} MiB"  # noqa: E731
    lines = [f"one rank's chunk of the symmetric heap: {mib(total).strip()} "
             f"(same layout on each of the {world} ranks; rank stride = chunk size)", ""]

    def block(title, offs, esize, tname, local, slots):
        lines.append(title)
        for n in NAMES:
            r, c = shapes[n]
            half = epn * r * c * esize
            lines.append(f"  {n:<5} @ {offs[n]:>14,d}  | {local} [{epn}, {r}, {c}] {tname} {mib(half)} "
                         f"| {slots} [{epn}, {r}, {c}] {tname} {mib(half)} |")
        lines.append("")

    block("weights", woff, es, dn, "local experts", "prefetch slots")
    if with_grads:
        block("gradients", goff, 4, "float32", "local grads  ", "reduce slots  ")
    r, c = shapes[NAMES[0]]
    lines += [
        "views (per projection):",
        f"  compute  [2*epn={2 * epn}, rows, cols]   local experts followed by this rank's slots -> grouped GEMM operand,",
        "           indexed by the VM group g of cu_seqlens: g < epn local expert g, g >= epn slot g - epn",
        f"  prefetch [R={world}, epn={epn}, rows, cols]  every rank's prefetch slots through one mapping -> Buffer.prefetch_weight",
        f"  reduce   [R={world}, epn={epn}, rows, cols]  every rank's fp32 reduce slots                   -> Buffer.reduce_grad",
        f"  (slot b of rank d holds expert plan.experts_to_copy[d, b]; e.g. one {NAMES[0]} matrix = "
        f"{mib(r * c * es).strip()} {dn}, {mib(r * c * 4).strip()} fp32)",
    ]
    return "\n".join(lines)


class SharedSlots:
    """One set of prefetch slots (and, for training, fp32 reduce slots) for ALL layers of a model:
    per projection a symmetric heap whose chunk is ``[epn, rows, cols]``.  Needs a process group with
    more than one rank (a single rank never replicates an expert)."""

    def __init__(self, epn: int, gate_shape, up_shape, down_shape, dtype=torch.bfloat16, group=None,
                 with_grads: bool = False):
        assert dist.is_initialized() and dist.get_world_size(group) > 1, "SharedSlots needs an EP group of 2 or more ranks"
        self.epn, self.dtype, self.with_grads, self._group = epn, dtype, with_grads, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.shapes = dict(zip(NAMES, (tuple(gate_shape), tuple(up_shape), tuple(down_shape))))
        es = torch.tensor([], dtype=dtype).element_size()
        self.weight_heaps, self.grad_heaps = {}, {}
        for n in NAMES:
            r, c = self.shapes[n]
            self.weight_heaps[n] = SymmetricHeap.create(epn * r * c * es, group=group)
            if with_grads:
                self.grad_heaps[n] = SymmetricHeap.create(epn * r * c * 4, group=group)
        self.bytes_per_rank = sum(h.chunk_bytes for h in (*self.weight_heaps.values(), *self.grad_heaps.values()))

    def prefetch_view(self, name) -> torch.Tensor:
        return self.weight_heaps[name].strided_view(0, (self.epn, *self.shapes[name]), self.dtype)

    def reduce_view(self, name) -> torch.Tensor:
        return self.grad_heaps[name].strided_view(0, (self.epn, *self.shapes[name]), torch.float32)

    def destroy(self) -> None:
        """Collective.  Every ``ExpertPools`` built on these slots must have been destroyed before."""
        if self.weight_heaps:
            torch.cuda.synchronize()
            if dist.is_initialized():
                dist.barrier(group=self._group)
            for h in (*self.weight_heaps.values(), *self.grad_heaps.values()):
                h.close()
            self.weight_heaps, self.grad_heaps = {}, {}


class ExpertPools:
    def __init__(self, epn: int, gate_shape, up_shape, down_shape, dtype=torch.bfloat16, group=None,
                 with_grads: bool = False, world: int | None = None, rank: int | None = None,
                 heap: SymmetricHeap | None = None, device=None, shared: SharedSlots | None = None):
        """``*_shape`` = (rows, cols) of one expert's matrix.  With ``world``/``rank``/``heap``
        given explicitly the pools live in an existing (e.g. single-process) heap.  With ``shared``
        the slots are those of a ``SharedSlots`` (one set for all layers) and only the local experts
        and gradients are allocated here."""
        self.epn = epn
        self.dtype = dtype
        self.with_grads = with_grads
        self._shapes = dict(zip(NAMES, (tuple(gate_shape), tuple(up_shape), tuple(down_shape))))
        if world is None:
            if dist.is_initialized():
                world, rank = dist.get_world_size(group), dist.get_rank(group)
            else:
                world, rank = 1, 0
        self.world, self.rank, self._group = world, rank, group
        self.shared = shared
        self._aliases, self._wview, self._gview = [], {}, {}
        if shared is not None:
            assert heap is None and shared.world == world and shared.epn == epn and shared.dtype == dtype
            assert shared.shapes == self._shapes and (shared.with_grads or not with_grads)
            self._map_behind_shared(device)
            return
        self._woff, self._goff, off = pool_layout(epn, self._shapes, dtype, with_grads)
        self._own_heap = heap is None
        if heap is None:
            if world > 1:
                heap = SymmetricHeap.create(off, group=group)
            else:
                heap = SymmetricHeap.local(1, off, device or torch.device("cuda", torch.cuda.current_device()))
        else:
            assert heap.chunk_bytes >= off, "heap chunk too small for the pools"
        self.heap = heap
        self.bytes_per_rank = off

    def _map_behind_shared(self, device) -> None:
        """Per projection: new physical memory for the local experts (gradients), the shared slot chunk
        mapped right behind it -> one contiguous ``[2*epn, rows, cols]`` compute view."""
        lib = _native.load()
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.heap, self._own_heap, self.bytes_per_rank = None, False, 0
        es = torch.tensor([], dtype=self.dtype).element_size()
        for kind, heaps, esz, dt, views in (("w", self.shared.weight_heaps, es, self.dtype, self._wview),
                                            ("g", self.shared.grad_heaps if self.with_grads else {}, 4, torch.float32, self._gview)):
            for n, h in heaps.items():
                r, c = self._shapes[n]
                local_bytes = self.epn * r * c * esz
                alias, va = C.c_void_p(), C.c_ulonglong(0)
                _native.check(lib.mep_alias_map(dev.index, local_bytes, h._chunk, C.byref(alias), C.byref(va)),
                              f"shared slots: compute view of {n} ({'weights' if kind == 'w' else 'grads'})")
                self._aliases.append(alias)
                raw = tensor_from_ptr(va.value, 2 * local_bytes, dev)
                views[n] = raw.view(dt).view(2 * self.epn, r, c)
                views[n][:self.epn].zero_()
                self.bytes_per_rank += local_bytes

    def shape(self, name):
        return self._shapes[name]

    def describe(self) -> str:
        """Text diagram of this allocation (see ``describe_layout``)."""
        return describe_layout(self.epn, self._shapes, self.dtype, self.with_grads, self.world)

    def _view(self, off, name, dtype, first, count, rank=None):
        r, c = self._shapes[name]
        es = torch.tensor([], dtype=dtype).element_size()
        rank = self.rank if rank is None else rank
        return self.heap.view(rank, off + first * r * c * es, (count, r, c), dtype)

    # ---- weights
    def local_weight(self, name, rank=None) -> torch.Tensor:
        if self.shared is not None:
            return self._wview[name][:self.epn]
        return self._view(self._woff[name], name, self.dtype, 0, self.epn, rank)

    def compute_weight(self, name, rank=None) -> torch.Tensor:
        """``[2*epn, rows, cols]``: local experts then this rank's prefetch slots."""
        if self.shared is not None:
            return self._wview[name]
        return self._view(self._woff[name], name, self.dtype, 0, 2 * self.epn, rank)

    def prefetch_view(self, name) -> torch.Tensor:
        """``[R, epn, rows, cols]`` view of every rank's prefetch slots."""
        if self.shared is not None:
            return self.shared.prefetch_view(name)
        r, c = self._shapes[name]
        es = torch.tensor([], dtype=self.dtype).element_size()
        return self.heap.strided_view(self._woff[name] + self.epn * r * c * es, (self.epn, r, c), self.dtype)

    # ---- grads
    def local_grad(self, name, rank=None) -> torch.Tensor:
        if self.shared is not None:
            return self._gview[name][:self.epn]
        return self._view(self._goff[name], name, torch.float32, 0, self.epn, rank)

    def compute_grad(self, name, rank=None) -> torch.Tensor:
        if self.shared is not None:
            return self._gview[name]
        return self._view(self._goff[name], name, torch.float32, 0, 2 * self.epn, rank)

    def reduce_view(self, name) -> torch.Tensor:
        if self.shared is not None:
            return self.shared.reduce_view(name)
        r, c = self._shapes[name]
        return self.heap.strided_view(self._goff[name] + self.epn * r * c * 4, (self.epn, r, c), torch.float32)

    # ---- keyword bundles for Buffer.prefetch_weight / Buffer.reduce_grad
    def prefetch_kwargs(self, rank=None) -> dict:
        kw = {}
        for n in NAMES:
            kw[f"local_{n}_weight"] = self.local_weight(n, rank)
            kw[f"{n}_prefetch_buffer"] = self.prefetch_view(n)
        return kw

    def reduce_kwargs(self, rank=None) -> dict:
        kw = {}
        for n in NAMES:
            kw[f"local_{n}_grad"] = self.local_grad(n, rank)
            kw[f"{n}_reduce_buffer"] = self.reduce_view(n)
        return kw

    def destroy(self) -> None:
        if self._aliases:
            torch.cuda.synchronize()
            self._wview, self._gview = {}, {}
            lib = _native.load()
            for a in self._aliases:
                lib.mep_alias_unmap(a)
            self._aliases = []
        if self.heap is not None and self._own_heap:
            torch.cuda.synchronize()
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self._group)
            self.heap.close()
        self.heap = None


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="print the expert pool layout of one rank")
    ap.add_argument("--epn", type=int, default=32)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--R", type=int, default=8)
    ap.add_argument("--no-grads", action="store_true")
    a = ap.parse_args()
    print(describe_layout(a.epn, {"gate": (a.H, a.Hp), "up": (a.H, a.Hp), "down": (a.Hp, a.H)},
                          with_grads=not a.no_grads, world=a.R))
