"""Communication plan produced by a fresh ``Buffer.dispatch``.

Same fields, shapes and encodings as the reference's ``MoonEPCommPlan``
(moonep/planning.py:31-86) so a saved plan can drive prefetch, combine and both
backward passes.

Encodings
---------
``dst[i]`` for flat top-k entry ``i = s*K + k``:
    ``d*NvS + loff`` when this entry is the *primary* (lowest ``k``) of token
    ``s`` on destination rank ``d``; ``-(d*NvS + loff) - 1`` when an earlier
    ``k`` of the same token already goes to rank ``d`` (duplicate: the payload
    is not re-sent, the destination expands it locally).
``experts_to_copy[d, b]``: global id of the redundant expert held in prefetch
    slot ``b`` of rank ``d`` or -1; identical on every rank.
``zero_fill_ranges[g] = (first_pad_row, n_pad_rows)`` of VM group ``g`` on this
    rank (``(0, 0)`` when there is nothing to clear).
``remote_stats = [#redundant experts received, #slots this rank's experts occupy
    elsewhere]``.
``dup_groups[j] = (primary_loff, start, n)`` with the duplicates of that primary
    row at ``dup_loffs[start:start+n]``; only the first ``dup_counts[0]`` groups
    and ``dup_counts[1]`` offsets are valid and their order is unspecified
    (consumers treat them as a set).
"""

from __future__ import annotations

from dataclasses import dataclass, fields

import torch


@dataclass(frozen=True)
class MoonEPCommPlan:
    dst: torch.Tensor
    experts_to_copy: torch.Tensor
    zero_fill_ranges: torch.Tensor
    remote_stats: torch.Tensor
    N: int
    R: int
    E: int
    NvS: int
    K: int
    dup_groups: torch.Tensor
    dup_loffs: torch.Tensor
    dup_counts: torch.Tensor

    def __post_init__(self) -> None:
        epn = self.E // self.R

        def chk(name, shape):
            t = getattr(self, name)
            assert t.dtype == torch.int32 and t.is_contiguous(), f"plan.{name}: int32 contiguous required"
            assert tuple(t.shape) == shape, f"plan.{name}: expected shape {shape}, got {tuple(t.shape)}"

        chk("dst", (self.N,))
        chk("experts_to_copy", (self.R, epn))
        chk("zero_fill_ranges", (2 * epn, 2))
        chk("remote_stats", (2,))
        chk("dup_groups", (self.NvS, 3))
        chk("dup_loffs", (self.NvS,))
        chk("dup_counts", (2,))

    def tensors(self):
        """The tensor fields, in declaration order (used for record_stream)."""
        return tuple(getattr(self, f.name) for f in fields(self)
                     if isinstance(getattr(self, f.name), torch.Tensor))

    def clone(self) -> "MoonEPCommPlan":
        kw = {}
        for f in fields(self):
            v = getattr(self, f.name)
            kw[f.name] = v.clone() if isinstance(v, torch.Tensor) else v
        return type(self)(**kw)

    def cpu(self) -> "MoonEPCommPlan":
        kw = {}
        for f in fields(self):
            v = getattr(self, f.name)
            kw[f.name] = v.cpu() if isinstance(v, torch.Tensor) else v
        return type(self)(**kw)

    # Plans are plain tensors + ints, so the default dataclass pickling works;
    # these two make the round trip explicit for debugging dumps.
    def __getstate__(self):
        return {f.name: (getattr(self, f.name).cpu() if isinstance(getattr(self, f.name), torch.Tensor)
                         else getattr(self, f.name)) for f in fields(self)}

    def __setstate__(self, state):
        for k, v in state.items():
            object.__setattr__(self, k, v)
