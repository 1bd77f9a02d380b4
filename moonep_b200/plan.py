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
    # Extension (plans made by ``Buffer.dispatch_ready``; None otherwise): the rows this rank puts on
    # the wire, as entries ``s*K + k``, ordered by (destination tile, destination rank), and
    # ``send_meta = [len(send_list), end of the used part of the local shard, 0, 0]``.
    send_list: torch.Tensor | None = None
    send_meta: torch.Tensor | None = None

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
        if self.send_list is not None or self.send_meta is not None:
            chk("send_list", (self.N,))
            chk("send_meta", (4,))

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


# ---- cross-rank consistency check (debugging aid)
#
# The planner is replicated: every rank solves the same problem from the same exchanged
# histograms and must arrive at the same tables.  A divergence (a tie broken differently, a
# stale histogram) would corrupt routing silently, so a plan can be fingerprinted on each rank
# and the fingerprints compared on the host.

def plan_fingerprint(plan: MoonEPCommPlan, rank: int) -> dict:
    """Host-side summary of ``plan`` as seen by ``rank`` (synchronises; small)."""
    import hashlib
    etc = plan.experts_to_copy.cpu()
    dst = plan.dst.cpu().long()
    raw = torch.where(dst >= 0, dst, -dst - 1)
    dest, loff = raw // plan.NvS, raw % plan.NvS
    epn = plan.E // plan.R
    mine = (etc >= rank * epn) & (etc < (rank + 1) * epn)
    stats = plan.remote_stats.tolist()
    return {
        "rank": rank,
        "etc_sha1": hashlib.sha1(etc.numpy().tobytes()).hexdigest(),
        "rows_to": torch.bincount(dest.clamp(0, plan.R - 1), minlength=plan.R).tolist(),
        "dest_in_range": bool(((dest >= 0) & (dest < plan.R)).all()),
        "max_loff": int(loff.max()) if loff.numel() else -1,
        "received": int((etc[rank] >= 0).sum()), "received_stat": int(stats[0]),
        "sent": int(mine.sum()), "sent_stat": int(stats[1]),
        "N": plan.N, "NvS": plan.NvS,
    }


def compare_fingerprints(fps) -> list[str]:
    """Problems found in the fingerprints of all ranks of one dispatch (empty list = consistent):
    identical redundant-expert tables, statistics that match the table, destinations in range,
    and exactly ``N`` rows arriving on every rank."""
    fps = sorted(fps, key=lambda f: f["rank"])
    errs = []
    if len({f["etc_sha1"] for f in fps}) != 1:
        errs.append("experts_to_copy differs between ranks: " + ", ".join(f"{f['rank']}:{f['etc_sha1'][:8]}" for f in fps))
    for f in fps:
        if not f["dest_in_range"]:
            errs.append(f"rank {f['rank']}: a destination rank is out of range")
        if f["max_loff"] >= f["NvS"]:
            errs.append(f"rank {f['rank']}: slot offset {f['max_loff']} beyond NvS={f['NvS']}")
        if f["received"] != f["received_stat"] or f["sent"] != f["sent_stat"]:
            errs.append(f"rank {f['rank']}: remote_stats ({f['received_stat']}, {f['sent_stat']}) disagree with the "
                        f"slot table ({f['received']}, {f['sent']})")
    R = len(fps)
    if all(len(f["rows_to"]) == R for f in fps):
        for d in range(R):
            got = sum(f["rows_to"][d] for f in fps)
            if got != fps[d]["N"]:
                errs.append(f"rank {d} receives {got} rows, expected exactly {fps[d]['N']}")
    else:
        errs.append("fingerprints come from groups of different sizes")
    return errs
