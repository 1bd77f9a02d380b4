"""All R ranks of an EP group hosted by ONE process on ONE GPU.

Every native kernel takes a list of rank contexts and runs them as the y-dimension of a
single cooperative launch, so cross-rank barriers, peer stores and peer loads behave as on R
GPUs (peer memory is simply another region of the same device).  This is how the multi-rank
logic is tested when only one GPU is available; it is not a performance path.
"""

from __future__ import annotations

import torch

from .. import engine
from ..api import OpsMixin
from ..geometry import Geometry, MAX_VRANKS
from ..parallel.symm import SymmetricHeap


class LocalCluster(OpsMixin):
    def __init__(self, S, H, K, E, R, num_sms=4, token_padding=128, device="cuda:0", num_sms_dedup=8,
                 budget_ms: float | None = None, push_combine: bool = False, enable_pdl: bool = True):
        assert 1 <= R <= MAX_VRANKS, f"LocalCluster hosts at most {MAX_VRANKS} ranks"
        self.geo = Geometry.make(S, H, K, E, R, token_padding, num_sms, push_combine=push_combine)
        self.device = torch.device(device)
        self.heap = SymmetricHeap.local(R, self.geo.chunk_bytes, self.device)
        bn = None if budget_ms is None else int(budget_ms * 1e6)
        self._states = [engine.make_rank_state(self.geo, r, self.heap, self.device, bn) for r in range(R)]
        self._num_sms_dedup = num_sms_dedup
        self.R = R
        self.enable_pdl = enable_pdl

    def dispatch(self, hidden, weights=None, topk=None, tpe=None, plans=None, *, inter_rank_sync=True,
                 zero_copy=False, router_weights_zero_copy=False):
        return self._dispatch_lists(hidden, weights, topk, tpe, plans, inter_rank_sync=inter_rank_sync,
                                    zero_copy=zero_copy, w_zero_copy=router_weights_zero_copy)

    def dispatch_ready(self, hidden, weights=None, topk=None, tpe=None, plans=None, *, inter_rank_sync=True,
                       same_stream=False):
        """Flagged dispatch of all hosted ranks (one launch); see ``Buffer.dispatch_ready``."""
        if getattr(self, "_comm_stream", None) is None:
            self._comm_stream = torch.cuda.Stream(device=self.device)
        return self._dispatch_ready_lists(hidden, weights, topk, tpe, plans, None if same_stream else self._comm_stream,
                                          inter_rank_sync=inter_rank_sync)

    def tile_ready(self, rank: int):
        return self._tile_ready(rank)

    def slot_ready(self, rank: int):
        return self._slot_ready(rank)

    def combine(self, plans, hidden_nvsh, weights_nvs=None, *, inter_rank_sync=True, zero_copy=False,
                router_weights_zero_copy=False):
        return self._combine_lists(plans, hidden_nvsh, weights_nvs, inter_rank_sync=inter_rank_sync,
                                   zero_copy=zero_copy, w_zero_copy=router_weights_zero_copy)

    def push_target(self, rank: int):
        return self._push_target(rank)

    def combine_pushed(self, want_weights: bool = False):
        return self._push_reduce_lists(want_weights)

    def prefetch(self, plans, pairs_list):
        self._prefetch_lists(plans, pairs_list)

    def reduce_grad(self, plans, pairs_list, inter_rank_sync=True, clear_slots=True):
        self._reduce_lists(plans, pairs_list, inter_rank_sync, clear_slots)

    def check(self):
        for s in self._states:
            st = engine.read_status(s)
            if st is not None:
                raise engine.MoonEPTimeout(st)

    def make_pool(self, shape_per_rank, dtype, pad_elems=0):
        """``[R, *shape]`` pool on this device with an optional gap between ranks."""
        n = 1
        for s in shape_per_rank:
            n *= int(s)
        stride = n + pad_elems
        flat = torch.zeros(self.R * stride, dtype=dtype, device=self.device)
        strides, acc = [], 1
        for s in reversed(shape_per_rank):
            strides.append(acc)
            acc *= int(s)
        return flat.as_strided((self.R, *shape_per_rank), [stride] + list(reversed(strides))), flat
