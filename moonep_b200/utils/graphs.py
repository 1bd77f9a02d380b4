"""CUDA-graph capture of whole training steps.

Every kernel of this package keeps its launch-to-launch state in device memory (barrier epochs,
the planner's epoch, tile ticket counters), launches on the current stream and never synchronises
with the host, so a complete step -- routing, dispatch, grouped GEMMs, combine, gradient
reduction, optimizer, including the work forked onto the communication and side streams -- can be
captured once and replayed with a single launch per step.  That removes the per-kernel launch
cost of the ~100 kernels of a step from the host's critical path.
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedSteps:
    """``step_fn(x) -> loss`` captured once per static input buffer.

    ``inputs`` are the device tensors the steps read (typically two, so that the next batch can
    be copied in while a step runs); ``replay(i)`` runs the step on ``inputs[i]`` and leaves its
    loss in ``losses[i]`` (device) and, asynchronously, in ``host_losses[i]`` (pinned).  The graphs
    share one memory pool and must be replayed one after the other on one stream.
    Run a few eager warm-up steps before constructing this object.
    """

    def __init__(self, step_fn: Callable[..., torch.Tensor], inputs: Sequence[torch.Tensor],
                 health: Callable[[], None] | None = None, host_inputs: Sequence[torch.Tensor] | None = None,
                 pool=None):
        """``health``: called before every replay; it should raise if an earlier replay recorded a
        device-side failure (e.g. ``lambda: (buf.healthy() or buf.check())``).  Such checks read a
        flag in host memory, so they cost nothing and do not synchronise.

        ``host_inputs`` (pinned host tensors, one per input buffer): the step on ``inputs[i]`` also copies
        ``host_inputs[i+1]`` into ``inputs[i+1]`` on a side stream inside the same graph, i.e. every replay
        brings in the batch of the next one (the caller refills the pinned buffer in between and copies the
        very first batch itself).  ``step_fn`` is then called as ``step_fn(x, stage_next)`` and decides
        where in the step the copy starts by calling ``stage_next()`` (at the end if it never does): a
        host-to-device copy slows kernels that use system-scope fences while it runs, so it belongs beside
        local work (the optimizer, weight-gradient GEMMs), not beside dispatch or combine.
        ``pool``: memory pool of an earlier ``GraphedSteps`` to share (the two must not replay concurrently)."""
        self.health = health
        self.inputs = list(inputs)
        self.graphs, self.losses, self.host_losses = [], [], []
        side = torch.cuda.Stream() if host_inputs is not None else None
        for i, x in enumerate(self.inputs):
            host = torch.zeros(1, dtype=torch.float32).pin_memory()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                if host_inputs is None:
                    loss = step_fn(x)
                else:
                    staged = []

                    def stage_next(i=i, staged=staged):
                        if staged:
                            return
                        staged.append(True)
                        nxt = (i + 1) % len(self.inputs)
                        side.wait_stream(torch.cuda.current_stream())
                        with torch.cuda.stream(side):
                            self.inputs[nxt].detach().copy_(host_inputs[nxt], non_blocking=True)

                    loss = step_fn(x, stage_next)
                    stage_next()
                    torch.cuda.current_stream().wait_stream(side)
                host.copy_(loss.detach().reshape(1).float(), non_blocking=True)
            pool = g.pool()
            self.graphs.append(g)
            self.losses.append(loss)
            self.host_losses.append(host)
        self.pool = pool

    def __len__(self) -> int:
        return len(self.graphs)

    def replay(self, i: int) -> None:
        if self.health is not None:
            self.health()
        self.graphs[i % len(self.graphs)].replay()
