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

    def __init__(self, step_fn: Callable[[torch.Tensor], torch.Tensor], inputs: Sequence[torch.Tensor],
                 health: Callable[[], None] | None = None):
        """``health``: called before every replay; it should raise if an earlier replay recorded a
        device-side failure (e.g. ``lambda: (buf.healthy() or buf.check())``).  Such checks read a
        flag in host memory, so they cost nothing and do not synchronise."""
        self.health = health
        self.inputs = list(inputs)
        self.graphs, self.losses, self.host_losses = [], [], []
        pool = None
        for x in self.inputs:
            host = torch.zeros(1, dtype=torch.float32).pin_memory()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                loss = step_fn(x)
                host.copy_(loss.detach().reshape(1).float(), non_blocking=True)
            pool = g.pool()
            self.graphs.append(g)
            self.losses.append(loss)
            self.host_losses.append(host)

    def __len__(self) -> int:
        return len(self.graphs)

    def replay(self, i: int) -> None:
        if self.health is not None:
            self.health()
        self.graphs[i % len(self.graphs)].replay()
