"""The synthetic training loss of the step benchmarks, shared by both arms: mean(y^2) over the
layer output, with the gradient returned in the output's dtype.  Written as one autograd function
so that it costs two passes over ``y`` (a norm and a scale) instead of the seven elementwise
kernels of ``(y.float() ** 2).mean()`` -- the loss is harness, not the thing being measured."""

import torch


class _MeanSquare(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y):
        ctx.save_for_backward(y)
        n = torch.linalg.vector_norm(y.reshape(-1), dtype=torch.float32)
        return n * n / y.numel()

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        return y * (g * (2.0 / y.numel()))        # fp32 scalar x bf16 tensor -> bf16, fp32 arithmetic


def mean_square(y: torch.Tensor) -> torch.Tensor:
    return _MeanSquare.apply(y)
