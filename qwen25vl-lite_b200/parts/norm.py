"""RMS normalisation fused with the residual update.

Formula (reference src/qwen25vl_lite/layers.py:27-31): ``x * rsqrt(mean(x^2) + eps) * w``,
statistics in float32, plain (not 1 + w) weight.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import DeferredNorm
from .base import Norm, TensorSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, dim: int, eps: float):
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight = None

    def tensor_specs(self):
        return (TensorSpec("weight", (self.dim,), init="norm"),)

    def load(self, tensors, device, dtype):
        self.weight = tensors["weight"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, ctx, x, delta, rows=None, defer=False):
        """``defer``: the caller's consumer can normalise inside its own kernel; when nothing
        has to be added first and the step is small enough for that kernel, no kernel is
        launched here and a ``DeferredNorm`` is returned instead of the activation."""
        if (defer and delta is None and rows is None and ctx.dtype == torch.bfloat16
                and x.shape[0] <= kernels.SKINNY_MAX_ROWS):
            return DeferredNorm(x, self.weight, self.eps, ctx.dtype)
        n_out = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_out, self.dim), dtype=ctx.dtype, device=x.device)
        kernels.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        return out
