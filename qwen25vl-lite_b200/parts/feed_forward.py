"""SwiGLU feed-forward: ``down(silu(gate x) * up x)``, no biases
(reference src/qwen25vl_lite/text.py:56-66).  gate and up are held as one matrix so one
product feeds the activation; in the decode kernel the activation is its epilogue."""

from __future__ import annotations

import torch

from ..ops import kernels, linear
from ..ops.linear import DeferredNorm, Linear
from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_deferred_norm = True     # forward takes a DeferredNorm as its input
    accepts_residual = True          # forward can add its result into the residual stream itself

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.gate_up_proj = None
        self.down_proj = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return (TensorSpec("gate_proj.weight", (i, h)), TensorSpec("up_proj.weight", (i, h)),
                TensorSpec("down_proj.weight", (h, i)))

    def load(self, tensors, device, dtype):
        gate, up = tensors["gate_proj.weight"].to(device), tensors["up_proj.weight"].to(device)
        self.paired = self.intermediate_size % 8 == 0
        if self.paired:
            # rows in groups of 16: 8 gate features, then their 8 up features, so that the
            # weight-streaming kernel can form silu(gate) * up in its epilogue
            h = self.hidden_size
            gu = torch.stack([gate.reshape(-1, 8, h), up.reshape(-1, 8, h)], dim=1).reshape(2 * self.intermediate_size, h)
        else:
            gu = torch.cat([gate, up], dim=0)
        self.gate_up_proj = Linear(gu.to(dtype=dtype).contiguous())
        self.down_proj = Linear(tensors["down_proj.weight"].to(device=device, dtype=dtype).contiguous())

    def forward(self, ctx, h, residual=None):
        """Returns the update of the residual stream, or None after adding it into ``residual``."""
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=ctx.dtype, device=h.device)
        w = self.gate_up_proj.weight
        deferred = isinstance(h, DeferredNorm)
        if self.paired and deferred and kernels.gemm_skinny_norm_supports(h.x, w):
            kernels.gemm_skinny_norm(h.x, h.weight, h.eps, w, None, act, kernels.SKINNY_SWIGLU)
        else:
            if deferred:
                h = h.materialize()
            if self.paired and kernels.gemm_skinny_supports(h, w):
                kernels.gemm_skinny(h, w, None, act, kernels.SKINNY_SWIGLU)
            elif self.paired and linear.use_tcgen05(h, w, fused_epilogue=True):
                kernels.gemm_tcgen05(h, w, None, act, kernels.SKINNY_SWIGLU)
            else:
                kernels.silu_mul(self.gate_up_proj(h), act, self.paired)
        return self.down_proj(act, residual=residual)
