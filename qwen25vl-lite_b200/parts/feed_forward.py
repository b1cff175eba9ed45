"""SwiGLU feed-forward: ``down(silu(gate x) * up x)``, no biases
(reference src/qwen25vl_lite/text.py:56-66).  gate and up are held as one matrix so one
product feeds the activation kernel."""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import Linear
from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.gate_up_proj = None
        self.down_proj = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return (TensorSpec("gate_proj.weight", (i, h)), TensorSpec("up_proj.weight", (i, h)),
                TensorSpec("down_proj.weight", (h, i)))

    def load(self, tensors, device, dtype):
        gu = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0)
        self.gate_up_proj = Linear(gu.to(device=device, dtype=dtype).contiguous())
        self.down_proj = Linear(tensors["down_proj.weight"].to(device=device, dtype=dtype).contiguous())

    def forward(self, ctx, h):
        gu = self.gate_up_proj(h)
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=h.dtype, device=h.device)
        kernels.silu_mul(gu, act)
        return self.down_proj(act)
