"""Grouped-query softmax attention over the paged cache.

Reference (src/qwen25vl_lite/text.py:69-185): biased q/k/v projections, no bias on o
(:80-83); position encoding on q and k (:118); the step's k, v go into the pages before
the whole context is read back (:125-147); scores scaled by D^-1/2 (:78), query at
absolute index a sees keys j <= a (src/qwen25vl_lite/attention.py:366-372); query head h
reads kv head h // (nq / nkv) (attention.py:143-148).  ``window`` additionally hides keys
j <= a - window; the reference parses a window (src/qwen25vl_lite/config.py:93-94) but
never applies one.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import attention as attention_ops
from ..ops.linear import Linear
from .base import KVCacheNeed, Mixer, TensorSpec, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position,
                 qkv_bias: bool = True, out_bias: bool = False, window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head size {head_dim} is not supported: the kernels take multiples of 16 up to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.position = position
        self.qkv_bias, self.out_bias = bool(qkv_bias), bool(out_bias)
        self.window = None if not window else int(window)
        self.scale = float(head_dim) ** -0.5
        self.rows_per_token = num_heads // num_kv_heads      # query heads that share one kv head
        self.graph_safe = True                               # forward is a fixed sequence of launches
        self.qkv_proj = None
        self.o_proj = None

    def tensor_specs(self):
        q, kv, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.hidden_size
        specs = [TensorSpec("q_proj.weight", (q, h)), TensorSpec("k_proj.weight", (kv, h)),
                 TensorSpec("v_proj.weight", (kv, h)), TensorSpec("o_proj.weight", (h, q))]
        if self.qkv_bias:
            specs += [TensorSpec("q_proj.bias", (q,), "bias"), TensorSpec("k_proj.bias", (kv,), "bias"),
                      TensorSpec("v_proj.bias", (kv,), "bias")]
        if self.out_bias:
            specs.append(TensorSpec("o_proj.bias", (h,), "bias"))
        return tuple(specs)

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def load(self, tensors, device, dtype):
        w = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0)
        b = None
        if self.qkv_bias:
            b = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], dim=0)
            b = b.to(device=device, dtype=torch.float32).contiguous()
        self.qkv_proj = Linear(w.to(device=device, dtype=dtype).contiguous(), b)
        ob = tensors["o_proj.bias"].to(device=device, dtype=torch.float32).contiguous() if self.out_bias else None
        self.o_proj = Linear(tensors["o_proj.weight"].to(device=device, dtype=dtype).contiguous(), ob)

    accepts_deferred_norm = True     # forward takes a DeferredNorm as its input
    accepts_residual = True          # forward can add its result into the residual stream itself

    def plan_key(self):
        """Mixers with equal keys read the same work lists, which are then built once a step."""
        return ("gqa_attention", self.rows_per_token, self.num_kv_heads, bool(self.window))

    def plan_step(self, host):
        """The attention kernels' work lists for a step of this shape (int32 arrays by name)."""
        places = 2 * attention_ops.kernels.sm_count() // self.num_kv_heads      # two CTAs of the tcgen05 kernel fit an SM
        return attention_ops.plan_step(host, self.rows_per_token, self.window or 0, places)

    def forward(self, ctx, h, stop, residual=None):
        """Returns the update of the residual stream, or None after adding it into ``residual``."""
        qkv = self.qkv_proj(h)
        out = attention_ops.attend(ctx, ctx.plan(self), qkv, ctx.kv(stop), self.position, self.num_heads,
                                   self.num_kv_heads, self.head_dim, self.window, self.scale, stop.owns_cache)
        return self.o_proj(out, residual=residual)
