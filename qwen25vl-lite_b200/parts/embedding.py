"""Token embedding and output head (reference src/qwen25vl_lite/text.py:213;
src/qwen25vl_lite/model.py:84-86,200-202): a row gather without scaling, and
``logits = h . W^T`` without bias, where W is the embedding table again when the head is
tied and the checkpoint stores no head of its own (model.py:381-388,416-418)."""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import Linear
from .base import Part, TensorSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight = None

    def tensor_specs(self):
        return (TensorSpec("weight", (self.vocab_size, self.hidden_size)),)

    def load(self, tensors, device, dtype):
        self.weight = tensors["weight"].to(device=device, dtype=dtype).contiguous()

    def exports(self):
        return {"weight": self.weight}

    def forward(self, ctx):
        x = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=self.weight.device)
        kernels.embed_gather(self.weight, ctx.token_ids, x)
        return x


@register_head("linear_head")
class LinearHead(Part):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_deferred_norm = True     # its product is a ``Linear``, which normalises inside the kernel when it can

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, tied_to: str = "embed_tokens.weight"):
        """``tied``: without a weight of its own in the checkpoint the head reads the tensor that
        another part holds under the canonical name ``tied_to`` (the embedding table)."""
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.tied_to = tied_to
        self._tied_weight = None
        self.proj = None

    def tensor_specs(self):
        return (TensorSpec("weight", (self.vocab_size, self.hidden_size), optional=self.tied),)

    def imports(self):
        return (self.tied_to,) if self.tied else ()

    def receive(self, tensors):
        self._tied_weight = tensors.get(self.tied_to)

    def load(self, tensors, device, dtype):
        if "weight" in tensors:      # an explicit head wins over the tie
            self.proj = Linear(tensors["weight"].to(device=device, dtype=dtype).contiguous())
        elif self.tied and self._tied_weight is not None:
            if tuple(self._tied_weight.shape) != (self.vocab_size, self.hidden_size):
                raise ValueError(f"output head is tied to {self.tied_to}, whose shape {tuple(self._tied_weight.shape)} "
                                 f"is not [{self.vocab_size}, {self.hidden_size}]")
            self.proj = Linear(self._tied_weight)
        else:
            raise ValueError("output head has no weight of its own" + (f" and no earlier part holds {self.tied_to!r}, "
                             "which it is tied to" if self.tied else " and is not tied"))

    def forward(self, ctx, h):
        return self.proj(h, out_dtype=torch.float32)
