"""Pre-norm residual arrangement (reference src/qwen25vl_lite/text.py:196-206):
``x += mixer(norm1(x)); x += ffn(norm2(x))``.  The additions are carried as a pending update
into the next norm kernel, so each is fused with the normalisation that follows it."""

from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    def forward(self, ctx, x, pending, stop):
        h = self.norms[0].forward(ctx, x, pending)
        mixed = self.mixer.forward(ctx, h, stop)
        h = self.norms[1].forward(ctx, x, mixed)
        return self.feed_forward.forward(ctx, h)
