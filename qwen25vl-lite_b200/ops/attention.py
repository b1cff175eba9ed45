"""Choice of the attention kernel for a step.

The general kernel (``csrc/attention_generic.cu``) serves the 32-bit path and every size;
the serving path switches to the tensor-core kernels where their sizes fit.
"""

from __future__ import annotations

import torch

from . import kernels


def paged_attention(ctx, qkv, kv, nq: int, nkv: int, head_dim: int, window, scale: float) -> torch.Tensor:
    """qkv: [N, (nq + 2 nkv) * D] with q already position-encoded; kv: the stop's pages and
    block table for this step.  Returns [N, nq * D]."""
    out = torch.empty((qkv.shape[0], nq * head_dim), dtype=qkv.dtype, device=qkv.device)
    kernels.paged_attention_generic(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.token_seq, ctx.cu_q,
                                    ctx.q_start_pos, nq, nkv, head_dim, kv.page_size, window or 0, scale)
    return out
