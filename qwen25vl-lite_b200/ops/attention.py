"""Choice of the attention kernel for a step.

bfloat16 with a head size and page size the tensor-core kernels take (``csrc/attention_mma.cu``):
entries that bring one token go to the split-KV decode kernel, runs of tokens to the
prefill kernel.  Everything else (float32, other sizes) goes to the general kernel
(``csrc/attention_generic.cu``).
"""

from __future__ import annotations

import torch

from . import kernels

SM_COUNT = 148
_scratch = {}


def decode_splits(n_items: int, nkv: int, max_kv_len: int) -> int:
    """Into how many key ranges a decode entry is cut: enough CTAs for two per SM, but at
    least 256 keys (two 32-key tiles per warp) in each."""
    by_work = max(1, -(-max_kv_len // 256))
    by_sms = max(1, (2 * SM_COUNT) // max(1, n_items * nkv))
    return int(min(by_work, by_sms, 64))


def _scratch_floats(n: int, device) -> torch.Tensor:
    """Scratch memory for split partials, grown on demand and kept (stream-ordered reuse)."""
    buf = _scratch.get(device)
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def paged_attention(ctx, qkv, kv, nq: int, nkv: int, head_dim: int, window, scale: float) -> torch.Tensor:
    """qkv: [N, (nq + 2 nkv) * D] with q already position-encoded; kv: the stop's pages and
    block table for this step.  Returns [N, nq * D]."""
    out = torch.empty((qkv.shape[0], nq * head_dim), dtype=qkv.dtype, device=qkv.device)
    window = int(window or 0)
    group = nq // nkv
    if not kernels.attention_mma_supports(qkv.dtype, head_dim, kv.page_size) or group not in ctx.prefill_tiles:
        kernels.paged_attention_generic(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.token_seq, ctx.cu_q,
                                        ctx.q_start_pos, nq, nkv, head_dim, kv.page_size, window, scale)
        return out
    if ctx.decode_items is not None and group <= 16:
        n_items = ctx.decode_items.shape[0]
        visible = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(n_items, nkv, visible)
        scratch = _scratch_floats(n_items * nq * splits * (head_dim + 2), qkv.device) if splits > 1 else None
        kernels.attention_decode(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                 ctx.decode_items, nq, nkv, head_dim, kv.page_size, window, scale, splits, scratch)
    tiles = ctx.prefill_tiles[group]
    if tiles is not None:
        kernels.attention_prefill(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos, tiles,
                                  nq, nkv, head_dim, kv.page_size, window, scale)
    return out
