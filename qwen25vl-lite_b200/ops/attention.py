"""Choice of the attention kernels for a step.

bfloat16 with a head size and page size the tensor-core kernels take (``csrc/attention_mma.cu``):

* a step in which every entry brings one token, with a rotary position encoding that can hand
  out its tables: one fused kernel rotates q and the new k, writes the new k and v into the
  pages, attends, and merges its key ranges (the CTA that finishes last does it);
* otherwise the position encoding runs first (``rotate_and_store``), then entries that bring one
  token go to the split-KV decode kernel (partials through scratch memory and a combine
  kernel) and runs of tokens to the prefill kernel.

Everything else (float32, other sizes) goes to the general kernel
(``csrc/attention_generic.cu``) after ``rotate_and_store``.
"""

from __future__ import annotations

import torch

from . import kernels

SM_COUNT = 148
# which kernel attends runs of tokens at head size 128: "tcgen05" (scores and P.V on the 5th-generation
# tensor cores) or "mma" (mma.sync, the kernel of every other head size)
PREFILL_ATTENTION = __import__("os").environ.get("Q25VL_PREFILL_ATTENTION", "tcgen05")
_scratch = {}


def decode_splits(n_items: int, nkv: int, max_kv_len: int, most: int = 64) -> int:
    """Into how many key ranges a decode entry is cut.  Measured on B200 (3B sizes, batch 1 to
    64, contexts 2k to 16k): fastest is the largest count that still gives every CTA an SM of its
    own (the kernel's shared memory allows one CTA per SM, a second wave doubles the time), as
    long as a range keeps at least 256 keys (two 32-key tiles per warp)."""
    by_work = max(1, -(-max_kv_len // 256))
    by_sms = max(1, SM_COUNT // max(1, n_items * nkv))
    return int(min(by_work, by_sms, most))


def _scratch_floats(n: int, device) -> torch.Tensor:
    """Scratch memory for split partials, grown on demand and kept (stream-ordered reuse)."""
    buf = _scratch.get(device)
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def attend(ctx, qkv, kv, position, nq: int, nkv: int, head_dim: int, window, scale: float, store: bool) -> torch.Tensor:
    """Position-encodes q and k, writes this step's k and v into the pages (``store``), and
    attends.  qkv: [N, (nq + 2 nkv) * D] as projected; kv: the stop's pages, slots and block
    table for this step.  Returns [N, nq * D]."""
    window = int(window or 0)
    group = nq // nkv
    tables = getattr(position, "rope_tables", None)
    if (store and tables is not None and ctx.decode_items is not None and ctx.decode_items.shape[0] == ctx.n_seqs
            and ctx.prefill_tiles.get(group, 0) is None
            and kernels.attention_fused_supports(qkv.dtype, head_dim, kv.page_size, group)):
        inv_freq, axis = tables()
        # the angles are the same for every layer of the step: the first one to ask computes them
        shared = getattr(ctx, "shared", None)
        key = ("rope_angles", inv_freq.data_ptr())
        angles = shared.get(key) if shared is not None else None
        if angles is None:
            angles = kernels.rope_angles(ctx.positions, inv_freq, axis)
            if shared is not None:
                shared[key] = angles
        out = torch.empty((qkv.shape[0], nq * head_dim), dtype=qkv.dtype, device=qkv.device)
        visible = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(ctx.n_seqs, nkv, visible)
        scratch = _scratch_floats(ctx.n_seqs * nq * splits * (head_dim + 2), qkv.device) if splits > 1 else None
        kernels.attention_decode_fused(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                       ctx.decode_items, nq, nkv, head_dim, kv.page_size, window, scale, splits,
                                       ctx.positions, inv_freq, axis, kv.kv_slot, scratch, angles,
                                       dense=True)          # every entry of the step is one token, in order
        return out
    position.rotate_and_store(ctx, qkv, nq, nkv, head_dim, kv if store else None)
    return paged_attention(ctx, qkv, kv, nq, nkv, head_dim, window, scale)


def paged_attention(ctx, qkv, kv, nq: int, nkv: int, head_dim: int, window, scale: float) -> torch.Tensor:
    """qkv: [N, (nq + 2 nkv) * D] with q already position-encoded and this step's keys and
    values already in the pages.  Returns [N, nq * D]."""
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
        tiles128 = getattr(ctx, "prefill_tiles128", {}).get(group)
        if PREFILL_ATTENTION == "tcgen05" and tiles128 is not None and group <= 128 \
                and kernels.attention_tcgen05_supports(qkv.dtype, head_dim, kv.page_size, qkv):
            kernels.attention_prefill_tcgen05(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                              tiles128, nq, nkv, head_dim, kv.page_size, window, scale)
        else:
            kernels.attention_prefill(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos, tiles,
                                      nq, nkv, head_dim, kv.page_size, window, scale)
    return out
