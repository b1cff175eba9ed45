"""Choice of the attention kernels for a step, and the work lists those kernels read.

bfloat16 with a head size and page size the tensor-core kernels take (``csrc/attention_mma.cu``):

* a step in which every entry brings one token, with a rotary position encoding that can hand
  out its tables: one fused kernel rotates q and the new k, writes the new k and v into the
  pages, attends, and merges its key ranges (the CTA that finishes last does it);
* otherwise the position encoding runs first (``rotate_and_store``), then entries that bring one
  token go to the split-KV decode kernel (partials through scratch memory and a combine
  kernel) and runs of tokens to the prefill kernel (tcgen05 at head size 128, mma.sync else).

Everything else (float32, other sizes) goes to the general kernel
(``csrc/attention_generic.cu``) after ``rotate_and_store``.

The tensor-core kernels walk work lists: the entries that bring one token, and (entry, row tile)
pairs for the others.  ``plan_step`` builds them on the host from the step's shape; the step
function packs whatever a part's ``plan_step`` returns into the step's one transfer and hands
the device copies back through ``ctx.plan(part)``.
"""

from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from . import kernels

PREFILL_TILE_ROWS = (64, 128)   # row tiles of the two prefill attention kernels (mma.sync, tcgen05)
KEY_TILE = 64                   # keys per iteration of the tcgen05 prefill kernel
MIN_PART_TILES = 4              # a row tile's keys are cut into parts of at least this many key tiles
MIN_CUT_WALK = 24               # and only when the longest walk of the step has this many key tiles
MAX_PARTS = 15
_scratch = {}


def plan_step(host, group: int, window: int = 0, places: int = 0) -> Dict[str, np.ndarray]:
    """Work lists for a mixer whose kv heads each serve ``group`` query heads.  ``host`` describes
    the step (``q_lens``: tokens each entry brings, ``starts``: tokens it already has in the cache).

    ``decode_items``: the entries that bring one token (groups of more than 16 heads do not fit the
    decode kernel's 16 rows and go with the runs).  ``tiles64``: flat (entry, tile) pairs of the
    other entries, a tile being 64 consecutive rows of the entry's (token, head of the group) pairs;
    the tiles of a run's last tokens see the most keys, so they go first and the short ones fill in
    behind them.  ``tiles128``: the same in tiles of 128 rows for the tcgen05 kernel, as triples
    (entry, tile, code), with the keys of the long tiles cut into parts (``split_keys``), and
    ``merge128``: the tiles whose parts a second kernel adds up, as (entry, tile, first part, parts).
    ``places``: CTAs of the tcgen05 kernel that run at a time for one kv head (0: nothing is cut)."""
    q_lens, starts = host.q_lens, host.starts
    runs = [i for i, n in enumerate(q_lens) if n > 1 or group > 16]
    run_set = set(runs)
    out = {"decode_items": np.asarray([i for i in range(len(q_lens)) if i not in run_set], dtype=np.int32)}
    pairs = [(i, t) for i in runs for t in range(-(-q_lens[i] * group // 64))]
    pairs.sort(key=lambda it: -(starts[it[0]] + (it[1] + 1) * 64 // group))
    out["tiles64"] = np.asarray(pairs, dtype=np.int32).reshape(-1)
    # tiles of 128 rows: how many key tiles each walks (a tile's last row sees the most keys)
    tiles = []
    for i in runs:
        for t in range(-(-q_lens[i] * group // 128)):
            last_token = min((t * 128 + 127) // group, q_lens[i] - 1)
            tiles.append((i, t, (starts[i] + last_token) // KEY_TILE + 1))
    triples, merges = split_keys(tiles, bool(window), places)
    out["tiles128"] = np.asarray(triples, dtype=np.int32).reshape(-1)
    out["merge128"] = np.asarray(merges, dtype=np.int32).reshape(-1)
    return out


def split_keys(tiles, windowed: bool, places: int, shortest: int = MIN_PART_TILES, min_walk: int = MIN_CUT_WALK):
    """Cuts the keys of long row tiles into parts when a step has few row tiles.  A CTA of the tcgen05
    prefill kernel walks a tile's keys one key tile after the other (about 1.1 us each), so a step
    takes as long as its longest walk however many SMs are idle: 128 tokens after 8,000 are 16 CTAs
    of 126 key tiles each.  The tiles are then cut into parts of at most ``length`` key tiles, each a
    piece of work of its own that leaves unnormalised sums, and a merge kernel adds the parts up.
    ``places``: CTAs that run at a time, for one kv head.  Measured on B200 (16 query and 2 kv heads,
    so 296 places in all; whole -> cut):

    * the pieces must fit the places: a second round of CTAs costs more than shorter walks save
      (2,048 tokens: 256 CTAs 45 us, cut into 384 CTAs 57 us; 512 tokens after 3,000: 64 CTAs 64 us,
      280 CTAs 36 us, 440 CTAs 48 us), so ``length`` is the smallest, from ``shortest`` on, with
      which they do;
    * where the whole tiles fill more than half the places, the cut saves what the merge kernel and
      the fuller SMs cost (2,048 tokens with the 20 longest tiles halved: 45 -> 47 us; 1,500 tokens
      after 500: 51 -> 47 us), and with short walks it loses (1,024 tokens, 16 key tiles at most:
      25 -> 28 us), so those steps stay whole;
    * the others: 128 tokens after 8,000: 134 -> 29 us; 64 after 2,000: 41 -> 16 us; four runs of
      256 after 100 to 5,000: 92 -> 45 us; 300 and 200 after 4,000: 94 -> 30 us.

    A tile has at most ``MAX_PARTS`` parts.  Windowed attention is not cut (a part may hold no key
    that a row sees).  ``tiles``: (entry, tile, key tiles).  Returns the work list, longest first, as
    (entry, tile, code) with code = first part << 8 | part << 4 | parts (1 for a whole tile), and the
    list of cut tiles as (entry, tile, first part, parts); parts are numbered through the whole step."""
    counts = np.asarray([n for _, _, n in tiles], dtype=np.int64)
    length = 0
    if not windowed and len(tiles) and 2 * len(tiles) <= places and counts.max() >= max(min_walk, shortest + 1):
        pieces = lambda length: int(np.minimum(MAX_PARTS, -(-counts // length)).sum())
        lo, hi = shortest, int(counts.max())            # pieces(hi) = len(tiles) fits
        while lo < hi:
            mid = (lo + hi) // 2
            if pieces(mid) <= places:
                hi = mid
            else:
                lo = mid + 1
        length = lo
    work, merges, next_part = [], [], 0
    for i, t, n in tiles:
        parts = min(MAX_PARTS, -(-n // length)) if length else 1
        if parts == 1:
            work.append((n, i, t, 1))
            continue
        per = -(-n // parts)
        parts = -(-n // per)                       # no empty part
        merges.append((i, t, next_part, parts))
        for p in range(parts):
            work.append((min(per, n - p * per), i, t, (next_part << 8) | (p << 4) | parts))
        next_part += parts
    work.sort(key=lambda w: -w[0])
    return [(i, t, code) for _, i, t, code in work], merges


def decode_splits(n_items: int, nkv: int, max_kv_len: int, most: int = 64) -> int:
    """Into how many key ranges a decode entry is cut.  Measured on B200 (3B sizes, batch 1 to
    64, contexts 2k to 16k): fastest is the largest count that still gives every CTA an SM of its
    own (the kernel's shared memory allows one CTA per SM, a second wave doubles the time), as
    long as a range keeps at least 256 keys (two 32-key tiles per warp)."""
    by_work = max(1, -(-max_kv_len // 256))
    by_sms = max(1, kernels.sm_count() // max(1, n_items * nkv))
    return int(min(by_work, by_sms, most))


def _scratch_floats(n: int, device) -> torch.Tensor:
    """Scratch memory for split partials, grown on demand and kept (stream-ordered reuse)."""
    buf = _scratch.get(device)
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def _pairs(flat, width: int = 2):
    return None if flat is None else flat.view(-1, width)


def attend(ctx, plan, qkv, kv, position, nq: int, nkv: int, head_dim: int, window, scale: float, store: bool) -> torch.Tensor:
    """Position-encodes q and k, writes this step's k and v into the pages (``store``), and
    attends.  qkv: [N, (nq + 2 nkv) * D] as projected; kv: the stop's pages, slots and block
    table for this step; plan: the device copies of what ``plan_step`` returned (None entries
    for empty lists).  Returns [N, nq * D]."""
    window = int(window or 0)
    group = nq // nkv
    tables = position.rope_tables()
    decode_items = plan.get("decode_items")
    if (store and tables is not None and decode_items is not None and decode_items.shape[0] == ctx.n_seqs
            and plan.get("tiles64") is None
            and kernels.attention_fused_supports(qkv.dtype, head_dim, kv.page_size, group)):
        inv_freq, axis = tables
        # the angles are the same for every layer of the step that shares the tables: the first
        # one to ask computes them
        key = ("rope_angles", inv_freq.data_ptr(), axis.data_ptr())
        angles = ctx.shared.get(key)
        if angles is None:
            angles = ctx.shared[key] = kernels.rope_angles(ctx.positions, inv_freq, axis)
        out = torch.empty((qkv.shape[0], nq * head_dim), dtype=qkv.dtype, device=qkv.device)
        visible = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(ctx.n_seqs, nkv, visible)
        scratch = _scratch_floats(ctx.n_seqs * nq * splits * (head_dim + 2), qkv.device) if splits > 1 else None
        kernels.attention_decode_fused(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                       decode_items, nq, nkv, head_dim, kv.page_size, window, scale, splits,
                                       ctx.positions, inv_freq, axis, kv.kv_slot, scratch, angles,
                                       dense=True)          # every entry of the step is one token, in order
        return out
    position.rotate_and_store(ctx, qkv, nq, nkv, head_dim, kv if store else None)
    return paged_attention(ctx, plan, qkv, kv, nq, nkv, head_dim, window, scale)


def paged_attention(ctx, plan, qkv, kv, nq: int, nkv: int, head_dim: int, window, scale: float) -> torch.Tensor:
    """qkv: [N, (nq + 2 nkv) * D] with q already position-encoded and this step's keys and
    values already in the pages.  Returns [N, nq * D]."""
    out = torch.empty((qkv.shape[0], nq * head_dim), dtype=qkv.dtype, device=qkv.device)
    window = int(window or 0)
    group = nq // nkv
    if not kernels.attention_mma_supports(qkv.dtype, head_dim, kv.page_size):
        kernels.paged_attention_generic(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.token_seq, ctx.cu_q,
                                        ctx.q_start_pos, nq, nkv, head_dim, kv.page_size, window, scale)
        return out
    decode_items = plan.get("decode_items")
    if decode_items is not None:
        n_items = decode_items.shape[0]
        visible = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(n_items, nkv, visible)
        scratch = _scratch_floats(n_items * nq * splits * (head_dim + 2), qkv.device) if splits > 1 else None
        kernels.attention_decode(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                 decode_items, nq, nkv, head_dim, kv.page_size, window, scale, splits, scratch)
    tiles64, tiles128 = _pairs(plan.get("tiles64")), _pairs(plan.get("tiles128"), 3)
    if tiles64 is not None:
        if tiles128 is not None and group <= 128 and kernels.attention_tcgen05_supports(qkv.dtype, head_dim, kv.page_size, qkv):
            merge128 = _pairs(plan.get("merge128"), 4)
            # every piece of work may be a part: room for that many partial results
            scratch = None if merge128 is None else _scratch_floats(
                tiles128.shape[0] * nkv * 128 * (head_dim + 2), qkv.device)
            kernels.attention_prefill_tcgen05(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                              tiles128, nq, nkv, head_dim, kv.page_size, window, scale, merge128, scratch)
        else:
            kernels.attention_prefill(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos, tiles64,
                                      nq, nkv, head_dim, kv.page_size, window, scale)
    return out
