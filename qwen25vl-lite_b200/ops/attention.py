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

from typing import Dict, Optional

import numpy as np
import torch

from . import kernels

KEY_TILE = 64                   # keys per iteration of the tcgen05 prefill kernel
MIN_PART_TILES = 4              # a row tile's keys are cut into parts of at least this many key tiles
MIN_CUT_WALK = 24               # in steps whose longest walk has this many key tiles
MIN_PAIR_WALK = 6               # a cluster of two CTAs halves a tile's walk of this many key tiles or more,
MIN_PAIRS_WALK = 12             # in steps whose longest walk has this many
MAX_PARTS = 15
_scratch = {}
_retired = []


def plan_step(host, group: int, window: int = 0, places: int = 0) -> Dict[str, np.ndarray]:
    """Work lists for a mixer whose kv heads each serve ``group`` query heads.  ``host`` describes
    the step (``q_lens``: tokens each entry brings, ``starts``: tokens it already has in the cache).

    ``decode_items``: the entries that bring one token (groups of more than 16 heads do not fit the
    decode kernel's 16 rows and go with the runs).  ``tiles64``: flat (entry, tile) pairs of the
    other entries, a tile being 64 consecutive rows of the entry's (token, head of the group) pairs;
    the tiles of a run's last tokens see the most keys, so they go first and the short ones fill in
    behind them.  ``tiles128``: the same in tiles of 128 rows for the tcgen05 kernel, as triples
    (entry, tile, code), where a step of few tiles has the keys of its long tiles cut (``cut_keys``);
    ``merge128``: the tiles whose parts a second kernel adds up, as (entry, tile, first part, parts);
    ``pairs128`` is not empty when ``tiles128`` is meant for clusters of two CTAs (``pair_split``).
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
    triples, merges, clusters = cut_keys(tiles, bool(window), places)
    out["pairs128"] = np.ones(1 if clusters else 0, dtype=np.int32)        # its presence says how tiles128 is to be read
    out["tiles128"] = np.asarray(triples, dtype=np.int32).reshape(-1)
    out["merge128"] = np.asarray(merges, dtype=np.int32).reshape(-1)
    return out


def cut_keys(tiles, windowed: bool, places: int):
    """How the tcgen05 prefill kernel takes a step's row tiles.  A CTA walks a tile's keys one key tile
    after the other (about 1.1 us each, after 8 us of start and end), two CTAs to an SM, so a step
    with few row tiles takes as long as its longest walk however many SMs are idle.  There are two
    ways to cut walks, and three outcomes; ``tiles`` is (entry, tile, key tiles), ``places`` the CTAs
    that run at a time for one kv head (0: nothing is cut), and the result (work list, merges,
    pairs) as ``plan_step`` describes them:

    * parts through scratch memory (``split_keys``): up to ``MAX_PARTS`` parts a tile, as many pieces as
      there are places, a merge kernel behind; costs about 6 key tiles' time;
    * clusters of two CTAs (``pair_split``) that halve a tile's keys and add up through the cluster's
      shared memory: costs about 5 key tiles' time, and twice the places;
    * whole tiles, when the tiles fill more than three quarters of the places or the walks are short.

    Measured on B200, 16 query and 2 kv heads (296 places in all), whole / parts / pairs in us:
    128 tokens after 8,000: 134 / 29 / 75; 512 after 3,000: 64 / 37 / 41; four runs of 256 after 100
    to 5,000: 92 / 45 / 57; 1,024 after 1,024: 42 / 42 / 32; 1,024: 26 / 28 / 22; 1,200: 29 / - / 26;
    1,500 after 500: 51 / 47 (296 CTAs) / 46; 2,048: 45 / 47 (296 CTAs), 57 (384 CTAs) / 48; 4,096:
    89 / - / 124; 8,192: 291 / - / 354.  Windowed attention is not cut (a part may hold no key that a
    row sees)."""
    whole = lambda: ([(i, t, 1) for i, t, _ in sorted(tiles, key=lambda w: -w[2])], [], False)
    if windowed or not places or not tiles:
        return whole()
    longest = max(n for _, _, n in tiles)
    if 2 * len(tiles) <= places:
        length = part_length(tiles, places) if longest >= MIN_CUT_WALK else 0
        if length and -(-longest // 2) > length + 6:
            return split_keys(tiles, length) + (False,)
    if 4 * len(tiles) <= 3 * places and longest >= MIN_PAIRS_WALK:
        return pair_split(tiles), [], True
    return whole()


def pair_split(tiles):
    """The work list for clusters of two CTAs, longest walk first: (entry, tile, 2) for a tile whose
    keys the two halve (the second leaves its rows in its shared memory and the first adds them up),
    (entry, tile, 1) for a short one that the first CTA takes alone."""
    work = [(-(-n // 2) if n >= MIN_PAIR_WALK else n, i, t, 2 if n >= MIN_PAIR_WALK else 1) for i, t, n in tiles]
    work.sort(key=lambda w: -w[0])
    return [(i, t, code) for _, i, t, code in work]


def part_length(tiles, places: int, shortest: int = MIN_PART_TILES) -> int:
    """The least number of key tiles per part, from ``shortest`` on, with which the parts of all
    tiles still fit the places: a second round of CTAs costs more than shorter walks save."""
    counts = np.asarray([n for _, _, n in tiles], dtype=np.int64)
    pieces = lambda length: int(np.minimum(MAX_PARTS, -(-counts // length)).sum())
    lo, hi = shortest, max(shortest, int(counts.max()))            # pieces(longest walk) = len(tiles) fits
    while lo < hi:
        mid = (lo + hi) // 2
        if pieces(mid) <= places:
            hi = mid
        else:
            lo = mid + 1
    return lo


def split_keys(tiles, length: int):
    """Cuts the keys of the tiles that walk more than ``length`` key tiles into parts of at most that
    many (``MAX_PARTS`` parts at most), each a piece of work of its own that leaves unnormalised sums
    in scratch memory; a merge kernel adds the parts up.  Returns the work list, longest first, as
    (entry, tile, code) with code = first part << 8 | part << 4 | parts (1 for a whole tile), and the
    list of cut tiles as (entry, tile, first part, parts); parts are numbered through the whole step."""
    work, merges, next_part = [], [], 0
    for i, t, n in tiles:
        parts = min(MAX_PARTS, -(-n // length))
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


def _scratch_floats(n: int, device, use: str = "decode") -> torch.Tensor:
    """Scratch memory for partial results, grown on demand and kept (stream-ordered reuse).  One
    buffer per use: captured decode steps hold the address of theirs, so the far larger needs of a
    prompt's parts must not make it move."""
    buf = _scratch.get((device, use))
    if buf is None or buf.numel() < n:
        if buf is not None and use == "decode":
            _retired.append(buf)                    # a captured step may still point at it
        buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=device)
        _scratch[(device, use)] = buf
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
    out = None
    if (store and tables is not None and decode_items is not None
            and kernels.attention_fused_supports(qkv.dtype, head_dim, kv.page_size, group)):
        # The entries of one token go through the fused kernel, which rotates q and k, stores k and
        # v and attends by itself, from qkv as projected.
        inv_freq, axis = tables
        # the angles are the same for every layer of the step that shares the tables: the first
        # one to ask computes them
        key = ("rope_angles", inv_freq.data_ptr(), axis.data_ptr())
        angles = ctx.shared.get(key)
        if angles is None:
            angles = ctx.shared[key] = kernels.rope_angles(ctx.positions, inv_freq, axis)
        out = torch.empty((qkv.shape[0], nq * head_dim), dtype=qkv.dtype, device=qkv.device)
        n_items = decode_items.shape[0]
        alone = n_items == ctx.n_seqs and plan.get("tiles64") is None
        visible = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(n_items, nkv, visible)
        scratch = _scratch_floats(n_items * nq * splits * (head_dim + 2), qkv.device) if splits > 1 else None
        kernels.attention_decode_fused(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                       decode_items, nq, nkv, head_dim, kv.page_size, window, scale, splits,
                                       ctx.positions, inv_freq, axis, kv.kv_slot, scratch, angles,
                                       dense=alone)          # every entry of the step is one token, in order
        if alone:
            return out
        # The runs beside them: q and k of all tokens are rotated now (the single tokens' too, whose
        # rows of the output are written already, and their keys and values are stored a second
        # time with the same values), then the runs' kernels fill their rows.
    position.rotate_and_store(ctx, qkv, nq, nkv, head_dim, kv if store else None)
    return paged_attention(ctx, plan, qkv, kv, nq, nkv, head_dim, window, scale, out)


def paged_attention(ctx, plan, qkv, kv, nq: int, nkv: int, head_dim: int, window, scale: float,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """qkv: [N, (nq + 2 nkv) * D] with q already position-encoded and this step's keys and
    values already in the pages.  Returns [N, nq * D].  ``out``: the result with the rows of the
    one-token entries already written (only the runs are left to do)."""
    single_done = out is not None
    if out is None:
        out = torch.empty((qkv.shape[0], nq * head_dim), dtype=qkv.dtype, device=qkv.device)
    window = int(window or 0)
    group = nq // nkv
    if not kernels.attention_mma_supports(qkv.dtype, head_dim, kv.page_size):
        kernels.paged_attention_generic(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.token_seq, ctx.cu_q,
                                        ctx.q_start_pos, nq, nkv, head_dim, kv.page_size, window, scale)
        return out
    decode_items = plan.get("decode_items")
    if decode_items is not None and not single_done:
        n_items = decode_items.shape[0]
        visible = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(n_items, nkv, visible)
        scratch = _scratch_floats(n_items * nq * splits * (head_dim + 2), qkv.device) if splits > 1 else None
        kernels.attention_decode(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                 decode_items, nq, nkv, head_dim, kv.page_size, window, scale, splits, scratch)
    pairs = plan.get("pairs128") is not None
    tiles64, tiles128 = _pairs(plan.get("tiles64")), _pairs(plan.get("tiles128"), 3)
    if tiles64 is not None:
        if tiles128 is not None and group <= 128 and kernels.attention_tcgen05_supports(qkv.dtype, head_dim, kv.page_size, qkv):
            merge128 = _pairs(plan.get("merge128"), 4)
            # every piece of work may be a part: room for that many partial results
            scratch = None if merge128 is None else _scratch_floats(
                tiles128.shape[0] * nkv * 128 * (head_dim + 2), qkv.device, "parts")
            kernels.attention_prefill_tcgen05(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos,
                                              tiles128, nq, nkv, head_dim, kv.page_size, window, scale, merge128, scratch,
                                              pairs=pairs)
        else:
            kernels.attention_prefill(qkv, out, kv.k_pages, kv.v_pages, kv.block_table, ctx.cu_q, ctx.q_start_pos, tiles64,
                                      nq, nkv, head_dim, kv.page_size, window, scale)
    return out
