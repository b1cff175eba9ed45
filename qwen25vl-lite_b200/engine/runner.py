"""The step function: one batch of (request, its next tokens) through the model, from the
cache that earlier steps left, returning logits at the wanted places.

The reference runs prompt portions one request at a time and decoded tokens as a separate
batch (``ModelRunner.run_prefill_chunk`` / ``run_decode``, src/qwen25vl_lite/engine.py:
318-335, 430-472) and rebuilds its index tensors from Python lists every step
(engine.py:296,314,322,439-452).  Here a step is one flat batch: portions of prompts of any
length beside single decoded tokens, described by a handful of int32 arrays that are packed
on the host and copied to the device in one transfer.

Per step, for S entries holding N tokens in all (everything int32):

    token_ids[N]          positions[axes, N]      token_seq[N]   entry of each token
    cu_q[S + 1]           first token of each entry
    q_start_pos[S]        tokens of the request already in the cache
    slot_ids[S]           per-request state slot
    logit_rows[M]         flat indices of the tokens whose logits are wanted
    per cache group:      kv_slot[N] (page * page_size + offset), block_table[S, W]
"""

from __future__ import annotations

import gc
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..models.decoder import DecoderModel, StopRuntime
from ..ops import kernels


@dataclass(eq=False)
class Request:
    """A live request as the step function sees it."""

    request_id: object
    cache: RequestCache
    # per cache group: the block table as the kernels read it (an array, no negative entries), with
    # the table's length and released count when it was made
    _tables: Dict[int, tuple] = field(default_factory=dict, repr=False, compare=False)

    @property
    def num_computed(self) -> int:
        return self.cache.num_tokens

    def block_table(self, group: int) -> np.ndarray:
        """The group's block table as an int64 array with 0 where no page is held; converted
        again only when the table has grown or a window has released pages."""
        table = self.cache.tables[group]
        released = self.cache.released[group] if self.cache.released else 0
        hit = self._tables.get(group)
        if hit is None or hit[0] != len(table) or hit[1] != released:
            hit = self._tables[group] = (len(table), released, np.maximum(np.asarray(table, dtype=np.int64), 0))
        return hit[2]


@dataclass
class StepEntry:
    request: Request
    tokens: Sequence[int]
    want: Sequence[int] = ()                     # indices into ``tokens``
    # [axes, k] for the first k <= len(tokens) tokens; the others (all of them with None) are plain
    # text and sit where the model's position encoding puts plain text after what came before
    positions: Optional[np.ndarray] = None


@dataclass
class HostStep:
    """A step's shape as the host knows it, for parts that plan work lists for their kernels."""

    q_lens: List[int]          # tokens each entry brings
    starts: List[int]          # tokens each entry's request already has in the cache
    n_tokens: int
    n_seqs: int


@dataclass
class KVStep:
    """A cache group's side of one step, as a mixer's kernels need it."""

    k_pages: torch.Tensor = None
    v_pages: torch.Tensor = None
    kv_slot: torch.Tensor = None
    block_table: torch.Tensor = None
    page_size: int = 0


@dataclass
class StepContext:
    dtype: torch.dtype
    device: torch.device
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    cu_q: torch.Tensor
    q_start_pos: torch.Tensor
    slot_ids: torch.Tensor
    logit_rows: Optional[torch.Tensor]
    logits_every_row: bool       # every entry brings one token and wants its logits: logit_rows is 0 .. n_tokens - 1
    max_q_len: int
    max_kv_len: int
    group_kv_slot: List[torch.Tensor]
    group_block_table: List[torch.Tensor]
    cache: CacheManager
    # device copies of what the parts' ``plan_step`` returned, by plan key and array name
    plans: Dict[object, Dict[str, Optional[torch.Tensor]]] = field(default_factory=dict)
    # host copies, for parts written with torch operators (toy parts in tests)
    host_q_lens: List[int] = field(default_factory=list)
    host_q_start: List[int] = field(default_factory=list)
    host_slots: List[int] = field(default_factory=list)
    # what parts compute once per forward pass and share between layers (the model empties it
    # when a pass begins); keyed by whoever puts it there
    shared: Dict[object, object] = field(default_factory=dict)

    def plan(self, part) -> Dict[str, Optional[torch.Tensor]]:
        """The work lists ``part.plan_step`` asked for, on the device (None for an empty one)."""
        return self.plans[part.plan_key()]

    def kv(self, stop: StopRuntime) -> KVStep:
        group, k_pages, v_pages = self.cache.stop_pages(stop.index)
        return KVStep(k_pages, v_pages, self.group_kv_slot[group.index], self.group_block_table[group.index],
                      group.page_size)


GRAPH_WIDTH_STEP = 16      # block-table widths of captured steps are rounded up to 1, 1.5, 2, 3, 4, 6, 8, ... times this many pages
MAX_GRAPHS = 128           # captured steps kept; the one unused for longest goes first
CAPTURE_ON_USE = 3         # a (batch size, table width) is captured when it comes for the third time


def graph_width(pages: int) -> int:
    """The block-table width a captured step is given for requests of up to ``pages`` pages: the
    next of 16, 24, 32, 48, 64, 96, 128, ... (steps of a factor 1.5 or 1.33).  A captured step serves
    one (batch size, width); with widths in equal steps of 256 tokens a batch that decodes on crossed
    into a new width, two uncaptured steps and a capture, every 256 tokens."""
    unit = GRAPH_WIDTH_STEP
    while True:
        if pages <= unit:
            return unit
        if pages <= unit + unit // 2:
            return unit + unit // 2
        unit *= 2


def graph_batch(entries: int) -> int:
    """The batch size a captured step is given for ``entries`` one-token entries: itself up to 8 (the
    chained products take up to 8 rows), then the next multiple of 8, of 16 beyond 64.  The rows
    that are added read and write a page of their own and their logits are dropped.  While the
    requests of a batch end one after the other every batch size lives a few steps only, too few
    to pay for its capture (11 ms at the 7B sizes: 81 captures were 0.9 s of a 6.8 s trace of 128
    requests)."""
    if entries <= 8:
        return entries
    unit = 8 if entries <= 64 else 16
    return -(-entries // unit) * unit


class ModelRunner:
    """Owns the model, the cache and the staging buffers; ``step`` is the step function."""

    def __init__(self, model: DecoderModel, num_pages: int, page_size: int, max_requests: int,
                 max_step_tokens: int = 8192, cuda_graphs: bool = True):
        if model.dtype is None:
            raise ValueError("the model has no weights loaded")
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.cache = CacheManager(model.stop_needs(), num_pages, page_size, max_requests)
        self.cache.allocate_device(self.device, self.dtype)
        for stop in model.stops:
            stop.state = self.cache.states.get(stop.index)
        self.position = model.position             # defines the tokens' positions
        self.axes = model.position.axes
        # parts whose kernels read work lists built per step: one planner per distinct plan key
        self._planners: Dict[object, object] = {}
        for part in model.planning_parts() if hasattr(model, "planning_parts") else ():
            self._planners.setdefault(part.plan_key(), part)
        self.vocab_size = model.head.vocab_size
        self._staging: Optional[torch.Tensor] = None
        self._staging_free = torch.cuda.Event() if self.device.type == "cuda" else None
        self._reserve(max_step_tokens * (3 + self.axes + len(self.cache.groups)) + 4096)
        self.live: Dict[object, Request] = {}
        self.steps = 0
        # Steps that bring one token per request are launch-bound (hundreds of small kernels), so
        # they are captured once per (batch size, block-table width) and replayed.  Only when every
        # part of the model says its forward can be captured (``graph_safe``: a fixed sequence of this
        # engine's kernels, no host-side loop over the batch, no library operator that synchronises).
        blocks = getattr(model, "blocks", [])
        parts = [p for b in blocks for p in (b.mixer, b.feed_forward, *b.norms)]
        parts += [getattr(model, name, None) for name in ("embedding", "final_norm", "head")]
        parts += model.position_encodings() if hasattr(model, "position_encodings") else [model.position]
        self.cuda_graphs = bool(cuda_graphs and self.device.type == "cuda" and blocks
                                and all(getattr(p, "graph_safe", False) for p in parts))
        self._graphs: Dict[tuple, tuple] = {}
        self._padding = None                    # the request of the rows that fill a captured step's batch, while a step is packed
        self._graph_seen: Dict[tuple, int] = {}
        self._capture_stream = None
        self._graph_pool = None
        self.graph_replays = 0
        # kernels with bounded waits report a wait that gave up here; read back after every step
        # and looked at before the next one
        self._error_host = torch.zeros(1, dtype=torch.int32, pin_memory=self.device.type == "cuda")

    # ---- requests ----------------------------------------------------------------------
    def open_request(self, request_id) -> Request:
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        req = Request(request_id, self.cache.open())
        self.live[request_id] = req
        return req

    def close_request(self, req: Request) -> None:
        self.cache.close(req.cache)
        self.live.pop(req.request_id, None)

    # ---- the step ----------------------------------------------------------------------
    def _reserve(self, n_ints: int) -> None:
        if self._staging is not None and self._staging.numel() >= n_ints:
            return
        n_ints = max(n_ints, 1 << 16)
        pin = self.device.type == "cuda"
        self._staging = torch.empty(n_ints, dtype=torch.int32, pin_memory=pin)
        self._staging_np = self._staging.numpy()
        self._device_ints = torch.empty(n_ints, dtype=torch.int32, device=self.device)

    def _replay(self, key, make_ctx, layout) -> torch.Tensor:
        """Runs a one-token-per-request step from its captured graph.  The step's int arrays sit
        at the same device addresses for the same key (same counts, same packing order), so a
        replay only needs the new values, which ``step`` has already copied.  A key's first
        steps run uncaptured (kernel by kernel, the products chained); when it comes for the third
        time it is captured and replayed from then on: capturing costs tens of steps' worth of
        time, and while requests of a batch end one after the other most keys come only once or
        twice.  ``make_ctx`` builds the step's context; a replay does not need it (a dozen tensor
        views that would stand between the sampled ids and the launch)."""
        hit = self._graphs.pop(key, None)
        if hit is not None and hit[2] != layout:
            hit = None                                  # the staging buffer was re-allocated since
        if hit is not None:
            self._graphs[key] = hit                     # used last: kept longest
        if hit is None:
            seen = self._graph_seen[key] = self._graph_seen.get(key, 0) + 1
            if seen < CAPTURE_ON_USE:
                return self._forward_chained(make_ctx())
            if len(self._graphs) >= MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            ctx = make_ctx()
            graph = torch.cuda.CUDAGraph()
            before = kernels.launch_count()
            # No garbage collection while the stream captures: a dead cycle that holds CUDA graphs
            # or pinned memory (a discarded engine) would be torn down in the middle of the capture,
            # and the calls that does are not allowed then; they invalidate the capture.
            collecting = gc.isenabled()
            gc.disable()
            try:
                logits = self._capture(graph, ctx)
            finally:
                if collecting:
                    gc.enable()
            hit = (graph, logits, layout, kernels.launch_count() - before)
            self._graphs[key] = hit
        hit[0].replay()
        kernels.count_replayed(hit[3])
        self.graph_replays += 1
        return hit[1]

    def _capture(self, graph, ctx: StepContext) -> torch.Tensor:
        """Captures one step into ``graph`` on a side stream that follows the current one.  The
        ``torch.cuda.graph`` context manager would first synchronise the device and hand the
        allocator's cached memory back to the driver, 70 ms with a few tens of GB cached: more
        than ten decode steps for every captured shape, over five seconds of a 128-request trace.
        All graphs draw their buffers from one pool; they never run at the same time."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
            self._graph_pool = torch.cuda.graph_pool_handle()
        side, main = self._capture_stream, torch.cuda.current_stream(self.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            graph.capture_begin(pool=self._graph_pool)
            try:
                logits = self._forward_chained(ctx)
            finally:
                graph.capture_end()
        main.wait_stream(side)
        return logits

    def _forward_chained(self, ctx: StepContext) -> torch.Tensor:
        """The model's forward with the weight-streaming products of consecutive parts gathered
        into single persistent kernels (``kernels.chain_begin``).  Only for steps whose forward
        launches nothing but this engine's kernels, which is what ``graph_safe`` parts promise."""
        if self.dtype != torch.bfloat16:                  # the 32-bit path has no weight-streaming products
            return self.model.forward(ctx)
        kernels.chain_begin()
        try:
            return self.model.forward(ctx)
        finally:
            kernels.chain_end()

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the tokens the entries bring, as one batch.  Returns float32 logits
        [number of wanted places, vocab] on the device, in the order of the entries and of
        each entry's ``want`` (None when nothing is wanted).  On return the tokens are in
        the cache and every request's count has advanced."""
        if not entries:
            return None
        return self._pack(entries)()

    def prepare_decode(self, requests: Sequence[Request]):
        """Everything of a step in which each of ``requests`` brings one token at its default
        position and wants its logits, except the tokens themselves: pages, block tables, slots
        and positions are packed now (while the step before still runs on the device), and
        ``launch_prepared`` only has to add the token ids.  Nothing else may be stepped between."""
        return self._pack([StepEntry(r, (0,), (0,)) for r in requests])

    def launch_prepared(self, prepared, tokens: Optional[Sequence[int]], device_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs a prepared step with its token ids: from the host (``tokens``), or from the device
        (``device_ids`` int32, one per request in order: the ids the sampler has just drawn, which
        the step then reads without their trip to the host and back)."""
        return prepared(tokens, device_ids)

    def drop_prepared(self, prepared) -> None:
        """A prepared step that will not be launched: the page and slot of the rows that filled its
        batch go back."""
        self._close_padding()

    def _pack(self, entries: Sequence[StepEntry]):
        """Builds the step's arrays in the staging buffer; returns the function that runs the step
        (optionally with other token ids than the entries brought, for ``prepare_decode``)."""
        self._close_padding()                               # of a prepared step that was never launched
        try:
            return self._pack_arrays(entries)
        except BaseException:
            self._close_padding()
            raise

    def _close_padding(self) -> None:
        if self._padding is not None:
            self.cache.close(self._padding)
            self._padding = None

    def _pack_arrays(self, entries: Sequence[StepEntry]):
        self.check_kernel_errors()
        ps = self.cache.page_size
        groups = self.cache.groups
        q_lens = [len(e.tokens) for e in entries]
        if min(q_lens) <= 0:
            raise ValueError("a step entry brings no tokens")
        if len({id(e.request) for e in entries}) != len(entries):
            raise ValueError("a request appears twice in one step")
        S, N = len(entries), int(sum(q_lens))
        starts = [e.request.cache.num_tokens for e in entries]
        for e, n, s in zip(entries, q_lens, starts):
            self.cache.ensure(e.request.cache, s + n)       # no-op when the caller already did
        widths = [max(max(len(e.request.cache.tables[g.index]) for e in entries), 1) for g in groups]
        graph_key = None
        pad, pad_cache = 0, None
        if self.cuda_graphs and max(q_lens) == 1 and all(list(e.want) == [0] for e in entries):
            widths = [graph_width(w) for w in widths]
            if (graph_batch(S) > S and all(e.positions is None for e in entries)
                    and getattr(self.position, "default_is_linear", False)):
                pad_cache = self._padding = self._open_padding()
                if pad_cache is not None:
                    pad = graph_batch(S) - S
            graph_key = (S + pad, tuple(widths))
        M = sum(len(e.want) for e in entries)
        real = S
        if pad:                      # rows of one token at position 0 in a page of their own, all alike
            q_lens, starts = q_lens + [1] * pad, starts + [0] * pad
            S, N, M = S + pad, N + pad, M + pad

        # ---- pack ----
        host = HostStep(q_lens, starts, N, S)
        plans = {key: {name: np.ascontiguousarray(a, dtype=np.int32).reshape(-1)
                       for name, a in part.plan_step(host).items()} for key, part in self._planners.items()}
        n_work = sum(a.shape[0] + 4 for p in plans.values() for a in p.values())
        total = (N * (2 + self.axes + len(groups)) + (S + 1) + 2 * S + M + S * sum(widths) + n_work
                 + 4 * (8 + 2 * len(groups)))
        self._reserve(total)
        if self._staging_free is not None:
            self._staging_free.synchronize()               # the last copy out of the staging buffer is done
        buf = self._staging_np
        off = 0

        def take(n):
            nonlocal off
            view = buf[off:off + n]
            span = (off, n)
            off += (n + 3) & ~3                           # every array starts on a 16-byte boundary
            return view, span

        tok, tok_s = take(N)
        pos, pos_s = take(self.axes * N)
        pos = pos.reshape(self.axes, N)
        tseq, tseq_s = take(N)
        cu, cu_s = take(S + 1)
        qs, qs_s = take(S)
        sl, sl_s = take(S)
        rows, rows_s = take(M)
        g_slot, g_slot_s, g_tab, g_tab_s = [], [], [], []
        for g, w in zip(groups, widths):
            a, a_s = take(N)
            b, b_s = take(S * w)
            g_slot.append(a); g_slot_s.append(a_s); g_tab.append(b.reshape(S, w)); g_tab_s.append(b_s)

        plan_s = {}
        for key, arrays in plans.items():
            for name, a in arrays.items():
                view, plan_s[key, name] = take(a.shape[0])
                view[:] = a

        cu[0] = 0
        last_position = []
        if (max(q_lens) == 1 and all(e.positions is None for e in entries)
                and getattr(self.position, "default_is_linear", False)):
            # A step of single tokens at their default positions (the usual decode step): the
            # arrays are filled for all entries at once, and a request's block table is converted
            # only when it has grown.
            ids = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=real)
            if ids.min() < 0 or ids.max() >= self.vocab_size:
                raise ValueError(f"token id outside [0, {self.vocab_size}) in a decode step")
            st = np.asarray(starts, dtype=np.int64)
            place = st.copy()
            place[:real] += np.fromiter((e.request.cache.position_offset for e in entries), dtype=np.int64, count=real)
            tok[:real] = ids
            tok[real:] = 0
            pos[:, :] = place
            last_position = place[:real].tolist()
            tseq[:] = np.arange(S)
            cu[1:] = np.arange(1, S + 1)
            qs[:] = st
            sl[:real] = [e.request.cache.slot for e in entries]
            r = 0
            for i, e in enumerate(entries):
                for w_ in e.want:
                    if int(w_) != 0:
                        raise ValueError(f"wanted place {w_} is outside the 1 token of the entry")
                    rows[r] = i
                    r += 1
            if pad:
                sl[real:] = pad_cache.slot
                rows[real:] = np.arange(real, S)
            for g, gs, gt in zip(groups, g_slot, g_tab):
                for i, (e, s0) in enumerate(zip(entries, starts)):
                    table = e.request.block_table(g.index)
                    gs[i] = e.request.cache.tables[g.index][s0 // ps] * ps + s0 % ps
                    gt[i, :len(table)] = table
                    gt[i, len(table):] = 0
                if pad:
                    gs[real:] = pad_cache.tables[g.index][0] * ps
                    gt[real:, :] = 0
                    gt[real:, 0] = pad_cache.tables[g.index][0]
        else:
            # Any mix of runs and single tokens.  What is the same for every entry is filled for all
            # at once; the single tokens at their default positions (the decoding requests beside a
            # few prompt portions) too; only the runs, and tokens that bring positions, go one by one.
            q = np.asarray(q_lens, dtype=np.int64)
            ends = np.cumsum(q)
            first = ends - q                               # where each entry's tokens begin
            st = np.asarray(starts, dtype=np.int64)
            cu[1:] = ends
            tseq[:] = np.repeat(np.arange(S), q)
            qs[:] = st
            sl[:] = [e.request.cache.slot for e in entries]
            linear = getattr(self.position, "default_is_linear", False)
            single = np.fromiter((n == 1 and e.positions is None and linear for e, n in zip(entries, q_lens)),
                                 dtype=bool, count=S)
            last = np.zeros(S, dtype=np.int64)
            if single.any():
                which = np.nonzero(single)[0]
                ids = np.fromiter((entries[i].tokens[0] for i in which), dtype=np.int64, count=len(which))
                if ids.min() < 0 or ids.max() >= self.vocab_size:
                    raise ValueError(f"token id outside [0, {self.vocab_size}) in a step")
                place = st[which] + np.fromiter((entries[i].request.cache.position_offset for i in which), dtype=np.int64,
                                                count=len(which))
                tok[first[which]] = ids
                pos[:, first[which]] = place
                last[which] = place
            r = 0
            for i, (e, n, s) in enumerate(zip(entries, q_lens, starts)):
                at = int(first[i])
                if not single[i]:
                    ids = np.asarray(e.tokens, dtype=np.int64)
                    if ids.min() < 0 or ids.max() >= self.vocab_size:
                        raise ValueError(f"request {e.request.request_id!r}: token id outside [0, {self.vocab_size})")
                    tok[at:at + n] = ids
                    cache = e.request.cache
                    if e.positions is None:
                        pos[:, at:at + n] = self.position.default_positions(s, n, cache.position_offset)
                    else:
                        p = np.asarray(e.positions)
                        k = p.shape[1] if p.ndim == 2 else -1
                        if p.ndim != 2 or p.shape[0] != self.axes or not 0 < k <= n:
                            raise ValueError(f"positions must be [{self.axes}, 1..{n}], got {p.shape}")
                        pos[:, at:at + k] = p
                        if k < n:     # plain text after tokens that brought their positions
                            offset = self.position.offset_after(max(cache.max_position, int(p.max())), s + k)
                            pos[:, at + k:at + n] = self.position.default_positions(s + k, n - k, offset)
                    last[i] = int(pos[:, at:at + n].max())
                for w_ in e.want:
                    if not 0 <= int(w_) < n:
                        raise ValueError(f"wanted place {w_} is outside the {n} tokens of the entry")
                    rows[r] = at + int(w_)
                    r += 1
            last_position = last.tolist()
            for g, gs, gt in zip(groups, g_slot, g_tab):
                for i, (e, n, s) in enumerate(zip(entries, q_lens, starts)):
                    table = e.request.block_table(g.index)
                    at = int(first[i])
                    if n == 1:
                        gs[at] = table[s // ps] * ps + s % ps
                    else:
                        logical = np.arange(s, s + n)
                        gs[at:at + n] = table[logical // ps] * ps + logical % ps
                    gt[i, :len(table)] = table
                    gt[i, len(table):] = 0

        return lambda tokens=None, device_ids=None: self._run_packed(
            tokens, entries, q_lens, starts, widths, graph_key, off, N, S, M, ps, tok, tok_s, pos_s, tseq_s, cu_s, qs_s, sl_s,
            rows_s, g_slot_s, g_tab_s, plan_s, last_position, pad_cache, device_ids)

    def _open_padding(self):
        """A request of one token for the rows that fill a captured step's batch, or None when no
        slot or page is free for it.  It is closed again when the step has been launched."""
        try:
            cache = self.cache.open()
        except Exception:
            return None
        try:
            self.cache.ensure(cache, 1)
        except Exception:
            self.cache.close(cache)
            return None
        return cache

    def _run_packed(self, tokens, entries, q_lens, starts, widths, graph_key, off, N, S, M, ps, tok, tok_s, pos_s, tseq_s,
                    cu_s, qs_s, sl_s, rows_s, g_slot_s, g_tab_s, plan_s, last_position, pad_cache=None, device_ids=None):
        real = len(entries)
        if device_ids is not None and (tokens is not None or S != N or device_ids.dtype != torch.int32
                                       or device_ids.numel() < real or device_ids.device != self.device):
            raise ValueError(f"a prepared step takes {real} int32 token ids on {self.device}, or ids from the host")
        if tokens is not None:
            ids = np.asarray(tokens, dtype=np.int64)
            if ids.shape != (real,) or S != N or ids.min() < 0 or ids.max() >= self.vocab_size:
                raise ValueError(f"a prepared step needs {real} token ids in [0, {self.vocab_size})")
            tok[:real] = ids
        dev = self._device_ints
        dev[:off].copy_(self._staging[:off], non_blocking=True)
        if device_ids is not None:
            dev[tok_s[0]:tok_s[0] + real].copy_(device_ids[:real], non_blocking=True)
        if self._staging_free is not None:
            self._staging_free.record()

        def d(span, shape=None):
            t = dev[span[0]:span[0] + span[1]]
            return t if shape is None else t.view(shape)

        make_ctx = lambda: StepContext(
            dtype=self.dtype, device=self.device, n_tokens=N, n_seqs=S,
            token_ids=d(tok_s), positions=d(pos_s, (self.axes, N)), token_seq=d(tseq_s), cu_q=d(cu_s),
            q_start_pos=d(qs_s), slot_ids=d(sl_s), logit_rows=d(rows_s) if M else None,
            logits_every_row=(M == N == S and all(list(e.want) == [0] for e in entries)),
            max_q_len=max(q_lens),
            max_kv_len=(max(widths) * ps if graph_key else max(s + n for s, n in zip(starts, q_lens))),
            group_kv_slot=[d(s_) for s_ in g_slot_s],
            group_block_table=[d(s_, (S, w)) for s_, w in zip(g_tab_s, widths)],
            cache=self.cache,
            plans=self._plan_views(plan_s, d),
            host_q_lens=q_lens, host_q_start=starts,
            host_slots=[e.request.cache.slot for e in entries] + ([pad_cache.slot] * (S - real) if S > real else []),
        )
        try:
            if graph_key is None:
                logits = self.model.forward(make_ctx())
            else:
                logits = self._replay(graph_key, make_ctx, (dev.data_ptr(), off))
        finally:
            # the rows that filled the batch: their page goes back (whoever gets it next writes it
            # behind this step on the stream); their logits are dropped
            self._close_padding()
        if S > real:
            logits = logits[:real]

        if self.device.type == "cuda":
            self._error_host.copy_(kernels.error_flag(self.device), non_blocking=True)
        for e, n, p_max in zip(entries, q_lens, last_position):
            # where plain text that follows resumes is the position encoding's to say
            c = e.request.cache
            c.max_position = max(c.max_position, p_max)
            self.cache.advance(c, n)
            c.position_offset = self.position.offset_after(c.max_position, c.num_tokens)
        self.steps += 1
        return logits

    @staticmethod
    def _plan_views(plan_s, d):
        plans: Dict[object, Dict[str, Optional[torch.Tensor]]] = {}
        for (key, name), span in plan_s.items():
            plans.setdefault(key, {})[name] = d(span) if span[1] else None
        return plans

    def check_kernel_errors(self) -> None:
        """Raises if a kernel of a step whose results have reached the host gave up one of its
        bounded waits (the flag travels to the host after every step, behind the step's kernels
        and before anything that reads its logits).  The flag is cleared, so that one failed
        step does not condemn the steps after it."""
        code = int(self._error_host[0])
        if code != 0:
            self._error_host.zero_()
            if self.device.type == "cuda":
                kernels.reset_after_error(self.device)
            raise kernels.KernelError(f"a kernel of a step gave up waiting (code {code}); the step's results are invalid")
