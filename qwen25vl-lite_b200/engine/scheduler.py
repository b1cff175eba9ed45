"""Continuous batching above the step function: admit, cut prompts into portions under a
token budget, decode, finish, free; and what happens when pages run out.

After the reference's ``LLMEngine`` (src/qwen25vl_lite/engine.py:489-937), with these
decisions of its own:

* one step is one batch.  Every running request has ``pending`` tokens not yet in the
  cache (a whole prompt, the rest of one, or the one token it generated last); the step
  feeds ``min(pending, budget)`` of them and samples when the portion reaches the end.
  Decoded tokens are taken first (one each), prompts share what is left of
  ``max_num_batched_tokens``, continuing prompts before new admissions, all first come
  first served.  (The reference's budget counts prompt tokens only and each portion is a
  forward pass of its own, engine.py:631-698, 748-778.)
* a request whose prompt completes in a step samples its first token from that step and
  decodes from the next one on (the reference also decodes it in the same iteration,
  engine.py:780-805).
* pages run out: a waiting request is only admitted when its first portion fits, and
  never by evicting another.  When a *running* request cannot get the pages for its next
  tokens, the newest running request (lowest priority first) is preempted: its pages and
  state slot are given back and it returns to the front of the waiting queue with
  ``prompt + generated`` as the tokens to recompute, positions and sampling keys
  unchanged, so it continues exactly where it stopped.  (The reference's recompute
  re-runs the prompt only and loses the generated tokens' keys, engine.py:713-718.)
  If the request that lacks pages is the only one running, nothing can be freed:
  ``RuntimeError("pool too small ...")``.
* finishing: EOS unless ``ignore_eos``, ``stop_token_ids``, ``max_tokens``,
  ``prompt + output >= max_model_len`` (engine.py:831-872).
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence as Seq

import numpy as np

from ..cache.page_pool import OutOfPages
from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import new_seed
from .runner import Request, StepEntry


@dataclass
class RequestOutput:
    """A finished request as its caller sees it.  The attribute names (and the keys of
    ``metrics``) are those of the reference's record (src/qwen25vl_lite/engine.py:96-112), so code
    written against that engine reads these unchanged.  ``finish_reason`` is ``"stop"`` (the
    end-of-sequence token or one of ``stop_token_ids``) or ``"length"`` (``max_tokens`` or the
    engine's ``max_model_len``)."""

    seq_id: int
    prompt_token_ids: List[int]
    output_token_ids: List[int]
    finish_reason: str
    metrics: Dict[str, float] = field(default_factory=dict)

    num_prompt_tokens = property(lambda self: len(self.prompt_token_ids))
    num_output_tokens = property(lambda self: len(self.output_token_ids))

    @classmethod
    def of(cls, seq: "Sequence", reason: str, now: float) -> "RequestOutput":
        first = seq.first_token_at if seq.first_token_at is not None else now
        timing = {"ttft_s": max(first - seq.arrival, 0.0), "elapsed_s": max(now - seq.arrival, 0.0)}
        counts = {"prompt_tokens": float(len(seq.prompt_token_ids)), "completion_tokens": float(len(seq.output_token_ids)),
                  "preemptions": float(seq.preemptions)}
        return cls(seq.seq_id, list(seq.prompt_token_ids), list(seq.output_token_ids), reason, {**counts, **timing})


@dataclass(eq=False)          # a request is equal to itself only: membership tests must not compare token lists
class Sequence:
    seq_id: int
    prompt_token_ids: List[int]
    params: SamplingParams
    seed: int
    prompt_positions: Optional[np.ndarray] = None      # [axes, len(prompt)] or None (plain text)
    priority: int = 0
    output_token_ids: List[int] = field(default_factory=list)
    request: Optional[Request] = None                  # live handle of the step function
    status: str = "waiting"                            # waiting | running | finished
    arrival: float = field(default_factory=time.time)
    first_token_at: Optional[float] = None
    preemptions: int = 0

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_computed(self) -> int:
        return self.request.num_computed if self.request is not None else 0

    @property
    def pending(self) -> int:
        return self.num_tokens - self.num_computed

    def tokens(self, start: int, end: int) -> List[int]:
        p = len(self.prompt_token_ids)
        if end <= p:
            return self.prompt_token_ids[start:end]
        return (self.prompt_token_ids[start:] if start < p else []) + self.output_token_ids[max(start - p, 0):end - p]

    def positions(self, start: int, end: int) -> Optional[np.ndarray]:
        """The positions the prompt brought for tokens [start, end): those of the prompt's share
        of the range, None when the range lies behind the prompt.  Generated tokens (a range may
        reach into them when a preempted request is recomputed) bring none: where they sit
        follows from what came before them, and the step function asks the model's position
        encoding for it."""
        if self.prompt_positions is None or start >= len(self.prompt_token_ids):
            return None
        return self.prompt_positions[:, start:min(end, len(self.prompt_token_ids))]


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    _window: Deque = field(default_factory=lambda: deque(maxlen=64), repr=False)

    def record_step(self, seconds: float, decoded: int) -> None:
        if decoded:
            self._window.append((seconds, decoded))

    @property
    def decode_tokens_per_s(self) -> float:
        t = sum(s for s, _ in self._window)
        return sum(n for _, n in self._window) / t if t > 0 else 0.0


class LLMEngine:
    """``add_request`` / ``step`` / ``run_until_complete`` as in the reference.  ``runner``
    must offer ``cache``, ``open_request``, ``close_request`` and ``step(entries)``;
    ``sampler`` must offer ``sample(logits, params, seeds, token_indices, previous)``."""

    def __init__(self, runner, sampler, engine_cfg: EngineConfig, eos_token_id: Optional[int] = None):
        self.runner = runner
        self.sampler = sampler
        self.ecfg = engine_cfg
        self.eos_token_id = eos_token_id
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.finished: List[RequestOutput] = []
        self.stats_ = EngineStats()
        self._next_id = 0
        self._prepared = None                 # the next decode step, packed ahead (see ``step``)
        self._launched = None                 # the next decode step, already on the device: (logits, its requests)

    # ---- requests ----------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Seq[int], sampling_params: Optional[SamplingParams] = None, *,
                    positions=None, image_spans=None, priority: int = 0) -> int:
        """Registers a request and returns its id.  ``positions`` ([axes, len(prompt)]) or
        ``image_spans`` ([(start, t, h, w)], merged grid units) describe a prompt with image
        runs; without them the prompt is plain text."""
        params = sampling_params or SamplingParams()
        params.validate()
        if params.stop:
            raise ValueError("string stop sequences need a tokenizer; the engine accepts only stop_token_ids")
        ids = [int(t) for t in prompt_token_ids]
        if not ids:
            raise ValueError("prompt is empty")
        if len(ids) > self.ecfg.max_model_len:
            raise ValueError(f"prompt of {len(ids)} tokens exceeds max_model_len {self.ecfg.max_model_len}")
        if image_spans is not None and positions is None:
            positions = self.runner.position.prompt_positions(len(ids), image_spans)
        if positions is not None:
            positions = np.asarray(positions, dtype=np.int64)
            if positions.ndim != 2 or positions.shape[1] != len(ids):
                raise ValueError(f"positions must be [axes, {len(ids)}], got {positions.shape}")
        seq = Sequence(self._next_id, ids, params, params.seed if params.seed is not None else new_seed(),
                       positions, priority)
        probe_pages = -(-len(ids) // self.ecfg.block_size)
        if all(g.window is None for g in self.runner.cache.groups) and probe_pages > self.runner.cache.num_pages:
            raise ValueError(f"prompt of {len(ids)} tokens needs {probe_pages} pages, the pool has "
                             f"{self.runner.cache.num_pages}")
        self._next_id += 1
        self.waiting.append(seq)
        return seq.seq_id

    def abort(self, seq_id: int) -> bool:
        for seq in list(self.running) + list(self.waiting):
            if seq.seq_id == seq_id:
                self._release(seq)
                if seq in self.running:
                    self.running.remove(seq)
                else:
                    self.waiting.remove(seq)
                seq.status = "finished"
                return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- scheduling --------------------------------------------------------------------
    def _release(self, seq: Sequence) -> None:
        if seq.request is not None:
            self.runner.close_request(seq.request)
            seq.request = None

    def _preempt(self, victim: Sequence, scheduled: Dict[int, int]) -> None:
        self.running.remove(victim)
        scheduled.pop(victim.seq_id, None)
        self._release(victim)
        victim.status = "waiting"
        victim.preemptions += 1
        self.stats_.preemptions += 1
        self.waiting.appendleft(victim)

    def _portion(self, seq: Sequence, budget: int) -> int:
        if seq.pending <= budget:
            return seq.pending
        return budget if self.ecfg.enable_chunked_prefill else 0

    def schedule(self) -> Dict[int, int]:
        """Decides this step: ``{seq_id: number of tokens to feed}``; admits and preempts
        as a side effect.  Every chosen portion has its pages."""
        budget = self.ecfg.max_num_batched_tokens
        scheduled: Dict[int, int] = {}
        cache = self.runner.cache
        for want_decode in (True, False):
            for seq in list(self.running):
                if seq.status != "running" or seq.seq_id in scheduled or (seq.pending == 1) != want_decode:
                    continue
                n = self._portion(seq, budget)
                if n <= 0:
                    continue
                while True:
                    try:
                        cache.ensure(seq.request.cache, seq.num_computed + n)
                        break
                    except OutOfPages:
                        victim = min(self.running, key=lambda s: (s.priority, -s.arrival, -s.seq_id))
                        if len(self.running) == 1:
                            raise RuntimeError(
                                f"pool too small: request {seq.seq_id} needs pages for {seq.num_computed + n} tokens "
                                f"and nothing else is running that could give pages back") from None
                        budget += scheduled.get(victim.seq_id, 0)
                        self._preempt(victim, scheduled)
                        if victim is seq:
                            n = 0
                            break
                if n > 0:
                    scheduled[seq.seq_id] = n
                    budget -= n
        while self.waiting and budget > 0 and len(self.running) < self.ecfg.max_num_seqs and cache.free_slots > 0:
            seq = self.waiting[0]
            n = self._portion(seq, budget)
            if n <= 0:
                break
            request = self.runner.open_request(seq.seq_id)
            if not cache.can_hold(request.cache, n):
                self.runner.close_request(request)
                if not self.running:
                    raise RuntimeError(f"pool too small: the first {n} tokens of request {seq.seq_id} do not fit "
                                       f"an empty pool")
                break
            cache.ensure(request.cache, n)
            seq.request = request
            seq.status = "running"
            self.waiting.popleft()
            self.running.append(seq)
            scheduled[seq.seq_id] = n
            budget -= n
        return scheduled

    # ---- stepping ----------------------------------------------------------------------
    def step(self) -> List[RequestOutput]:
        """One scheduling iteration and one batch; returns the requests that finished.

        While the device runs a step whose requests will all decode one more token, the host
        already packs the next step (pages, block tables, positions: everything but the token
        ids), so that between two decode steps only the sampled ids have to travel.  With a sampler
        that says where the drawn ids lie on the device, that next step is launched at once and reads
        them there, before the host has them; a request that its id then ends draws nothing from the
        step that is already running.  Otherwise, when the ids (on the host) end no request, the next
        step is launched before this call does its bookkeeping and returns.  Either way the next call
        starts at that step's sampling (``_launched``)."""
        t0 = time.perf_counter()
        prepared, self._prepared = self._prepared, None
        launched, self._launched = self._launched, None
        entries, samplers = [], []
        decoded = 0
        if launched is not None:
            logits, samplers = launched                    # the step is running already
            decoded = len(samplers)
            self.stats_.decode_tokens += decoded
        elif prepared is not None and not self._could_admit() and [s.seq_id for s in self.running] == prepared[1] \
                and all(s.pending == 1 for s in self.running):
            samplers = list(self.running)
            decoded = len(samplers)
            self.stats_.decode_tokens += decoded
            logits = self.runner.launch_prepared(prepared[0], [s.output_token_ids[-1] for s in samplers])
        else:
            if prepared is not None:
                self._drop(prepared)                       # the batch changed: what was packed ahead is void
            scheduled = self.schedule()
            by_id = {s.seq_id: s for s in self.running}
            for seq_id, n in scheduled.items():
                seq = by_id[seq_id]
                start = seq.num_computed
                reaches_end = start + n == seq.num_tokens
                entries.append(StepEntry(seq.request, seq.tokens(start, start + n), [n - 1] if reaches_end else [],
                                         seq.positions(start, start + n)))
                if reaches_end:
                    samplers.append(seq)
                if n == 1 and seq.output_token_ids:
                    decoded += 1
                    self.stats_.decode_tokens += 1
                else:
                    self.stats_.prefill_tokens += n
            logits = self.runner.step(entries) if entries else None
        done: List[RequestOutput] = []
        if samplers:
            args = (logits, [s.params for s in samplers], [s.seed for s in samplers],
                    [len(s.output_token_ids) for s in samplers], [s.output_token_ids for s in samplers])
            if hasattr(self.sampler, "sample_async"):
                pending = self.sampler.sample_async(*args)
                self._prepared = self._prepare_next(samplers)          # host work under the device's step
                ids = getattr(self.sampler, "device_ids", lambda p: None)(pending)
                if self._prepared is not None and ids is not None:
                    # The drawn ids are on the device and the next step is packed: it goes to the
                    # device now and reads them there, before they have reached the host.  A
                    # request that its id then turns out to end draws nothing from that step (as
                    # one that is aborted while its step runs); nobody ends by length here, or
                    # nothing would have been prepared.
                    next_logits = self.runner.launch_prepared(self._prepared[0], None, device_ids=ids)
                    self._launched, self._prepared = (next_logits, samplers), None
                tokens = self.sampler.collect(pending)
                self._check_step()                         # the step's results are on the host: was it whole?
                if self._prepared is not None and not any(self._ends(seq, int(tok)) for seq, tok in zip(samplers, tokens)):
                    # nobody ends: the next step goes to the device now, the bookkeeping follows under it
                    next_logits = self.runner.launch_prepared(self._prepared[0], [int(tok) for tok in tokens])
                    self._launched, self._prepared = (next_logits, samplers), None
            else:
                tokens = self.sampler.sample(*args)
                self._check_step()
            for seq, token in zip(samplers, tokens):
                if seq.status == "running":                # a request aborted while its step ran draws nothing
                    self._accept(seq, int(token), done)
            if done and self._prepared is not None:
                self._drop(self._prepared)
                self._prepared = None
        self.stats_.steps += 1
        self.stats_.record_step(time.perf_counter() - t0, decoded)
        self.finished.extend(done)
        return done

    def _prepare_next(self, samplers: List[Sequence]):
        """Packs the next step while this one runs, if it is known already: nothing waits, every
        running request has just reached its end (so it decodes one token next), none of them
        ends by length with the token being drawn, and the pages are there.  Returns (what the
        runner prepared, the ids of the requests in order) or None.  A request that ends by its
        token, or anything else that changes the batch, makes ``step`` drop the preparation; the
        pages it took stay with their requests."""
        runner = self.runner
        if not hasattr(runner, "prepare_decode") or len(samplers) != len(self.running) \
                or len(self.running) > self.ecfg.max_num_batched_tokens:
            return None
        for seq in self.running:
            if seq.prompt_positions is not None and seq.num_computed < len(seq.prompt_token_ids):
                return None
            if len(seq.output_token_ids) + 1 >= seq.params.max_tokens or seq.num_tokens + 1 >= self.ecfg.max_model_len:
                return None
        try:
            for seq in self.running:
                runner.cache.ensure(seq.request.cache, seq.num_computed + 1)
        except OutOfPages:
            return None
        if self._could_admit():            # a request that waits would join the next step: that step is not known yet
            return None
        return runner.prepare_decode([seq.request for seq in self.running]), [s.seq_id for s in self.running]

    def _could_admit(self) -> bool:
        """Whether ``schedule`` would take the first waiting request into the next step, given that
        every running request decodes one token in it: a seat, a slot, budget, and pages for its
        first portion (as ``schedule`` asks for them).  While the pool is full the requests that wait
        cannot join, and the next decode step is known all the same."""
        if not self.waiting:
            return False
        cache = self.runner.cache
        if len(self.running) >= self.ecfg.max_num_seqs or cache.free_slots <= 0:
            return False
        budget = self.ecfg.max_num_batched_tokens - len(self.running)
        n = self._portion(self.waiting[0], budget) if budget > 0 else 0
        if n <= 0:
            return False
        pages = -(-n // cache.page_size)                   # what a request that holds nothing yet needs in every group
        return all(g.pool.num_free >= pages for g in cache.groups)

    def _drop(self, prepared) -> None:
        """A step that was packed ahead and will not run: the runner takes back what it held for it."""
        drop = getattr(self.runner, "drop_prepared", None)
        if drop is not None:
            drop(prepared[0])

    def _ends(self, seq: Sequence, token: int) -> bool:
        """Whether this token, drawn now, ends the request by what it is (ends by length are known
        before the token is drawn and keep ``_prepare_next`` from preparing anything)."""
        p = seq.params
        return (self.eos_token_id is not None and token == self.eos_token_id and not p.ignore_eos) \
            or token in (p.stop_token_ids or ())

    def _check_step(self) -> None:
        """Before a step's tokens are accepted: did one of its kernels give up a bounded wait?"""
        check = getattr(self.runner, "check_kernel_errors", None)
        if check is not None:
            check()

    def _length_reason(self, seq: Sequence) -> Optional[str]:
        """Ends that do not depend on which token was drawn."""
        if len(seq.output_token_ids) >= seq.params.max_tokens or seq.num_tokens >= self.ecfg.max_model_len:
            return "length"
        return None

    def _accept(self, seq: Sequence, token: int, done: List[RequestOutput]) -> None:
        """Takes a drawn token into the request and retires the request if that ends it: by the
        token itself first (``_ends``), else by length (src/qwen25vl_lite/engine.py:831-872 has the
        same precedence)."""
        now = time.time()
        if seq.first_token_at is None:
            seq.first_token_at = now
        seq.output_token_ids.append(token)
        self.stats_.generated_tokens += 1
        reason = "stop" if self._ends(seq, token) else self._length_reason(seq)
        if reason is not None:
            self._retire(seq, reason, done, now)

    def _retire(self, seq: Sequence, reason: str, done: List[RequestOutput], now: float) -> None:
        self._release(seq)
        self.running.remove(seq)
        seq.status = "finished"
        self.stats_.finished += 1
        done.append(RequestOutput.of(seq, reason, now))

    # ---- driver ------------------------------------------------------------------------
    def run_until_complete(self, max_steps: int = 1_000_000, max_stall: int = 64) -> List[RequestOutput]:
        """Steps until no request is left and returns every finished request so far.  A scheduler
        that cannot move (for instance a prompt that never fits the step budget with chunking
        off) would spin for ever: after ``max_stall`` steps in a row that changed nothing, and
        after ``max_steps`` steps in all, this raises (the reference guards its loop the same way,
        src/qwen25vl_lite/engine.py:878-905)."""
        idle, seen = 0, self._signature()
        for _ in range(max_steps):
            if not self.has_work():
                break
            self.step()
            now = self._signature()
            idle = idle + 1 if now == seen else 0
            seen = now
            if idle >= max_stall:
                raise RuntimeError(f"{max_stall} steps in a row changed nothing: {len(self.waiting)} request(s) waiting, "
                                   f"{len(self.running)} running; the scheduler cannot place them")
        else:
            if self.has_work():
                raise RuntimeError(f"{max_steps} steps did not finish the requests: {len(self.waiting)} waiting, "
                                   f"{len(self.running)} running")
        self._check_step()
        return self.finished

    def _signature(self):
        """Changes whenever a step moved anything: queue lengths, preemptions, tokens held or generated."""
        work = sum(s.num_computed + len(s.output_token_ids) for s in self.running)
        return (len(self.waiting), len(self.running), len(self.finished), self.stats_.preemptions, work)

    def stats(self) -> Dict[str, float]:
        st = self.stats_
        cache = self.runner.cache
        return {
            "steps": float(st.steps), "prefill_tokens": float(st.prefill_tokens),
            "decode_tokens": float(st.decode_tokens), "generated_tokens": float(st.generated_tokens),
            "preemptions": float(st.preemptions), "finished": float(st.finished),
            "waiting": float(len(self.waiting)), "running": float(len(self.running)),
            "kv_blocks_used": float(max(cache.pages_in_use(), default=0)),
            "kv_blocks_total": float(cache.num_pages),
            "decode_tokens_per_s": st.decode_tokens_per_s,
        }
