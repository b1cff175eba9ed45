"""The scheduler's decisions, on the host: a fake step function records what it is fed and
"generates" a token that depends on every token it has seen, so a lost or repeated token
changes the output."""

from typing import List

import pytest

from qwen25vl_lite.cache import CacheManager, StopNeeds
from qwen25vl_lite.config import EngineConfig
from qwen25vl_lite.engine.runner import Request
from qwen25vl_lite.engine.scheduler import LLMEngine
from qwen25vl_lite.parts import KVCacheNeed
from qwen25vl_lite.sampling import SamplingParams

VOCAB = 1000


def next_token(history: List[int]) -> int:
    return (sum((i + 1) * t for i, t in enumerate(history)) * 31 + len(history)) % VOCAB


class FakeRunner:
    """The step function's face without a model: checks that every request's tokens arrive
    in order, each exactly once, with the pages they need already held."""

    def __init__(self, num_pages, page_size, max_requests, window=None):
        self.cache = CacheManager([StopNeeds(KVCacheNeed(1, 16, window))], num_pages, page_size, max_requests)
        self.history = {}
        self.batches = []

    def open_request(self, rid):
        self.history[rid] = []
        return Request(rid, self.cache.open())

    def close_request(self, req):
        self.cache.close(req.cache)
        del self.history[req.request_id]

    def step(self, entries):
        self.batches.append([(e.request.request_id, len(e.tokens), len(e.want)) for e in entries])
        rows = []
        for e in entries:
            h = self.history[e.request.request_id]
            assert len(h) == e.request.cache.num_tokens
            assert self.cache.pages_missing(e.request.cache, len(h) + len(e.tokens)) == [0]
            for i, t in enumerate(e.tokens):
                h.append(int(t))
                if i in e.want:
                    rows.append(list(h))
            self.cache.advance(e.request.cache, len(e.tokens))
        self.cache.check([r for r in self._live()])
        return rows

    def _live(self):
        return [r for r in self._requests]

    _requests: list = []


class FakeSampler:
    def sample(self, rows, params, seeds, token_indices, previous):
        return [next_token(h) for h in rows]


def make_engine(num_pages=64, page_size=4, window=None, eos=None, **cfg):
    ecfg = EngineConfig(num_blocks=num_pages, block_size=page_size, **cfg)
    runner = FakeRunner(num_pages, page_size, ecfg.max_num_seqs, window)
    engine = LLMEngine(runner, FakeSampler(), ecfg, eos_token_id=eos)
    runner._requests = _LiveView(engine)
    return engine, runner


class _LiveView:
    def __init__(self, engine):
        self.engine = engine

    def __iter__(self):
        return iter(s.request.cache for s in self.engine.running if s.request is not None)


def expected(prompt, n):
    h = list(prompt)
    out = []
    for _ in range(n):
        out.append(next_token(h))
        h.append(out[-1])
    return out


def test_one_request_generates_the_chain():
    engine, runner = make_engine()
    prompt = [5, 9, 2, 7, 7, 1]
    engine.add_request(prompt, SamplingParams(max_tokens=8))
    outs = engine.run_until_complete()
    assert outs[0].output_token_ids == expected(prompt, 8) and outs[0].finish_reason == "length"
    assert runner.batches[0] == [(0, 6, 1)] and all(b == [(0, 1, 1)] for b in runner.batches[1:])
    assert len(runner.batches) == 8                       # first token from the prompt step, then 7 decodes
    assert runner.cache.pages_in_use() == [0] and runner.cache.free_slots == 8
    assert outs[0].metrics["prompt_tokens"] == 6 and outs[0].metrics["completion_tokens"] == 8


def test_prompts_are_cut_under_the_token_budget_and_decodes_go_first():
    engine, runner = make_engine(max_num_batched_tokens=16)
    a = engine.add_request(list(range(1, 11)), SamplingParams(max_tokens=30))
    engine.step()                                          # a's prompt (10 tokens)
    b = engine.add_request(list(range(100, 164)), SamplingParams(max_tokens=4))
    engine.step()
    assert runner.batches[-1] == [(a, 1, 1), (b, 15, 0)]   # one decoded token, the rest of the budget to b's prompt
    engine.step(); engine.step(); engine.step()
    assert [x for batch in runner.batches[2:5] for x in batch if x[0] == b] == [(b, 15, 0), (b, 15, 0), (b, 15, 0)]
    engine.step()
    assert runner.batches[-1] == [(a, 1, 1), (b, 4, 1)]    # the portion that reaches the end samples
    outs = {o.seq_id: o for o in engine.run_until_complete()}
    assert outs[a].output_token_ids == expected(range(1, 11), 30)
    assert outs[b].output_token_ids == expected(range(100, 164), 4)
    assert max(sum(n for _, n, _ in batch) for batch in runner.batches) <= 16


def test_without_chunked_prefill_a_prompt_runs_whole_or_not_at_all():
    engine, runner = make_engine(max_num_batched_tokens=32, enable_chunked_prefill=False)
    engine.add_request(list(range(20)), SamplingParams(max_tokens=2))
    engine.add_request(list(range(20)), SamplingParams(max_tokens=2))
    engine.step()
    assert runner.batches[0] == [(0, 20, 1)]               # the second prompt does not fit beside the first
    engine.run_until_complete()
    engine.add_request(list(range(40)), SamplingParams(max_tokens=2))
    with pytest.raises(RuntimeError, match="changed nothing"):
        engine.run_until_complete(max_stall=8)


def test_admission_is_limited_by_slots_and_first_come_first_served():
    engine, runner = make_engine(max_num_seqs=2)
    ids = [engine.add_request([i + 1] * 5, SamplingParams(max_tokens=3)) for i in range(5)]
    engine.step()
    assert [x[0] for x in runner.batches[0]] == ids[:2] and len(engine.waiting) == 3
    outs = engine.run_until_complete()
    assert sorted(o.seq_id for o in outs) == ids
    assert [o.seq_id for o in outs] == ids                  # same lengths: they finish in arrival order
    for o in outs:
        assert o.output_token_ids == expected(o.prompt_token_ids, 3)


def test_finish_reasons():
    prompt = [3, 1, 4, 1, 5]
    chain = expected(prompt, 10)
    engine, _ = make_engine(eos=chain[2])
    engine.add_request(prompt, SamplingParams(max_tokens=10))
    engine.add_request(prompt, SamplingParams(max_tokens=10, ignore_eos=True))
    engine.add_request(prompt, SamplingParams(max_tokens=10, ignore_eos=True, stop_token_ids=[chain[4]]))
    outs = {o.seq_id: o for o in engine.run_until_complete()}
    assert outs[0].output_token_ids == chain[:3] and outs[0].finish_reason == "stop"
    assert outs[1].output_token_ids == chain and outs[1].finish_reason == "length"
    assert outs[2].output_token_ids == chain[:5] and outs[2].finish_reason == "stop"
    engine, _ = make_engine(max_model_len=8)
    engine.add_request(prompt, SamplingParams(max_tokens=10))
    out = engine.run_until_complete()[0]
    assert len(out.output_token_ids) == 3 and out.finish_reason == "length"     # 5 + 3 = max_model_len


def test_bad_requests_are_refused():
    engine, _ = make_engine(max_model_len=16, num_pages=3)
    with pytest.raises(ValueError, match="empty"):
        engine.add_request([], SamplingParams())
    with pytest.raises(ValueError, match="max_model_len"):
        engine.add_request([1] * 17, SamplingParams())
    with pytest.raises(ValueError, match="stop"):
        engine.add_request([1], SamplingParams(stop=["x"]))
    with pytest.raises(ValueError, match="temperature"):
        engine.add_request([1], SamplingParams(temperature=-1))
    with pytest.raises(ValueError, match="pages"):
        engine.add_request([1] * 13, SamplingParams())      # 4 pages of 4, the pool has 3


def test_pages_run_out_newest_is_preempted_and_continues_exactly():
    prompts = [[i + 1, i + 2, i + 3] * 4 for i in range(4)]           # 12 tokens each
    reference, _ = make_engine(num_pages=256)
    for p in prompts:
        reference.add_request(p, SamplingParams(max_tokens=12))
    want = {o.seq_id: o.output_token_ids for o in reference.run_until_complete()}
    assert reference.stats()["preemptions"] == 0

    engine, runner = make_engine(num_pages=14)                        # 4 x 12 tokens fit (12 pages), growth does not
    for p in prompts:
        engine.add_request(p, SamplingParams(max_tokens=12))
    outs = engine.run_until_complete()
    assert {o.seq_id: o.output_token_ids for o in outs} == want       # nothing lost, nothing repeated
    assert engine.stats()["preemptions"] > 0
    assert max(o.metrics["preemptions"] for o in outs if o.seq_id == 0) == 0     # the oldest is never the victim
    assert runner.cache.pages_in_use() == [0] and runner.cache.free_slots == 8
    recomputed = [b for b in runner.batches for (rid, n, w) in b if n > 12]
    assert recomputed                                                 # prompt + generated came back as one portion


def test_a_waiting_request_never_evicts_a_running_one():
    engine, runner = make_engine(num_pages=8)
    engine.add_request([1] * 20, SamplingParams(max_tokens=4))        # 5 pages, then 6
    engine.step()
    engine.add_request([2] * 20, SamplingParams(max_tokens=4))        # does not fit beside it
    engine.step()
    assert len(engine.running) == 1 and len(engine.waiting) == 1 and engine.stats()["preemptions"] == 0
    outs = engine.run_until_complete()
    assert len(outs) == 2 and engine.stats()["preemptions"] == 0


def test_pool_too_small_for_the_only_running_request():
    engine, _ = make_engine(num_pages=4)
    engine.add_request([1] * 15, SamplingParams(max_tokens=8))        # 15 tokens fit 4 pages, the 17th does not
    with pytest.raises(RuntimeError, match="pool too small"):
        engine.run_until_complete()


def test_window_group_lets_a_long_request_run_in_few_pages():
    engine, runner = make_engine(num_pages=6, window=8, max_num_batched_tokens=8)
    prompt = list(range(1, 41))
    engine.add_request(prompt, SamplingParams(max_tokens=20))         # 60 tokens = 15 pages without a window
    out = engine.run_until_complete()[0]
    assert out.output_token_ids == expected(prompt, 20)
    assert engine.stats()["preemptions"] == 0 and runner.cache.pages_in_use() == [0]


def test_abort_and_stats():
    engine, runner = make_engine()
    a = engine.add_request([1, 2, 3], SamplingParams(max_tokens=50))
    b = engine.add_request([4, 5, 6], SamplingParams(max_tokens=3))
    engine.step()
    assert engine.abort(a) and not engine.abort(99)
    outs = engine.run_until_complete()
    assert [o.seq_id for o in outs] == [b]
    st = engine.stats()
    assert st["finished"] == 1 and st["running"] == 0 and st["kv_blocks_used"] == 0 and st["generated_tokens"] == 4


# ---- the next decode step packed while this one runs ------------------------------------------------
class PreparingRunner(FakeRunner):
    """A step function that also offers ``prepare_decode`` / ``launch_prepared`` and counts them.  Like
    the engine's own it holds something for a prepared step (a request of one page, when a slot and
    a page are free) until that step is launched or the engine says it is dropped."""

    prepared = launched = dropped = 0
    held = None

    def _release(self):
        if self.held is not None:
            self.cache.close(self.held)
            self.held = None

    def step(self, entries):
        assert self.held is None, "a prepared step was neither launched nor dropped before the next step"
        return super().step(entries)

    def prepare_decode(self, requests):
        self.prepared += 1
        assert self.held is None, "a prepared step was neither launched nor dropped before the next was prepared"
        for r in requests:
            assert self.cache.pages_missing(r.cache, r.cache.num_tokens + 1) == [0]      # the engine took the pages first
        if self.cache.free_slots:
            self.held = self.cache.open()
            if self.cache.can_hold(self.held, 1):
                self.cache.ensure(self.held, 1)
            else:
                self._release()
        return list(requests)

    fed_from_device = 0

    def launch_prepared(self, prepared, tokens, device_ids=None):
        from qwen25vl_lite.engine.runner import StepEntry
        self.launched += 1
        self._release()
        if tokens is None:                       # the ids the sampler left "on the device"
            tokens = list(device_ids)
            self.fed_from_device += 1
        assert len(tokens) == len(prepared)
        return self.step([StepEntry(r, [t], [0]) for r, t in zip(prepared, tokens)])

    def drop_prepared(self, prepared):
        self.dropped += 1
        self._release()


class AsyncSampler(FakeSampler):
    def sample_async(self, rows, params, seeds, token_indices, previous):
        return [next_token(h) for h in rows]

    def collect(self, pending):
        return pending


class DeviceFeedSampler(FakeSampler):
    """Like the engine's sampler it says where the drawn ids lie before the host has them, so the
    engine can launch the next step from there without waiting for them."""

    def sample_async(self, rows, params, seeds, token_indices, previous):
        ids = [next_token(h) for h in rows]
        return ids, None, len(ids), list(ids)

    def collect(self, pending):
        return pending[0]

    @staticmethod
    def device_ids(pending):
        return pending[3]


def test_prepared_decode_steps_change_nothing():
    """With a step function that can pack a decode step ahead, the engine uses it whenever the
    next batch is known (all running requests decode, nothing waits, nobody ends by length), drops
    it when a request ends by its token or a new one arrives, and the outputs are those of plain
    scheduling: no token lost, repeated or out of order, pages right at every step."""
    prompts = [[5, 6, 7], list(range(20, 31)), [9] * 6, [1, 2]]
    lengths = [9, 14, 5, 11]
    eos = next_token([5, 6, 7] + expected([5, 6, 7], 4))                    # request 0 ends by its 5th token
    ecfg = EngineConfig(num_blocks=64, block_size=4, max_num_seqs=3)
    runner = PreparingRunner(64, 4, ecfg.max_num_seqs + 1)
    engine = LLMEngine(runner, AsyncSampler(), ecfg, eos_token_id=eos)
    runner._requests = _LiveView(engine)
    ids = [engine.add_request(p, SamplingParams(max_tokens=n, ignore_eos=i != 0)) for i, (p, n) in enumerate(zip(prompts[:3], lengths))]
    outs = {}
    late = None
    for step in range(200):
        if step == 6:
            late = engine.add_request(prompts[3], SamplingParams(max_tokens=lengths[3], ignore_eos=True))   # arrives mid-run
        for o in engine.step():
            outs[o.seq_id] = o
        if not engine.has_work():
            break
    assert runner.launched > 5 and runner.prepared >= runner.launched         # preparations may be dropped,
    assert runner.dropped == runner.prepared - runner.launched                # and the step function was told of each
    want0 = expected(prompts[0], lengths[0])
    assert outs[ids[0]].output_token_ids == want0[:want0.index(eos) + 1] and outs[ids[0]].finish_reason == "stop"
    for i in (1, 2):
        assert outs[ids[i]].output_token_ids == expected(prompts[i], lengths[i])
    assert outs[late].output_token_ids == expected(prompts[3], lengths[3])
    runner.cache.check([])


def test_next_step_is_launched_before_the_bookkeeping_and_survives_an_abort():
    """When the drawn tokens end no request, the engine hands the packed next step to the device
    inside the same ``step`` call (the next call starts at its sampling).  A request aborted while
    such a step runs draws nothing from it; the others go on as if nothing had happened."""
    prompts = [[5, 6, 7], list(range(20, 31)), [9] * 6]
    ecfg = EngineConfig(num_blocks=64, block_size=4, max_num_seqs=3)
    runner = PreparingRunner(64, 4, ecfg.max_num_seqs + 1)
    engine = LLMEngine(runner, AsyncSampler(), ecfg, eos_token_id=None)
    runner._requests = _LiveView(engine)
    ids = [engine.add_request(p, SamplingParams(max_tokens=12, ignore_eos=True)) for p in prompts]
    outs = {}
    early = 0
    for step in range(200):
        before = runner.launched
        for o in engine.step():
            outs[o.seq_id] = o
        if engine._launched is not None:
            early += 1
            assert runner.launched == before + 1 or runner.launched == before + 2     # this call's own launch, and the next one's
        if step == 5:
            assert engine._launched is not None and engine.abort(ids[1])               # its step is on the device
        if not engine.has_work():
            break
    assert early >= 5
    assert ids[1] not in outs
    for i in (0, 2):
        assert outs[ids[i]].output_token_ids == expected(prompts[i], 12)
    runner.cache.check([])


@pytest.mark.parametrize("sampler", [AsyncSampler, DeviceFeedSampler])
@pytest.mark.parametrize("seed", range(8))
def test_random_arrivals_stops_and_aborts_with_steps_packed_and_launched_ahead(seed, sampler):
    """Requests of random lengths arrive at random steps, some end by a stop token, some are
    aborted, the pool is small enough for preemptions: every finished request has exactly the
    tokens of its own history (the fake step function derives each token from all before it), no
    page is lost, and the steps that are packed or launched ahead are really used.  With a sampler
    that leaves its ids "on the device" the next step is launched before the host knows whether a
    request has just ended by its token: such a request draws nothing from that step."""
    import random
    rng = random.Random(seed)
    ecfg = EngineConfig(num_blocks=40, block_size=4, max_num_seqs=4, max_num_batched_tokens=16)
    runner = PreparingRunner(40, 4, ecfg.max_num_seqs + 1)
    engine = LLMEngine(runner, sampler(), ecfg, eos_token_id=None)
    runner._requests = _LiveView(engine)
    plans, outs, aborted = {}, {}, set()
    to_add = 10
    for step in range(2000):
        if to_add and rng.random() < 0.3:
            prompt = [rng.randrange(VOCAB) for _ in range(rng.randint(1, 20))]
            n = rng.randint(1, 25)
            full = expected(prompt, n)
            stop = full[rng.randrange(len(full))] if rng.random() < 0.4 else None      # ends early by this token
            sid = engine.add_request(prompt, SamplingParams(max_tokens=n, ignore_eos=True,
                                                            stop_token_ids=(stop,) if stop is not None else ()))
            plans[sid] = (prompt, n, stop)
            to_add -= 1
        if engine.running and rng.random() < 0.03:
            victim = rng.choice(engine.running).seq_id
            assert engine.abort(victim)
            aborted.add(victim)
        for o in engine.step():
            outs[o.seq_id] = o
        if not to_add and not engine.has_work():
            break
    assert not engine.has_work()
    for sid, (prompt, n, stop) in plans.items():
        if sid in aborted:
            assert sid not in outs
            continue
        full = expected(prompt, n)
        want = full[:full.index(stop) + 1] if stop is not None else full
        assert outs[sid].output_token_ids == want, (sid, prompt, n, stop)
        assert outs[sid].finish_reason == ("stop" if stop is not None else "length")
    assert runner.launched > 0 and runner.dropped == runner.prepared - runner.launched and runner.held is None
    assert (runner.fed_from_device > 0) == (sampler is DeviceFeedSampler)
    runner.cache.check([])


def test_steps_are_packed_ahead_while_a_request_waits_that_cannot_join():
    """Two seats, three requests: while the third waits for a seat the two that run decode in steps
    that are packed and launched ahead (the next step is known: nobody can join it); when one of
    them ends, the one that waits joins the very next step, and every request has its own tokens."""
    prompts = [[5, 6, 7], [9] * 6, [1, 2, 3, 4]]
    lengths = [6, 14, 5]
    ecfg = EngineConfig(num_blocks=64, block_size=4, max_num_seqs=2)
    runner = PreparingRunner(64, 4, ecfg.max_num_seqs + 1)
    engine = LLMEngine(runner, DeviceFeedSampler(), ecfg, eos_token_id=None)
    runner._requests = _LiveView(engine)
    ids = [engine.add_request(p, SamplingParams(max_tokens=n, ignore_eos=True)) for p, n in zip(prompts, lengths)]
    outs, ahead_while_waiting, joined_at, ended_at = {}, 0, None, None
    for step in range(200):
        before = runner.launched
        for o in engine.step():
            outs[o.seq_id] = o
            if o.seq_id == ids[0] and ended_at is None:
                ended_at = step
        if engine.waiting and runner.launched > before:
            ahead_while_waiting += 1
        if joined_at is None and any(s.seq_id == ids[2] for s in engine.running):
            joined_at = step
        if not engine.has_work():
            break
    assert ahead_while_waiting >= 3
    assert ended_at is not None and joined_at is not None and joined_at <= ended_at + 1
    for i in range(3):
        assert outs[ids[i]].output_token_ids == expected(prompts[i], lengths[i])
    runner.cache.check([])
