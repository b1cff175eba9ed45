"""Measurements of an engine instance: a prefill step, decode steps timed on the device, decode
through the scheduler, and a continuous-batching trace; with the byte and flop counts their
rooflines are taken against.

The reference's harness (bench/run_bench.py:104-108, 208-233) feeds a deterministic pseudo-prompt
through its engine, greedy with ``ignore_eos``, and divides generated tokens by wall time; the
functions here time steps with CUDA events (or the wall clock where the host is part of what is
measured), on seeded uniform-random token ids.  ``bench.py`` at the repository's root and the
``bench`` subcommand of the command line both call these.
"""

from __future__ import annotations

import statistics
import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..ops import kernels
from ..sampling.params import SamplingParams
from .runner import StepEntry


# ---- what a step must move or compute -----------------------------------------------------------
def layer_matrix_params(t: Dict) -> int:
    """Matrix elements of one layer (q, k, v, o, gate, up, down) from a text_config dict."""
    h, d = t["hidden_size"], t["hidden_size"] // t["num_attention_heads"]
    nq, nkv, inter = t["num_attention_heads"], t["num_key_value_heads"], t["intermediate_size"]
    return h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter


def weight_bytes(t: Dict, layers: int, element_size: int = 2) -> int:
    """Bytes of every weight a decode step reads once: the layers' matrices and the output head
    (the embedding table again when tied; either way it is read once, the embedding rows of the
    batch are negligible)."""
    return element_size * (layers * layer_matrix_params(t) + t["vocab_size"] * t["hidden_size"])


def kv_bytes_per_token(t: Dict, layers: int, element_size: int = 2) -> int:
    d = t["hidden_size"] // t["num_attention_heads"]
    return layers * 2 * t["num_key_value_heads"] * d * element_size


def prefill_flops(t: Dict, layers: int, n_tokens: int) -> int:
    """Multiply-adds x 2 of a prompt of ``n_tokens`` whose last position goes through the head:
    the layers' products, causal attention (scores and P.V over i + 1 keys for token i), one row
    of the head."""
    d = t["hidden_size"] // t["num_attention_heads"]
    attention = layers * 4 * t["num_attention_heads"] * d * n_tokens * (n_tokens + 1) // 2
    return n_tokens * layers * 2 * layer_matrix_params(t) + attention + 2 * t["vocab_size"] * t["hidden_size"]


# ---- timed regions ----------------------------------------------------------------------------------
def random_prompts(rng, vocab: int, lengths: Sequence[int]) -> List[List[int]]:
    return [rng.integers(0, vocab, size=int(n)).tolist() for n in lengths]


def time_prefill(runner, n_tokens: int, vocab: int, rng, warmup: int = 3, repeats: int = 5) -> float:
    """Median milliseconds of one step that runs a whole prompt of ``n_tokens`` (logits at its end)."""
    def once():
        req = runner.open_request("prefill")
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ids = random_prompts(rng, vocab, [n_tokens])[0]
        torch.cuda.synchronize()
        a.record()
        runner.step([StepEntry(req, ids, [n_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.close_request(req)
        return a.elapsed_time(b)

    for _ in range(warmup):
        once()
    return statistics.median(once() for _ in range(repeats))


def time_decode_steps(runner, batch: int, prompt_len: int, steps: int, warmup: int, vocab: int, rng,
                      prefill_group: int = 4, settle_s: float = 0.0) -> Dict[str, float]:
    """``steps`` decode steps of ``batch`` requests (after prompts of ``prompt_len``), fed
    back-to-back with given tokens and each followed by the greedy draw, timed on the device."""
    reqs = [runner.open_request(f"d{i}") for i in range(batch)]
    prompts = random_prompts(rng, vocab, [prompt_len] * batch)
    for i in range(0, batch, prefill_group):
        runner.step([StepEntry(r, p, []) for r, p in zip(reqs[i:i + prefill_group], prompts[i:i + prefill_group])])
    feed = rng.integers(0, vocab, size=(steps + warmup, batch))
    out = torch.empty(batch, dtype=torch.int32, device=runner.device)
    if settle_s > 0:
        # The prompts' products run at the power cap and leave the SM clock lowered for some tens of
        # milliseconds; decode steps are what is measured, at the clock they run at by themselves.
        torch.cuda.synchronize()
        time.sleep(settle_s)

    def one(k):
        logits = runner.step([StepEntry(r, [int(feed[k, i])], [0]) for i, r in enumerate(reqs)])
        kernels.sample_rows(logits, None, None, None, out)

    for k in range(warmup):
        one(k)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    launches0 = kernels.launch_count()
    a.record()
    for k in range(warmup, warmup + steps):
        one(k)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    launches = kernels.launch_count() - launches0
    runner.check_kernel_errors()
    for r in reqs:
        runner.close_request(r)
    return {"tokens_per_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
            "context": prompt_len + warmup + steps // 2}


def time_decode_e2e(engine, batch: int, prompt_len: int, steps: int, warmup: int, vocab: int, rng, settle_s: float = 0.0) -> float:
    """Decoded tokens a second through the scheduler: host token ids in, sampled ids out, every
    step; timed with the wall clock around ``steps`` calls of ``engine.step()``."""
    params = SamplingParams(max_tokens=warmup + steps + 8, ignore_eos=True)
    for p in random_prompts(rng, vocab, [prompt_len] * batch):
        engine.add_request(p, params)
    while engine.waiting or any(s.pending > 1 for s in engine.running):
        engine.step()
    if settle_s > 0:                     # as in time_decode_steps: the clock the prompts left lowered comes back
        torch.cuda.synchronize()
        time.sleep(settle_s)
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for s in list(engine.running):
        engine.abort(s.seq_id)
    return batch * steps / dt


def run_trace(engine, prompts: Sequence[Sequence[int]], output_lengths: Sequence[int]) -> Dict[str, float]:
    """A continuous-batching trace: every request arrives at once, request i generates
    ``output_lengths[i]`` greedy tokens (``ignore_eos``); runs until all have finished.  Returns wall
    time, throughputs and the time to first token."""
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p, n in zip(prompts, output_lengths):
        engine.add_request(p, SamplingParams(max_tokens=int(n), ignore_eos=True))
    before = len(engine.finished)
    stats0 = engine.stats()
    engine.run_until_complete()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    outs = engine.finished[before:]
    generated = sum(len(o.output_token_ids) for o in outs)
    prompt_tokens = sum(len(p) for p in prompts)
    ttft = sorted(o.metrics["ttft_s"] for o in outs)
    stats = engine.stats()
    return {"requests": len(outs), "wall_s": wall, "prompt_tokens": prompt_tokens, "generated_tokens": generated,
            "generated_tokens_per_s": generated / wall, "total_tokens_per_s": (generated + prompt_tokens) / wall,
            "ttft_s_median": ttft[len(ttft) // 2], "ttft_s_max": ttft[-1], "steps": stats["steps"] - stats0["steps"],
            "preemptions": stats["preemptions"] - stats0["preemptions"],
            # the reference's figure: generated tokens over the wall time after the last first token
            "decode_tokens_per_s_after_ttft": generated / max(wall - ttft[-1], 1e-9)}


def quick_bench(llm, batch: int, prompt_len: int, steps: int, warmup: int = 3, seed: int = 0) -> Dict[str, Optional[float]]:
    """What the ``bench`` subcommand prints: one prefill and ``steps`` decode steps of ``batch``."""
    rng = np.random.default_rng(seed)
    vocab = llm.runner.vocab_size
    prefill_ms = time_prefill(llm.runner, prompt_len, vocab, rng, warmup=2, repeats=3)
    dec = time_decode_steps(llm.runner, batch, prompt_len, steps, max(warmup, 3), vocab, rng)
    e2e = time_decode_e2e(llm.engine, batch, prompt_len, steps, max(warmup, 3), vocab, rng)
    return {"prefill_tokens_per_s": prompt_len / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
            "decode_tokens_per_s": dec["tokens_per_s"], "decode_ms_per_step": dec["ms_per_step"],
            "decode_tokens_per_s_end_to_end": e2e, "batch": batch, "prompt_len": prompt_len, "steps": steps}
