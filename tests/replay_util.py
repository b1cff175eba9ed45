"""Helpers of the replay tests: traces as lists of step records, an oracle from the plain
implementation, and a driver that runs a trace through ``bin/trace_run``'s own session."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np

from plain import decoder as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def oracle(model_dir: str, requests: Dict[str, Sequence[int]], positions: Dict[str, np.ndarray] = None):
    """Request id -> float64 logits [len, vocab] of the whole sequence, from the plain decoder."""
    cfg, w = plain.load_model_dir(model_dir, np.float64)
    return {rid: plain.forward_logits(cfg, w, ids, None if not positions or rid not in positions else positions[rid])
            for rid, ids in requests.items()}


def whole(requests: Dict[str, Sequence[int]]) -> List[dict]:
    """Each request alone and whole, one step each, all logits wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": list(ids), "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(requests.items())]


def prefill_then_decode(requests: Dict[str, Sequence[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        ids = list(ids)
        head = max(len(ids) - tail, 1)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}],
                      "end": []})
        for i in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def portions(requests: Dict[str, Sequence[int]], sizes: Sequence[int]) -> List[dict]:
    """Each request in portions whose sizes cycle through ``sizes``."""
    steps = []
    for rid, ids in requests.items():
        ids = list(ids)
        at, k = 0, 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[at:at + n], "want": list(range(n))}],
                          "end": []})
            at += n
            k += 1
        steps[-1]["end"] = [rid]
    return steps


def mixed(requests: Dict[str, Sequence[int]], seed: int, max_live: int = 4, decode_tail: int = 6,
          chosen_share: float = 0.75, longest: int = 24) -> List[dict]:
    """Up to ``max_live`` requests at a time; every step takes a random subset of the live
    ones (each with probability ``chosen_share``) and gives each a portion of random size (two
    to ``longest`` - 1 tokens) while it is in its prompt, single tokens over its last
    ``decode_tail`` tokens; a finished request ends and the next one starts, so pages are used
    again."""
    rng = np.random.default_rng(seed)
    todo = list(requests.items())
    live: Dict[str, List] = {}
    steps = []
    while todo or live:
        while todo and len(live) < max_live:
            rid, ids = todo.pop(0)
            live[rid] = [list(ids), 0]
        chosen = [rid for rid in live if rng.random() < chosen_share] or [next(iter(live))]
        entries, end = [], []
        for rid in chosen:
            ids, at = live[rid]
            left = len(ids) - at
            if left <= decode_tail:
                n = 1
            else:
                n = int(min(rng.integers(2, longest), left - decode_tail))
            entries.append({"id": rid, "tokens": ids[at:at + n], "want": list(range(n))})
            live[rid][1] = at + n
            if at + n == len(ids):
                end.append(rid)
        for rid in end:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps: List[dict]) -> int:
    """Most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held: Dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def run_in_process(model_dir: str, dtype: str, steps: List[dict], max_tokens: int, page_size: int = 16,
                   max_requests: int = 8):
    """Replays through the engine's trace session; returns {request id: [len, vocab] logits}."""
    from qwen25vl_lite.engine.trace import TraceSession, make_runner

    runner = make_runner(model_dir, dtype, max_tokens, page_size, max_requests)
    session = TraceSession(runner, None)
    return collect(steps, [session.run_step(s) for s in steps]), runner


def collect(steps: List[dict], outputs: List[np.ndarray]) -> Dict[str, np.ndarray]:
    rows: Dict[str, List[np.ndarray]] = {}
    for s, out in zip(steps, outputs):
        r = 0
        for e in s["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(out[r])
                r += 1
    return {rid: np.stack(v) for rid, v in rows.items()}


def run_program(model_dir: str, dtype: str, steps: List[dict], max_tokens: int, out_dir: str, env=None):
    """Replays through the ``bin/trace_run`` program, checking its ``done <step>`` lines."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for s in steps:
        proc.stdin.write(json.dumps(s) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {s['step']}", f"trace_run answered {line!r} to step {s['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    outs = []
    vocab = None
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        if n == 0:
            outs.append(None)
            continue
        flat = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4")
        vocab = flat.size // n
        outs.append(flat.reshape(n, vocab))
    return collect(steps, outs)
