"""Trace replay: given token ids go through the model step by step and the logits at the
wanted places are written out.  Nothing is sampled.

It drives the same model, step function, cache and kernels as generation; it has no
forward pass, cache or loader of its own.  The reference has no such tool; its nearest are
the hand-driven loops of tests/test_chunked_prefill.py:44-68,108-152.

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
``entries[i].positions`` ([axes][len(tokens)]) may give explicit positions (image spans).
Output: ``<out>/<step>.f32`` = little-endian float32 [wanted, vocab] for every step that
wants something, and a flushed line ``done <step>`` after every step.
"""

from __future__ import annotations

import json
import os
import sys
from typing import Dict, Iterable, Optional, TextIO

import numpy as np
import torch

from ..weights.loader import load_model
from .runner import ModelRunner, Request, StepEntry


class TraceSession:
    def __init__(self, runner: ModelRunner, out_dir: Optional[str]):
        self.runner = runner
        self.out_dir = out_dir
        self.requests: Dict[str, Request] = {}
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)

    def run_step(self, record: dict) -> Optional[np.ndarray]:
        entries = []
        for e in record.get("entries", []):
            rid = e["id"]
            req = self.requests.get(rid)
            if req is None:
                req = self.requests[rid] = self.runner.open_request(rid)
            positions = None if e.get("positions") is None else np.asarray(e["positions"], dtype=np.int64)
            entries.append(StepEntry(req, list(e["tokens"]), list(e.get("want", ())), positions))
        logits = self.runner.step(entries) if entries else None
        out = None
        if logits is not None:
            out = logits.to("cpu").numpy().astype("<f4", copy=False)
        elif self.runner.device.type == "cuda":
            torch.cuda.synchronize(self.runner.device)
        self.runner.check_kernel_errors()          # before the logits count: did a kernel give up a wait?
        if out is not None and self.out_dir:
            out.tofile(os.path.join(self.out_dir, f"{record['step']}.f32"))
        for rid in record.get("end", []):
            req = self.requests.pop(rid, None)
            if req is None:
                raise ValueError(f"step {record.get('step')}: request {rid!r} ends but is not live")
            self.runner.close_request(req)
        return out


def replay(lines: Iterable[str], runner: ModelRunner, out_dir: Optional[str], reply: TextIO = sys.stdout) -> None:
    session = TraceSession(runner, out_dir)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        session.run_step(record)
        reply.write(f"done {record['step']}\n")
        reply.flush()


def make_runner(model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, max_requests: int = 8,
                device: str = "cuda:0") -> ModelRunner:
    """A runner whose pools hold ``max_tokens`` tokens (a multiple of 64) per cache group."""
    if max_tokens <= 0 or max_tokens % 64:
        raise ValueError("--max-tokens must be a positive multiple of 64")
    if page_size <= 0 or 64 % page_size:
        raise ValueError("the page size must divide 64")
    _, model = load_model(model_dir, dtype, device)
    return ModelRunner(model, max_tokens // page_size, page_size, max_requests)


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description="feed given token ids through a model, write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--page-size", type=int, default=16, help="tokens in a cache page (divides 64)")
    ap.add_argument("--max-requests", type=int, default=8, help="per-request state slots")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    runner = make_runner(args.model, args.dtype, args.max_tokens, args.page_size, args.max_requests, args.device)
    replay(sys.stdin, runner, args.out)
    return 0
