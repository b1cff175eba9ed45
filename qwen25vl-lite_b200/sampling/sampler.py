"""Choosing the next token of every row of a logits matrix, on the device.

Order of operations as in the reference (src/qwen25vl_lite/sampling.py:44-106;
src/qwen25vl_lite/engine.py:813-821): penalties on the logits, then for temperature > 0
``scores = logits / T``, top-k, min-p, top-p, softmax and one draw; temperature 0 is argmax.

Greedy rows, plain temperature rows and penalties run in the engine's own kernels
(``csrc/sampling.cu``), all rows of a step in one launch.  A row that asks for top-k, min-p
or top-p is first narrowed with device-side sort and scan primitives and then drawn by the
same kernel.  The draw is keyed by ``(seed, index of the token being drawn)`` like the
reference's ``seed + len(outputs)`` generator (engine.py:823-829); a request without a seed
gets a fresh random one.
"""

from __future__ import annotations

import secrets
from collections import Counter
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import kernels
from .params import SamplingParams


def new_seed() -> int:
    return secrets.randbits(63)


def filter_scores(scores: torch.Tensor, top_k: int, min_p: float, top_p: float) -> torch.Tensor:
    """One row of scaled logits -> the same row with dropped tokens at -inf
    (sampling.py:74-101: top-k keeps ties with the k-th value; min-p compares with
    ``min_p * max probability``; top-p keeps the smallest sorted prefix whose cumulative
    probability reaches top_p, the crossing token included)."""
    neg_inf = torch.full_like(scores, float("-inf"))
    if top_k and top_k > 0:
        k = min(int(top_k), scores.numel())
        kth = torch.topk(scores, k).values[-1]
        scores = torch.where(scores < kth, neg_inf, scores)
    if min_p > 0:
        probs = torch.softmax(scores, dim=-1)
        scores = torch.where(probs < min_p * probs.max(), neg_inf, scores)
    if top_p < 1.0:
        sorted_scores, order = torch.sort(scores, descending=True, stable=True)
        cumulative = torch.cumsum(torch.softmax(sorted_scores, dim=-1), dim=-1)
        # keep everything up to and including the first position whose cumulative >= top_p
        keep = torch.ones_like(cumulative, dtype=torch.bool)
        keep[1:] = cumulative[:-1] < top_p
        filtered = torch.where(keep, sorted_scores, torch.full_like(sorted_scores, float("-inf")))
        scores = torch.empty_like(scores).scatter_(0, order, filtered)
    return scores


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._host = None                     # pinned buffer the sampled ids are copied to

    def _upload(self, values, dtype) -> torch.Tensor:
        return torch.tensor(values, dtype=dtype).to(self.device, non_blocking=True)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               token_indices: Sequence[int], previous: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """``logits`` [rows, vocab] float32 on the device; one token id per row.

        ``seeds[r]`` and ``token_indices[r]`` key the draw of row r; ``previous[r]`` are the
        tokens generated so far (only read for rows with penalties)."""
        return self.collect(self.sample_async(logits, params, seeds, token_indices, previous))

    def collect(self, pending) -> List[int]:
        """Waits for the draw that ``sample_async`` started and returns its token ids."""
        if pending is None:
            return []
        host, event, rows = pending[:3]
        if event is None:
            return host
        event.synchronize()
        return host[:rows].tolist()

    @staticmethod
    def device_ids(pending):
        """The ids a pending draw leaves on the device (int32 [rows]), for a next step that is fed
        from there before the ids have reached the host; None when there are none."""
        return pending[3] if isinstance(pending, tuple) and len(pending) > 3 else None

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                     token_indices: Sequence[int], previous: Optional[Sequence[Sequence[int]]] = None):
        """Starts the draw and the copy of its result to pinned host memory; the host is free until
        ``collect``.  Returns (pinned ids, event of the copy, rows, ids on the device)."""
        rows = logits.shape[0]
        if rows == 0:
            return None
        if any(p.has_penalties for p in params):
            logits = logits.clone()
            ids: List[int] = []
            counts: List[int] = []
            offsets = [0]
            for p, prev in zip(params, previous or [[]] * rows):
                if p.has_penalties and prev:
                    c = Counter(int(t) for t in prev)
                    ids += list(c.keys())
                    counts += list(c.values())
                offsets.append(len(ids))
            if ids:
                kernels.apply_penalties(
                    logits, self._upload(ids, torch.int32), self._upload(counts, torch.int32),
                    self._upload(offsets, torch.int32),
                    self._upload([p.repetition_penalty for p in params], torch.float32),
                    self._upload([p.presence_penalty for p in params], torch.float32),
                    self._upload([p.frequency_penalty for p in params], torch.float32))
        temps = [float(p.temperature) for p in params]
        if any(p.has_filters for p in params):
            logits = logits.clone() if not any(p.has_penalties for p in params) else logits
            for r, p in enumerate(params):
                if p.has_filters:
                    logits[r] = filter_scores(logits[r] / p.temperature, p.top_k, p.min_p, p.top_p)
                    temps[r] = 1.0
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(t <= 0 for t in temps):
            kernels.sample_rows(logits, None, None, None, out)
        else:
            seed_arr = np.asarray([int(s) & ((1 << 64) - 1) for s in seeds], dtype=np.uint64).view(np.int64)
            kernels.sample_rows(logits, self._upload(temps, torch.float32),
                                torch.from_numpy(seed_arr).to(self.device, non_blocking=True),
                                self._upload([int(t) for t in token_indices], torch.int32), out)
        if self.device.type != "cuda":
            return out.tolist(), None, rows, out
        if self._host is None or self._host.numel() < rows:
            self._host = torch.empty(max(rows, 64), dtype=torch.int32, pin_memory=True)
        self._host[:rows].copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return self._host, event, rows, out
