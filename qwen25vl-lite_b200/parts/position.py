"""Multimodal rotary position encoding (MRoPE) of the Qwen2.5-VL text decoder.

Formulas (reference src/qwen25vl_lite/rope.py): ``inv_freq[j] = theta^(-2j/D)`` (:26-33);
the angle of rotary channel j is ``pos[axis(j)] * inv_freq[j]`` in float32 (:48-68) where
the three sections of ``mrope_section`` assign the channels to the axes t, h, w (:71-96);
pairs are (j, j + D/2) (:36-40).  Plain text has the same index on all three axes, and a
decoded token sits at ``tokens computed + rope_delta`` (:238-247).
"""

from __future__ import annotations

from typing import Sequence, Tuple

import numpy as np
import torch

from ..ops import kernels
from .base import PositionEncoding, register_position_encoding


def prompt_positions(num_tokens: int, image_spans: Sequence[Tuple[int, int, int, int]] = ()):
    """Positions [3, num_tokens] of a prompt and its ``rope_delta``.

    ``image_spans`` are ``(start, t, h, w)`` with the grid in merged units: the span covers
    t*h*w tokens from index ``start``.  This restates the reference's ``get_rope_index``
    (rope.py:137-235) for prompts whose image tokens are given by place instead of by id
    (the vision tower that would fill them is not part of this engine): a text run puts
    cursor + i on all axes and advances the cursor by its length; an image run at cursor c
    gets (c + t_idx, c + row, c + col) in t-major, row-major order (rope.py:99-126, interval
    1) and advances the cursor by max(h, w); rope_delta = max(pos) + 1 - num_tokens."""
    cols = []
    cursor = 0
    at = 0
    for start, t, h, w in sorted(image_spans):
        if start < at or start + t * h * w > num_tokens:
            raise ValueError(f"image span {(start, t, h, w)} overlaps another or leaves the prompt")
        run = np.arange(start - at, dtype=np.int64) + cursor
        cols.append(np.stack([run, run, run]))
        cursor += start - at
        grid = np.stack(np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")).reshape(3, -1)
        cols.append(grid.astype(np.int64) + cursor)
        cursor += max(h, w)
        at = start + t * h * w
    run = np.arange(num_tokens - at, dtype=np.int64) + cursor
    cols.append(np.stack([run, run, run]))
    pos = np.concatenate(cols, axis=1)
    delta = int(pos.max()) + 1 - num_tokens if num_tokens else 0
    return pos, delta


@register_position_encoding("mrope")
class MRope(PositionEncoding):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    axes = 3

    def __init__(self, head_dim: int, theta: float, sections: Sequence[int]):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.sections = tuple(int(s) for s in sections)
        if sum(self.sections) * 2 != self.head_dim:
            raise ValueError(f"mrope sections {self.sections} must sum to head_dim/2 = {self.head_dim // 2}")
        self.axes = len(self.sections)
        self.inv_freq = None
        self.axis = None

    def load(self, tensors, device, dtype):
        idx = torch.arange(0, self.head_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (idx / self.head_dim))).to(torch.float32).to(device)
        axis = []
        for a, n in enumerate(self.sections):
            axis += [a] * n
        self.axis = torch.tensor(axis, dtype=torch.int32, device=device)

    # plain text: token i of a request sits at i + offset on every axis, which lets the step
    # function fill the positions of a whole decode batch at once
    default_is_linear = True

    def default_positions(self, start: int, count: int, offset: int):
        run = np.arange(start + offset, start + offset + count, dtype=np.int64)
        return np.broadcast_to(run, (self.axes, count))

    def rope_tables(self):
        """(inv_freq float32 [D/2], axis int32 [D/2]) for kernels that rotate by themselves."""
        return self.inv_freq, self.axis

    def prompt_positions(self, num_tokens: int, image_spans):
        """Positions [3, num_tokens] of a prompt whose image runs are ``(start, t, h, w)``."""
        return prompt_positions(num_tokens, image_spans)[0]

    def rotate_and_store(self, ctx, qkv, nq, nkv, head_dim, kv):
        """kv: the pages and slots of the stop's cache group, or None to store nothing."""
        if head_dim != self.head_dim:
            raise ValueError(f"mrope built for head size {self.head_dim}, mixer has {head_dim}")
        angles = None
        if ctx.dtype == torch.bfloat16:
            # the angles are the same for every layer of the step that shares the tables: the first
            # one to ask computes them (the 32-bit path computes them in place, in every layer)
            key = ("rope_angles", self.inv_freq.data_ptr(), self.axis.data_ptr())
            angles = ctx.shared.get(key)
            if angles is None:
                angles = ctx.shared[key] = kernels.rope_angles(ctx.positions, self.inv_freq, self.axis)
        if kv is None:
            kernels.rope_store(qkv, ctx.positions, self.inv_freq, self.axis, None, None, None, nq, nkv, head_dim, 1, angles)
        else:
            kernels.rope_store(qkv, ctx.positions, self.inv_freq, self.axis, kv.k_pages, kv.v_pages, kv.kv_slot,
                               nq, nkv, head_dim, kv.page_size, angles)
