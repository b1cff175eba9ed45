"""Interfaces of the parts a layer is put together from, and the registries that resolve a
``PartSpec.kind`` to a class.

A part is constructed from its own parameters only (sizes, constants); it never sees a
model configuration and does not know which model it is in.  Four things are asked of it:

* ``tensor_specs()``: the tensors it needs, by the name they carry in a checkpoint
  (relative to the part's prefix), with shape and the kind of random initialisation;
* ``load(tensors, device, dtype)``: take those tensors (CPU views of the file) and keep
  what the kernels want on the device (fused, cast);
* what it needs from the cache manager: pages of keys and values (``cache_need``) and / or
  a fixed-size per-request state (``state_need``); only mixers have either;
* ``forward``: see each class.

Registering a class under a new kind (``MIXERS["my_kind"] = MyMixer``) is all it takes to
use it from a ``ModelSpec``; nothing else in the package names the kinds.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class TensorSpec:
    name: str                       # relative checkpoint name, e.g. "q_proj.weight"
    shape: Tuple[int, ...]
    init: str = "matrix"            # "matrix": N(0, std); "norm": 1 + N(0, std); "bias": N(0, std)
    optional: bool = False          # may be absent from a checkpoint (e.g. a tied head)


@dataclass(frozen=True)
class KVCacheNeed:
    """Pages of keys and values: all keys (window None) or the last ``window`` of them."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per live request, zeroed when the request is admitted."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


class Part:
    # What a part may declare about itself (class attributes); the defaults promise nothing.
    graph_safe = False              # forward is a fixed sequence of this engine's kernels: a step may be captured
    accepts_residual = False        # forward takes ``residual=`` and may add its result into the float32 stream
    accepts_deferred_norm = False   # forward takes an ``ops.linear.DeferredNorm`` to normalise inside its first product

    def tensor_specs(self) -> Sequence[TensorSpec]:
        return ()

    def load(self, tensors: Dict[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        pass

    # Sharing of device tensors between parts (a tied output head reads the embedding table):
    # after ``load`` a part's ``exports()`` are offered to the parts that follow it under their
    # canonical checkpoint names; a part that lists a name in ``imports()`` is handed it through
    # ``receive`` before its own ``load``.
    def exports(self) -> Dict[str, torch.Tensor]:
        return {}

    def imports(self) -> Sequence[str]:
        return ()

    def receive(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    # Work lists for a part's kernels, built per step on the host and packed into the step's one
    # transfer by the step function: a part that wants some returns a key from ``plan_key`` (parts
    # with equal keys share one plan) and int arrays by name from ``plan_step(host)``, ``host``
    # being the step's shape (``engine.runner.HostStep``); it finds their device copies under
    # ``ctx.plan(self)``.  The default asks for nothing.
    def plan_key(self):
        return None

    def plan_step(self, host) -> Dict[str, object]:
        return {}


class Norm(Part):
    """``forward(ctx, x, delta, rows=None) -> h``: x (float32 residual stream, [N, H]) takes
    the pending update ``delta`` first (x += delta, fused), then h = norm(x) in the
    activation dtype.  With ``rows`` (int32 indices) only those rows are produced and x is
    left untouched."""

    def forward(self, ctx, x, delta, rows=None, defer=False):
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions reach queries and keys, and what a token's position is when nobody says.

    A model has one encoding that defines its tokens' positions (``ModelSpec.position``): how many
    integers describe a position (``axes``), and the positions of plain text.  A layer may apply
    another encoding to those same positions (``LayerSpec.position``), or none.

    ``default_positions(start, count, offset)``: positions of ``count`` tokens of plain text
    starting at index ``start`` of a request whose per-request offset is ``offset``
    -> int array [axes, count].
    ``offset_after(max_position, num_tokens)``: the request's offset once ``num_tokens`` tokens
    with positions up to ``max_position`` are in: where plain text resumes after tokens that
    brought positions of their own.
    ``default_is_linear``: set True when ``default_positions`` is ``start + offset + i`` on every
    axis, which lets the step function fill a whole batch of single tokens at once.
    ``rotate_and_store(ctx, qkv, ...)``: encode q and k in place and write k, v to the pages.
    ``rope_tables() -> (inv_freq float32 [D/2], axis int32 [D/2])`` or None: a rotary encoding
    (channel j turns by ``position[axis[j]] * inv_freq[j]``, any number of axes) hands out its
    tables, which lets the fused decode attention kernel do the rotation itself; None (the default)
    sends every step through ``rotate_and_store``.
    ``prompt_positions(num_tokens, image_spans)``: positions of a prompt with image runs; the
    default refuses (an encoding that does not place images).
    """

    axes = 1
    default_is_linear = False

    def default_positions(self, start: int, count: int, offset: int):
        raise NotImplementedError

    def offset_after(self, max_position: int, num_tokens: int) -> int:
        """Plain text resumes one past the largest position seen so far (the reference's
        ``rope_delta = max(pos) + 1 - length``, src/qwen25vl_lite/rope.py:235)."""
        return int(max_position) + 1 - int(num_tokens)

    def rotate_and_store(self, ctx, qkv, nq, nkv, head_dim, kv):
        raise NotImplementedError

    def rope_tables(self):
        return None

    def prompt_positions(self, num_tokens: int, image_spans):
        raise ValueError("image_spans given, but the model's position encoding does not place image runs")


class Mixer(Part):
    """The token-mixing part of a layer.

    ``forward(ctx, h, stop) -> [N, H]`` in the activation dtype.  Every part may declare
    ``graph_safe = True``: its forward is a fixed sequence of this engine's kernels (no loop over
    the batch on the host, no library operator), so a step can be captured into a CUDA graph; a
    model is captured only when all its parts say so.  Two more optional capabilities a
    mixer (or feed-forward) may declare as class attributes: ``accepts_residual`` -- forward
    takes ``residual=`` (the float32 stream) and may add its result into it, returning None;
    ``accepts_deferred_norm`` -- ``h`` may be an ``ops.linear.DeferredNorm`` to be normalised
    inside the part's first product.  ``stop`` is the runtime
    record of the schedule stop being run (``engine.runner.StopRuntime``): ``stop.kv`` gives
    the pages of this stop (or of the stop whose cache it reads) with ``stop.owns_cache``
    telling whether to write this step's keys and values; ``stop.state`` is the fixed-size
    state tensor [max_seqs, *shape] when ``state_need`` asked for one, indexed by
    ``ctx.slot_ids``.  A mixer with state must process a request's tokens in order and must
    give the same result wherever the run of tokens is cut.

    A part whose kernels read per-step work lists may define ``plan_step(host) -> {name: int32
    array}`` (``host.q_lens``, ``host.starts``, ``host.n_tokens``, ``host.n_seqs`` describe the
    step) and ``plan_key()`` (parts with equal keys share one plan).  The step function packs the
    arrays into its one transfer; ``ctx.plan(part)`` returns their device copies by name (None for
    an empty array).  The sizes may depend only on ``q_lens``, so that a captured step finds them at
    the same place in every replay.
    """

    def cache_need(self) -> Optional[KVCacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, ctx, h, stop):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(ctx, h) -> [N, H]`` in the activation dtype."""

    def forward(self, ctx, h):
        raise NotImplementedError


class Block:
    """The arrangement of one layer's parts around the residual stream.

    ``forward(ctx, x, pending, stop) -> pending``: ``x`` is the float32 residual stream,
    ``pending`` an update not yet added to it (or None); the block returns its own last
    update unadded, so the next norm can fuse the addition."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Sequence[Norm]):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = list(norms)

    def forward(self, ctx, x, pending, stop):
        raise NotImplementedError


MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}


def _register(table: Dict[str, type], kind: str):
    def deco(cls):
        if kind in table and table[kind] is not cls:
            raise ValueError(f"part kind {kind!r} is already registered")
        table[kind] = cls
        cls.kind = kind
        return cls
    return deco


def register_mixer(kind): return _register(MIXERS, kind)
def register_feed_forward(kind): return _register(FEED_FORWARDS, kind)
def register_norm(kind): return _register(NORMS, kind)
def register_position_encoding(kind): return _register(POSITION_ENCODINGS, kind)
def register_block(kind): return _register(BLOCKS, kind)
def register_embedding(kind): return _register(EMBEDDINGS, kind)
def register_head(kind): return _register(HEADS, kind)


def build_part(table: Dict[str, type], spec, what: str, **extra):
    if spec.kind not in table:
        raise ValueError(f"unknown {what} kind {spec.kind!r}; known: {sorted(table)}")
    return table[spec.kind](**spec.params, **extra)
