"""Assembly of a decoder from a ``ModelSpec``: embedding, the scheduled stops (each a block
of parts), final norm, output head.  Nothing here is specific to one architecture.

The forward pass mirrors the reference's order (src/qwen25vl_lite/text.py:243-279 and
src/qwen25vl_lite/model.py:200-202): embed, run the layers, normalise, keep the wanted
positions, project to the vocabulary -- except that only the wanted rows are normalised.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..cache.manager import StopNeeds
from ..config.spec import ModelSpec
from ..parts import base as parts


@dataclass
class StopRuntime:
    """One schedule stop at run time."""

    index: int
    layer: int
    cache_of: Optional[int]
    owns_cache: bool
    state: Optional[torch.Tensor] = None     # [max_requests, *shape], set by the runner


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        # the encoding that defines the tokens' positions; a layer that names another one gets that
        # (equal descriptions are built once)
        self._positions: Dict[str, parts.PositionEncoding] = {}
        self.position = self._position_for(spec.position)
        self.embedding = parts.build_part(parts.EMBEDDINGS, spec.embedding, "embedding")
        self.blocks: List[parts.Block] = []
        self._named_parts: List[Tuple[str, parts.Part]] = [(spec.embedding.prefix, self.embedding)]
        for layer in spec.layers:
            if layer.block not in parts.BLOCKS:
                raise ValueError(f"unknown block kind {layer.block!r}; known: {sorted(parts.BLOCKS)}")
            mixer = parts.build_part(parts.MIXERS, layer.mixer, "mixer",
                                     position=self._position_for(layer.position or spec.position))
            ffn = parts.build_part(parts.FEED_FORWARDS, layer.feed_forward, "feed-forward")
            norms = [parts.build_part(parts.NORMS, n, "norm") for n in layer.norms]
            self.blocks.append(parts.BLOCKS[layer.block](mixer, ffn, norms))
            self._named_parts.append((layer.prefix + layer.mixer.prefix, mixer))
            self._named_parts.append((layer.prefix + layer.feed_forward.prefix, ffn))
            for nspec, n in zip(layer.norms, norms):
                self._named_parts.append((layer.prefix + nspec.prefix, n))
        self.final_norm = parts.build_part(parts.NORMS, spec.final_norm, "norm")
        self.head = parts.build_part(parts.HEADS, spec.head, "output head")
        self._named_parts.append((spec.final_norm.prefix, self.final_norm))
        self._named_parts.append((spec.head.prefix, self.head))
        self.stops = [StopRuntime(i, s.layer, s.cache_of, s.cache_of is None) for i, s in enumerate(spec.schedule)]
        self.dtype: Optional[torch.dtype] = None
        self.device = None

    def _position_for(self, pspec) -> parts.PositionEncoding:
        key = repr((pspec.kind, sorted(pspec.params.items(), key=lambda kv: kv[0])))
        if key not in self._positions:
            part = parts.build_part(parts.POSITION_ENCODINGS, pspec, "position encoding")
            if part.axes > getattr(self, "position", part).axes:
                raise ValueError(f"a layer's position encoding reads {part.axes} axes, the model's positions have "
                                 f"{self.position.axes}")
            self._positions[key] = part
        return self._positions[key]

    def position_encodings(self) -> List[parts.PositionEncoding]:
        return list(self._positions.values())

    def planning_parts(self) -> List[parts.Part]:
        """The parts whose kernels read work lists that the step function packs (``plan_step``)."""
        return [part for _, part in self._named_parts if part.plan_key() is not None]

    # ---- weights -----------------------------------------------------------------------
    def expected_tensors(self) -> Dict[str, parts.TensorSpec]:
        """Canonical (un-prefixed) checkpoint name -> what is expected under it."""
        out: Dict[str, parts.TensorSpec] = {}
        for prefix, part in self._named_parts:
            for ts in part.tensor_specs():
                out[prefix + ts.name] = ts
        return out

    def load(self, get_tensor: Callable[[str], torch.Tensor], available, device, dtype: torch.dtype) -> None:
        """``get_tensor(canonical name)`` returns a CPU tensor; ``available`` is the set of
        canonical names the checkpoint has."""
        self.device, self.dtype = torch.device(device), dtype
        for position in self._positions.values():
            position.load({}, device, dtype)
        # A part may offer tensors it holds on the device to the parts loaded after it
        # (``exports``, by canonical name) and take such tensors instead of loading its own
        # (``imports``): how a tied output head comes to read the embedding table.
        shared: Dict[str, torch.Tensor] = {}
        for prefix, part in self._named_parts:
            tensors = {ts.name: get_tensor(prefix + ts.name) for ts in part.tensor_specs()
                       if (prefix + ts.name) in available}
            wanted = {name: shared[name] for name in part.imports() if name in shared}
            if wanted:
                part.receive(wanted)
            part.load(tensors, device, dtype)
            shared.update({prefix + name: t for name, t in part.exports().items()})

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for _, part in self._named_parts:
            for v in vars(part).values():
                for t in (v.weight, v.bias) if hasattr(v, "weight") and hasattr(v, "bias") else (v,):
                    if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                        seen.add(t.data_ptr())
                        total += t.numel() * t.element_size()
        return total

    # ---- cache needs -------------------------------------------------------------------
    def stop_needs(self) -> List[StopNeeds]:
        out = []
        for s in self.stops:
            mixer = self.blocks[s.layer].mixer
            out.append(StopNeeds(mixer.cache_need(), mixer.state_need(), s.cache_of))
        return out

    # ---- forward -----------------------------------------------------------------------
    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs the step described by ``ctx`` and returns float32 logits [wanted, vocab]
        (None when nothing is wanted)."""
        if hasattr(ctx, "shared"):
            ctx.shared.clear()
        x = self.embedding.forward(ctx)
        pending = None
        for stop in self.stops:
            pending = self.blocks[stop.layer].forward(ctx, x, pending, stop)
        if ctx.logit_rows is None or ctx.logit_rows.shape[0] == 0:
            return None
        # a step of single tokens that all want their logits needs no gather, and a head that can
        # normalise inside its product then gets the norm handed on instead of its result
        rows = None if getattr(ctx, "logits_every_row", False) else ctx.logit_rows
        h = self.final_norm.forward(ctx, x, pending, rows=rows,
                                    defer=rows is None and self.head.accepts_deferred_norm)
        return self.head.forward(ctx, h)
