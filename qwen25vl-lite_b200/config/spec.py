"""The description of a model as data: which parts each layer is made of, with their sizes
and constants, and the order in which layers run.

An architecture's *spec builder* turns its typed configuration into a :class:`ModelSpec`;
the generic model assembly (``models/decoder.py``) and the cache manager read nothing else.
Parts are named by ``kind`` strings that the part registries resolve, so one model may use
different mixers and feed-forwards in different layers, and a test can describe a model out
of toy parts without touching this package.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` picks the class from its registry, ``params`` are the constructor
    arguments (every size and constant the part needs), ``prefix`` is prepended to the
    part's tensor names to form checkpoint names."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer = an arrangement (``block``) of a mixer, a feed-forward and its norms."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Tuple[PartSpec, ...]
    prefix: str = ""
    # the position encoding this layer's mixer applies; None: the model's (``ModelSpec.position``)
    position: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One stop of the forward pass.  ``layer`` indexes ``ModelSpec.layers`` and may repeat
    (the weights are then shared, each stop keeps a cache of its own).  ``cache_of`` names an
    earlier stop whose keys and values this stop reads instead of keeping its own."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    # defines the tokens' positions (how many axes, where plain text sits) and is what every layer
    # applies that names no encoding of its own
    position: PartSpec
    # checkpoint naming: prefixes that may precede every decoder tensor name, tried in this
    # order, and prefixes of tensors that belong to parts this engine does not build.
    name_prefixes: Tuple[str, ...] = ("",)
    ignored_prefixes: Tuple[str, ...] = ()
    # names that are never prefixed (e.g. the output head of the whole checkpoint)
    unprefixed_names: Tuple[str, ...] = ()

    def validate(self) -> None:
        for i, stop in enumerate(self.schedule):
            if not 0 <= stop.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {stop.layer}, model has {len(self.layers)}")
            if stop.cache_of is not None:
                if not 0 <= stop.cache_of < i:
                    raise ValueError(f"schedule[{i}].cache_of must name an earlier stop, got {stop.cache_of}")
                if self.schedule[stop.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}].cache_of names stop {stop.cache_of}, which keeps no cache itself")
