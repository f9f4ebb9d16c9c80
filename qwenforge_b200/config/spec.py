"""Architecture-neutral description of a model: which parts each layer is made of,
with which sizes, which tensors of the weight files they own, and in which order
the layers run.

A configuration class (one per architecture, see `registry.py`) turns the keys of
its own config.json into a `ModelSpec`. Everything below the configuration (weight
loading, random weights, the cache, the model runtime) reads only the spec, so none
of it knows the architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer.

    kind     name under which the part's class is registered (`parts.registry`)
    params   the part's sizes and constants (everything it needs besides weights)
    tensors  the part's own logical tensor names -> tensor names in the weight files
    """
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    tensors: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (`block`, the name of a registered block kind) over named part specs.

    Which names there are, and which role each plays, is the block kind's business: `pre_norm` reads
    `mixer_norm`, `mixer`, `feed_forward_norm` and `feed_forward`; an arrangement with post-norms, a parallel
    residual or no feed-forward is another block kind with names of its own, and nothing else changes.
    """
    block: str
    parts: Mapping[str, PartSpec] = field(default_factory=dict)

    def part(self, name: str) -> PartSpec:
        try:
            return self.parts[name]
        except KeyError:
            raise KeyError(f"layer spec of block {self.block!r} names no part {name!r}; it has "
                           f"{', '.join(sorted(self.parts)) or 'none'}") from None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    layer       index into `ModelSpec.layers`; a layer may be named by several entries
                (its weights are then shared, each entry has a cache of its own)
    cache_from  index of an earlier schedule entry whose cache this run reads instead
                of writing one of its own; None means its own cache
    """
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: tuple = ()
    # tensor names that files may hold although no part asks for them, each with the wanted tensor it must
    # equal (a stored copy of a shared table); a copy that differs is an error
    redundant_tensors: Mapping[str, str] = field(default_factory=dict)

    def validate(self) -> None:
        if not self.schedule:
            raise ValueError("model spec: the schedule is empty")
        for pos, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"model spec: schedule entry {pos} names layer {entry.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < pos:
                    raise ValueError(f"model spec: schedule entry {pos} reads the cache of entry "
                                     f"{entry.cache_from}, which does not run before it")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(f"model spec: schedule entry {pos} reads the cache of entry "
                                     f"{entry.cache_from}, which has no cache of its own")
