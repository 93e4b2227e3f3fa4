"""Plain-data description of a model: which parts, with which sizes, in which order.

An architecture's recipe (``models/``) turns its typed config into a :class:`ModelSpec`; the decoder is built
from the spec alone, by looking each part's ``kind`` up in the part registries. Nothing here imports torch.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    kind: str
    """Key into the registry of this part's family (mixer, feed-forward, norm, position encoding, ...)."""
    params: Mapping[str, Any] = field(default_factory=dict)
    """Sizes and constants of the part; the part's constructor receives them as keyword arguments."""
    prefix: str = ""
    """Checkpoint-name prefix of the part's tensors, e.g. ``model.layers.3.self_attn.``."""

    def key(self) -> tuple:
        return (self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items())))


@dataclass(frozen=True)
class LayerSpec:
    """One block: a mixer and a feed-forward, each behind its norm, put together by ``arrangement``."""

    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec
    arrangement: str = "pre_norm"
    position: PartSpec | None = None
    """Position encoding handed to the mixer (shared between layers whose specs are equal)."""


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer. The schedule is data: it may run a layer twice (each run then has a cache of
    its own unless told otherwise) or let a run read the cache another run filled."""

    layer: int
    """Index into ``ModelSpec.layers``: whose parameters run."""
    cache_of: int | None = None
    """Schedule position whose cache this run reads instead of filling one of its own."""


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    """``params['tied']``: the head multiplies by the embedding table instead of a tensor of its own."""
    max_positions: int
    eos_token_ids: tuple[int, ...] = ()
    ignored_tensors: tuple[str, ...] = ()
    """Checkpoint names that may be present and are not used (regular expressions)."""
    name_prefixes: tuple[str, ...] = ("",)
    """Prefixes under which a checkpoint may store all names (the reference's files use ``llm.``,
    oxr_runtime/weight_names.py:11)."""
