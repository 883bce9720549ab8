"""The description of a model as data: which parts make each layer, with which sizes and
which checkpoint tensors, and in which order the layers run.

An architecture module turns its configuration into a ``ModelPlan``; everything after that
(loading, cache layout, the step function) reads only the plan, never the architecture.

Reference: the reference chooses a layer's mixer and feed-forward from the configuration,
layer by layer (``enum Mixer`` src/qwen.rs:39-43, ``enum Ffn`` src/qwen.rs:101-104,
selection src/qwen.rs:500-521) and lets a layer reuse another layer's keys and values
(src/model.rs:928-934).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional


@dataclasses.dataclass
class PartSpec:
    """One part: its registered ``kind``, its sizes and constants, and for each tensor it wants
    (by the part's own short name) the tensor's name in the checkpoint."""
    kind: str
    params: dict = dataclasses.field(default_factory=dict)
    tensors: Dict[str, str] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class LayerSpec:
    """A layer: a ``block`` kind and the parts it arranges, by the names that block kind reads.
    The ``prenorm`` block reads ``mixer_norm, mixer, ffn_norm, ffn``; another arrangement (a third
    norm, a pair of post-norms, a per-layer input) is another block kind with names of its own,
    and nothing else has to know them."""
    parts: Dict[str, PartSpec]
    block: str = "prenorm"

    @classmethod
    def prenorm(cls, mixer: PartSpec, ffn: PartSpec, mixer_norm: PartSpec, ffn_norm: PartSpec) -> "LayerSpec":
        """x += mixer(mixer_norm(x)); x += ffn(ffn_norm(x))."""
        return cls({"mixer_norm": mixer_norm, "mixer": mixer, "ffn_norm": ffn_norm, "ffn": ffn}, "prenorm")


@dataclasses.dataclass
class ScheduleEntry:
    """One run of a layer.  A layer may be named by several entries; each entry that keeps a
    cache has storage of its own.  ``cache_of`` is the position in the schedule of an earlier
    entry whose cache this run reads instead of writing one (None: its own)."""
    layer: int
    cache_of: Optional[int] = None


@dataclasses.dataclass
class ModelPlan:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    stop_ids: List[int] = dataclasses.field(default_factory=list)
    #: fnmatch patterns of checkpoint tensors the model does not use (not "unexpected")
    ignored_tensors: List[str] = dataclasses.field(default_factory=list)

    def validate(self):
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the plan has {n} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which keeps none of its own")
