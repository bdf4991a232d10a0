"""Architecture-independent description of a model as data.

An architecture's builder turns its typed configuration into a :class:`ModelSpec`:
which parts make each layer, which weights they read, and the order in which the
layers run.  The engine builds the model from this description alone; no part is
told which architecture it belongs to.

The reference writes its one transformer inline in ``EngineServer::step``
(src/engine/engine_server.cpp:1526-1881) with no layer classes; this description is
what replaces that so that a layer with another mixer or feed-forward is a new entry
in a list, not new plumbing.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class PartSpec:
    """One part of a layer: its kind (a name in the part registry) and every size and
    constant it needs.  ``prefix`` is where its tensors live in the checkpoint."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass
class LayerSpec:
    """A block: two norms, a mixer and a feed-forward, and how they are arranged.

    ``arrangement``:
      ``pre_norm``  h += mixer(norm1(h)); h += ffn(norm2(h))      (Qwen2, engine_server.cpp:1530-1880)
      ``parallel``  h += mixer(norm1(h)) + ffn(norm2(h)) with both read from the same h
    """

    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec
    arrangement: str = "pre_norm"


@dataclass
class RunEntry:
    """One entry of the run list: which layer runs, and whose cache it reads.

    ``cache_of`` is ``None`` when this run owns a cache plane (it writes its own keys
    and values or state), or the index of an earlier run entry whose plane it reads
    without writing."""

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    run: List[RunEntry]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        n = len(self.layers)
        for i, e in enumerate(self.run):
            if not 0 <= e.layer < n:
                raise ValueError(f"run[{i}] names layer {e.layer}, but the model has {n} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"run[{i}].cache_of={e.cache_of} must name an earlier run entry")
                if self.run[e.cache_of].cache_of is not None:
                    raise ValueError(f"run[{i}].cache_of={e.cache_of} names an entry that owns no cache")
