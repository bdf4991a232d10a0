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
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """One part of a layer: its kind (a name in the part registry) and every size and
    constant it needs.  ``prefix`` is where its tensors live in the checkpoint."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass
class SubBlock:
    """One branch of a layer around the residual stream ``h``:

        x = norm_before(h)            (without ``norm_before``: h itself, in the compute dtype)
        y = part(x)
        h = h + y                     without ``norm_after``
        h = h + norm_after(y)         ``after="branch"``: a norm on the branch's output (sandwich norms)
        h = norm_after(h + y)         ``after="stream"``: a norm on the stream itself (post-norm)

    ``role`` is the part's role in the registry: ``mixer`` (it may own cache) or ``ffn``."""

    role: str
    part: PartSpec
    norm_before: Optional[PartSpec] = None
    norm_after: Optional[PartSpec] = None
    after: str = "branch"


ARRANGEMENTS = ("sequential", "parallel")
_OLD_NAMES = {"pre_norm": "sequential"}


@dataclass
class LayerSpec:
    """A layer: an ordered list of sub-blocks and how they read the residual stream.

    ``arrangement``:
      ``sequential``  each sub-block reads the stream the one before it left    (Qwen2: norm, attention, add;
                      norm, feed-forward, add: engine_server.cpp:1530-1880)
      ``parallel``    all sub-blocks read the same stream, then every branch is added

    A layer may hold any number of sub-blocks, at most one of them a mixer (a run of the layer has one
    cache plane), so a layer without a feed-forward, with four norms or with post-norms is data.  The
    common case keeps its short form: ``LayerSpec(norm1, mixer, norm2, ffn)`` is the two sub-blocks
    ``(norm1, mixer)`` and ``(norm2, ffn)``; ``arrangement="pre_norm"`` is another word for ``sequential``."""

    norm1: Optional[PartSpec] = None
    mixer: Optional[PartSpec] = None
    norm2: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None
    arrangement: str = "sequential"
    sub_blocks: List[SubBlock] = field(default_factory=list)

    def __post_init__(self):
        self.arrangement = _OLD_NAMES.get(self.arrangement, self.arrangement)
        if self.arrangement not in ARRANGEMENTS:
            raise ValueError(f"unknown arrangement {self.arrangement!r}; known: {ARRANGEMENTS}")
        short = [self.norm1, self.mixer, self.norm2, self.ffn]
        if self.sub_blocks:
            if any(x is not None for x in short):
                raise ValueError("a layer is given either as sub_blocks or as norm1/mixer/norm2/ffn, not both")
        else:
            if self.mixer is not None:
                self.sub_blocks.append(SubBlock("mixer", self.mixer, self.norm1))
            if self.ffn is not None:
                self.sub_blocks.append(SubBlock("ffn", self.ffn, self.norm2))
            self.norm1 = self.mixer = self.norm2 = self.ffn = None
        if not self.sub_blocks:
            raise ValueError("a layer needs at least one sub-block")
        for sb in self.sub_blocks:
            if sb.role not in ("mixer", "ffn"):
                raise ValueError(f"a sub-block's role is 'mixer' or 'ffn', not {sb.role!r}")
            if sb.after not in ("branch", "stream"):
                raise ValueError(f"a sub-block's norm_after applies to the 'branch' or the 'stream', not {sb.after!r}")
            if sb.after == "stream" and sb.norm_after is not None and self.arrangement == "parallel":
                raise ValueError("a norm on the stream has no meaning between parallel branches")
        if sum(sb.role == "mixer" for sb in self.sub_blocks) > 1:
            raise ValueError("a layer holds at most one mixer: a run of the layer has one cache plane")


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
    # Endings of tensor names that a checkpoint of this architecture may carry without the model reading them.
    ignored_suffixes: Tuple[str, ...] = ()

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
