"""What a mixer asks of the cache: pages of keys and values, a fixed-size state, both or nothing.

The reference gives every layer the same geometry and allocates them in lockstep
(src/engine/engine_server.cpp:530-533, 1426-1438).  Here a mixer declares its needs and the
layout groups cache planes whose needs are equal, so that layers that keep every key and layers
that keep a window of them have pages of their own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class KVSpec:
    """Keys and values per token: ``kv_heads * head_dim`` each.  ``window`` = how many of the
    latest positions (the token itself included) stay visible; ``None`` = all of them."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, one ``shape`` tensor of ``dtype`` per request."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class CacheSpec:
    kv: Optional[KVSpec] = None
    state: Optional[StateSpec] = None


@dataclass
class PlaneRef:
    """Where one run entry's cache lives: group and plane for pages, index for state."""

    group: Optional[int] = None
    plane: Optional[int] = None
    state_plane: Optional[int] = None
    owns: bool = True          # False: the entry reads another entry's plane and writes nothing


@dataclass
class CacheLayout:
    """Groups of planes with equal needs, built from the cache specs of the run list."""

    groups: List[KVSpec] = field(default_factory=list)
    planes_per_group: List[int] = field(default_factory=list)
    state_planes: List[StateSpec] = field(default_factory=list)
    refs: List[PlaneRef] = field(default_factory=list)     # one per run entry

    @staticmethod
    def build(specs: Sequence[Optional[CacheSpec]], cache_of: Sequence[Optional[int]]) -> "CacheLayout":
        """``specs[i]`` is the cache spec of run entry i; ``cache_of[i]`` names the earlier entry
        whose plane entry i reads instead of owning one."""
        layout = CacheLayout()
        index: Dict[KVSpec, int] = {}
        for i, (spec, src) in enumerate(zip(specs, cache_of)):
            ref = PlaneRef()
            if src is not None:
                owner = layout.refs[src]
                want = spec.kv if spec else None
                have = layout.groups[owner.group] if owner.group is not None else None
                if want is not None and (have is None or (want.kv_heads, want.head_dim) != (have.kv_heads, have.head_dim)):
                    raise ValueError(
                        f"run entry {i} reads the cache of entry {src}, whose geometry {have} does not fit {want}")
                if want is not None and have.window is not None and (want.window is None or want.window > have.window):
                    raise ValueError(
                        f"run entry {i} needs a window of {want.window} but entry {src} keeps only {have.window} keys")
                ref = PlaneRef(owner.group, owner.plane, owner.state_plane, owns=False)
            elif spec is not None:
                if spec.kv is not None:
                    g = index.get(spec.kv)
                    if g is None:
                        g = len(layout.groups)
                        index[spec.kv] = g
                        layout.groups.append(spec.kv)
                        layout.planes_per_group.append(0)
                    ref.group, ref.plane = g, layout.planes_per_group[g]
                    layout.planes_per_group[g] += 1
                if spec.state is not None:
                    ref.state_plane = len(layout.state_planes)
                    layout.state_planes.append(spec.state)
            layout.refs.append(ref)
        return layout

    def bytes_per_page(self, group: int, page_size: int, element_bytes: int) -> int:
        s = self.groups[group]
        return 2 * self.planes_per_group[group] * page_size * s.kv_heads * s.head_dim * element_bytes

    def bytes_per_token(self, element_bytes: int) -> int:
        return sum(2 * n * s.kv_heads * s.head_dim * element_bytes
                   for s, n in zip(self.groups, self.planes_per_group))
