"""A model as the engine runs it: parts built from a :class:`ModelSpec`, weights bound by name."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache import CacheLayout
from ..config import ModelConfig, ModelSpec, load_config, model_spec_for
from ..parts import Block, Part, build_part
from ..weights import WeightSpec, dedup_specs, load_checkpoint_tensors


def _walk(part: Part):
    yield part
    for c in part.children():
        yield from _walk(c)


class Model:
    """Embedding, the layers, the run list over them, final norm and head.

    The run list is data (``spec.run``): it may name a layer twice (the weights are shared, each
    run has its own cache plane) or let a run read an earlier run's cache."""

    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.layers: List[Block] = [Block(ls) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.run = list(spec.run)
        mixers = [self.layers[e.layer].mixer for e in self.run]
        self.cache_layout = CacheLayout.build(
            [m.cache_spec() if m is not None else None for m in mixers], [e.cache_of for e in self.run])
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        self._prepare_hooks = None

    def parts(self) -> List[Part]:
        out: List[Part] = []
        for top in [self.embedding, *self.layers, self.final_norm, self.head]:
            out.extend(_walk(top))
        return out

    def weight_specs(self) -> List[WeightSpec]:
        specs: List[WeightSpec] = []
        for p in self.parts():
            if not isinstance(p, Block):
                specs.extend(p.weight_specs())
        return dedup_specs(specs)

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        self.dtype, self.device = dtype, device
        for p in self.parts():
            if not isinstance(p, Block):
                p.bind(tensors, dtype, device)

    def prepare(self, ctx, views) -> None:
        """Every part's ``prepare`` for this step, run entry by run entry (before the metadata copy)."""
        hooks = self._prepare_hooks
        if hooks is None:
            # the parts that have something to prepare (most do not override the hook), found once
            from ..parts.base import Part
            def own(part):
                hook = getattr(part, "prepare", None)
                return hook if hook is not None and getattr(type(part), "prepare", None) is not Part.prepare else None
            hooks, keys = [], set()

            def add(part, run_index):
                key = getattr(part, "prepare_key", None)
                if own(part) and (key is None or key not in keys):
                    hooks.append((own(part), run_index))
                    if key is not None:
                        keys.add(key)         # parts with equal keys prepare the same things: once is enough
            for i, entry in enumerate(self.run):
                for sb in self.layers[entry.layer].subs:
                    for part in sb.parts():
                        add(part, i if part is sb.part and sb.role == "mixer" else None)
            for part in (self.embedding, self.final_norm, self.head):
                add(part, None)
            self._prepare_hooks = hooks
        for hook, run_index in hooks:
            if run_index is None:
                hook(ctx)
            else:
                hook(ctx, views[run_index])

    def graph_blockers(self) -> List[str]:
        """The parts that keep this model's steps out of CUDA graphs: those that do not declare that their
        forward only launches kernels whose arguments are fixed by the step's counts."""
        return sorted({type(p).__name__ for p in self.parts()
                       if not isinstance(p, Block) and not getattr(p, "graph_safe", False)})

    def graph_safe(self) -> bool:
        """Whether a step of this model can be captured in a CUDA graph (no part blocks it)."""
        return not self.graph_blockers()

    def weight_bytes(self) -> int:
        """Bytes of the tensors a step reads (a tied table counts once)."""
        seen, total = set(), 0
        for p in self.parts():
            for v in vars(p).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total


def weight_specs_of(spec: ModelSpec) -> List[WeightSpec]:
    return Model(spec).weight_specs()


_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, torch.float32: torch.float32,
           torch.bfloat16: torch.bfloat16}


def compute_dtype(name) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be 'float32' or 'bfloat16', got {name!r}") from None


def random_model_on_device(config, seed: int, dtype, device: torch.device) -> Model:
    """A model of ``config`` (a config.json dictionary or its typed form) with random weights drawn on the device:
    for measurements at sizes whose weights would take minutes to write and read as a folder.  The distributions are
    those of the random-weights mode (each part's weight list says them); the values are not the folder's."""
    import hashlib
    from ..config import config_from_dict
    if isinstance(config, dict):
        config = config_from_dict(config, "random-weights configuration")
    model = Model(model_spec_for(config))
    model.config = config
    dt = compute_dtype(dtype)
    tensors: Dict[str, torch.Tensor] = {}
    for s in model.weight_specs():
        g = torch.Generator(device=device)
        g.manual_seed(int.from_bytes(hashlib.sha256(f"{seed}:{s.name}".encode()).digest()[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF)
        kind, shape = s.init[0], tuple(s.shape)
        if kind in ("normal", "one_plus_normal"):
            t = torch.randn(shape, generator=g, dtype=torch.float32, device=device) * float(s.init[1])
            if kind == "one_plus_normal":
                t += 1.0
        elif kind in ("zeros", "ones"):
            t = torch.full(shape, 0.0 if kind == "zeros" else 1.0, dtype=torch.float32, device=device)
        elif kind == "randint":
            t = torch.randint(int(s.init[1]), int(s.init[2]), shape, generator=g, dtype=torch.int32, device=device)
        else:
            raise ValueError(f"unknown init rule {s.init!r} for tensor {s.name!r}")
        tensors[s.name] = t if s.kind == "int" else t.to(dt)
    model.bind(tensors, dt, device)
    return model


def load_model(model_dir: str, dtype, device: torch.device) -> Model:
    """Build the model that ``model_dir/config.json`` names and bind ``model.safetensors`` to it."""
    config = load_config(model_dir)
    model = Model(model_spec_for(config))
    model.config = config
    dt = compute_dtype(dtype)
    tensors = load_checkpoint_tensors(model_dir, model.weight_specs(), dt, device, tuple(model.spec.ignored_suffixes))
    model.bind(tensors, dt, device)
    return model
