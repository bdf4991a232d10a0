"""Binding checkpoint tensors to a model's parts by tensor name.

The reference loads a fixed list of names (src/engine/engine_server.cpp:436-450) and
checks shapes only in its tests (tests/test_model.cpp:59-76); its loader's errors come
one at a time (src/model/model_loader.cpp:131,143,147).  Here every part declares the
tensors it reads (:class:`WeightSpec`), the whole list is compared with the file, and a
single :class:`WeightError` lists every missing tensor, unexpected tensor and wrong
shape at once.

Precision policy: with ``dtype=float32`` every floating tensor becomes float32.  With
``dtype=bfloat16`` tensors stored in 16 bits become bfloat16, a tensor stored in 32 bits
stays float32, and integer tables become int32.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import Checkpoint, TensorInfo


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every fault."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_type: Sequence[Tuple[str, str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_type = list(wrong_type)
        lines = [f"{where}: checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += [f"    {n}" for n in self.missing]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += [f"    {n}" for n in self.unexpected]
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += [f"    {n}: file has {list(got)}, model expects {list(want)}"
                      for n, got, want in self.wrong_shape]
        if self.wrong_type:
            lines.append(f"  wrong types ({len(self.wrong_type)}):")
            lines += [f"    {n}: file has {got}, model expects {want}" for n, got, want in self.wrong_type]
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class WeightSpec:
    """One tensor that a part reads.

    ``init`` tells the random-weights mode how to draw it:
    ``("normal", std)``, ``("one_plus_normal", std)``, ``("zeros",)``, ``("ones",)`` or
    ``("randint", low, high)`` for integer tables."""

    name: str
    shape: Tuple[int, ...]
    kind: str = "float"            # "float" or "int"
    init: Tuple = ("normal", 0.02)
    optional: bool = False


def target_dtype(info_dtype: str, kind: str, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device (see the module's precision policy)."""
    if kind == "int":
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if info_dtype in ("F32", "F64"):
        return torch.float32
    return torch.bfloat16


def check_against(specs: Sequence[WeightSpec], available: Dict[str, TensorInfo], where: str,
                  ignore: Iterable[str] = ()) -> None:
    """Raise one :class:`WeightError` if the file's tensors do not fit ``specs``."""
    ignore = tuple(ignore)
    wanted = {s.name: s for s in specs}
    missing = [s.name for s in specs if not s.optional and s.name not in available]
    unexpected = [n for n in available
                  if n not in wanted and not any(n.endswith(sfx) for sfx in ignore)]
    wrong_shape = []
    wrong_type = []
    for name, s in wanted.items():
        info = available.get(name)
        if info is None:
            continue
        if tuple(info.shape) != tuple(s.shape):
            wrong_shape.append((name, tuple(info.shape), tuple(s.shape)))
        if s.kind == "float" and not info.is_float:
            wrong_type.append((name, info.dtype, "a floating type"))
        if s.kind == "int" and info.is_float:
            wrong_type.append((name, info.dtype, "an integer type"))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(where, sorted(missing), sorted(unexpected), wrong_shape, wrong_type)


def dedup_specs(specs: Iterable[WeightSpec]) -> List[WeightSpec]:
    """Specs by name, first one wins; a name declared twice with two shapes is a fault of
    the model description."""
    out: Dict[str, WeightSpec] = {}
    for s in specs:
        if s.name in out:
            if tuple(out[s.name].shape) != tuple(s.shape):
                raise ValueError(f"tensor {s.name!r} is declared with shapes {out[s.name].shape} and {s.shape}")
            continue
        out[s.name] = s
    return list(out.values())


def load_checkpoint_tensors(model_dir: str, specs: Sequence[WeightSpec], compute_dtype: torch.dtype,
                            device: torch.device, ignore: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Read every tensor that ``specs`` names, convert it by the precision policy and put it
    on ``device``.  Fails with one :class:`WeightError` before anything is copied."""
    ckpt = Checkpoint(model_dir)
    try:
        specs = dedup_specs(specs)
        check_against(specs, ckpt.tensors, model_dir, ignore)
        out: Dict[str, torch.Tensor] = {}
        for s in specs:
            info = ckpt.tensors.get(s.name)
            if info is None:
                continue
            t = ckpt.read(s.name)
            dt = target_dtype(info.dtype, s.kind, compute_dtype)
            out[s.name] = t.to(dt).to(device).contiguous()
        return out
    finally:
        ckpt.close()
