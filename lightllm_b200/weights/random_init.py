"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode (it needs a downloaded checkpoint, README.md:54-62).
Each tensor is drawn from its own generator, seeded by a hash of (seed, tensor name),
so a tensor's values do not depend on which other tensors the model has.  Values are
drawn in float32 and rounded once when stored in 16 bits.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Iterable, Optional, Union

import torch

from ..config import ModelConfig, config_from_dict, model_spec_for
from .loader import WeightSpec, dedup_specs
from .safetensors_io import save_file

_STORE_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF)
    return g


def draw_tensor(spec: WeightSpec, seed: int) -> torch.Tensor:
    """One tensor drawn by its spec's ``init`` rule, in float32 (int32 for tables)."""
    g = _generator(seed, spec.name)
    kind = spec.init[0]
    shape = tuple(spec.shape)
    if kind == "normal":
        return torch.randn(shape, generator=g, dtype=torch.float32) * float(spec.init[1])
    if kind == "one_plus_normal":
        return 1.0 + torch.randn(shape, generator=g, dtype=torch.float32) * float(spec.init[1])
    if kind == "zeros":
        return torch.zeros(shape, dtype=torch.float32)
    if kind == "ones":
        return torch.ones(shape, dtype=torch.float32)
    if kind == "randint":
        return torch.randint(int(spec.init[1]), int(spec.init[2]), shape, generator=g, dtype=torch.int32)
    raise ValueError(f"unknown init rule {spec.init!r} for tensor {spec.name!r}")


def random_tensors(specs: Iterable[WeightSpec], seed: int, store_dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for s in dedup_specs(specs):
        t = draw_tensor(s, seed)
        out[s.name] = t if s.kind == "int" else t.to(store_dtype)
    return out


def write_random_model(config: Union[ModelConfig, Dict[str, Any]], seed: int, out_dir: str,
                       store_dtype: str = "bfloat16") -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` for ``config``.

    ``config`` is the architecture's own config.json content (a dictionary) or its typed
    form.  Linear and embedding weights are N(0, 0.02), biases N(0, 0.02) and norm weights
    1 + N(0, 0.01), as each part's weight list says."""
    from ..models.model import weight_specs_of  # late: parts register on import

    if store_dtype not in _STORE_DTYPES:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE_DTYPES)}, got {store_dtype!r}")
    if isinstance(config, dict):
        config = config_from_dict(config, "random-weights configuration")
    spec = model_spec_for(config)
    tensors = random_tensors(weight_specs_of(spec), seed, _STORE_DTYPES[store_dtype])
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_json_dict(), f, indent=1, sort_keys=True)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return out_dir
