"""The engine's core: a model, its cache and its step function on one GPU.

Generation, the command lines, the benchmark and the trace replay all drive this one object;
none of them has a forward pass, cache or loader of its own.  It plays the part of the
reference's ``EngineServer`` constructor (src/engine/engine_server.cpp:385-567): read the
configuration, load the weights, size the cache, allocate the scratch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable, Optional, Sequence

import torch

from ..cache import CacheManager
from ..models import Model, compute_dtype, load_model
from .batch import StepEntry
from .runner import ModelRunner


@dataclass
class EngineOptions:
    """Options of the engine, after the reference's constructor arguments
    (include/lightllm/engine/engine.h:286-293: ``max_seq_len``, ``max_batch_tokens``,
    ``kv_cache_mb``); ``dtype``, ``page_size``, ``num_pages`` and ``max_seqs`` are this engine's.

    ``max_seq_len`` <= 0 means the model's ``max_position_embeddings`` (engine_server.cpp:412-415).
    The pool has ``num_pages`` pages per cache group if given, else as many as ``kv_cache_mb``
    megabytes hold, else enough for ``max_seqs`` requests of ``max_seq_len`` tokens or what fits in 85 % of
    the device memory that is free after the weights are loaded, whichever is less."""

    dtype: str = "bfloat16"
    max_seq_len: int = 0
    max_batch_tokens: int = 256
    page_size: int = 16
    num_pages: Optional[int] = None
    kv_cache_mb: Optional[float] = None
    max_seqs: int = 64
    device: str = "cuda:0"
    use_cuda_graphs: bool = True


class EngineCore:
    def __init__(self, model_dir: str, options: Optional[EngineOptions] = None, model: Optional[Model] = None):
        self.options = opt = options or EngineOptions()
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; the engine has no CPU path")
        self.device = torch.device(opt.device)
        torch.cuda.set_device(self.device)
        self.dtype = compute_dtype(opt.dtype)
        self.model = model if model is not None else load_model(model_dir, self.dtype, self.device)
        spec = self.model.spec
        self.max_seq_len = opt.max_seq_len if opt.max_seq_len > 0 else spec.max_positions
        self.max_seq_len = min(self.max_seq_len, spec.max_positions)
        layout = self.model.cache_layout
        esize = 4 if self.dtype == torch.float32 else 2
        pages_per_seq = -(-self.max_seq_len // opt.page_size)
        if opt.num_pages is not None:
            num_pages = [opt.num_pages] * len(layout.groups)
        elif opt.kv_cache_mb is not None:
            per_page = sum(layout.bytes_per_page(g, opt.page_size, esize) for g in range(len(layout.groups)))
            n = int(opt.kv_cache_mb * 1024 * 1024 // max(1, per_page))
            num_pages = [max(1, n)] * len(layout.groups)
        else:
            # Room for max_seqs requests of max_seq_len tokens, but no more than most of the memory that is free
            # now that the weights are loaded (a model with 131,072 positions would ask for more than the device has).
            per_page = sum(layout.bytes_per_page(g, opt.page_size, esize) for g in range(len(layout.groups)))
            want = pages_per_seq * opt.max_seqs
            free_bytes = torch.cuda.mem_get_info(self.device)[0]
            fit = int(free_bytes * 0.85 // max(1, per_page))
            if fit < pages_per_seq:
                raise RuntimeError(
                    f"the cache of one request of {self.max_seq_len} tokens needs {pages_per_seq * per_page} bytes, but "
                    f"only {free_bytes} bytes of device memory are free: give max_seq_len, num_pages or kv_cache_mb")
            num_pages = [min(want, fit)] * len(layout.groups)
        self.cache = CacheManager(layout, opt.page_size, num_pages, opt.max_seqs, self.max_seq_len,
                                  self.dtype, self.device)
        self.runner = ModelRunner(self.model, self.cache, opt.max_batch_tokens, opt.max_seqs, opt.use_cuda_graphs)

    # The requests' lifetime, as the reference's create_request_state / release_request
    # (src/engine/engine_server.cpp:625-688, 694-717).
    def open(self, seq_id: Hashable) -> None:
        self.cache.open(seq_id)

    def close(self, seq_id: Hashable) -> None:
        self.cache.close(seq_id)

    def is_open(self, seq_id: Hashable) -> bool:
        return seq_id in self.cache.seqs

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None,
             token_map=None) -> Optional[torch.Tensor]:
        return self.runner.step(entries, device_tokens, token_map)

    def launch_count(self) -> int:
        """Kernels of the engine's own library launched so far in this process."""
        from ..csrc import ops
        return ops.launch_count() + self.runner.graph_launches

    @property
    def vocab_size(self) -> int:
        return self.model.spec.vocab_size

    @property
    def eos_token_ids(self) -> tuple:
        """The end-of-sequence ids that the model's config.json names (empty if it names none)."""
        config = getattr(self.model, "config", None)
        return tuple(config.eos_token_ids) if config is not None else ()
