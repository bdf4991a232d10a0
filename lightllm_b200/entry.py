"""The Python entry point: ``Engine(model_dir).generate(prompts)``.

The reference has no Python; its users drive ``EngineServer`` and ``BatchMainLoop`` from C++
(tools/bench_server.cpp:33-245).  This class gives the same two things under the same option
names: the engine's constructor arguments (include/lightllm/engine/engine.h:286-293) and the
loop's ``submit`` arguments (include/lightllm/engine/batch_loop.h:103-108).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from .engine import EngineCore, EngineOptions, StepEntry
from .engine.loop import BatchMainLoop
from .sampling import SamplingParams


class Engine:
    """A model on one GPU, ready to generate.

    ``model_dir`` holds ``config.json`` and ``model.safetensors``; the architecture is chosen by
    ``config.json``.  ``dtype`` is ``"bfloat16"`` (serving) or ``"float32"`` (true 32-bit
    everywhere).  ``model``: a model that is already bound on the device (then ``model_dir`` is not read).
    ``max_seq_len`` <= 0 means the model's own limit.  ``decode_ahead`` lets the serve loop
    launch a decode step before the ids of the step before it have reached the host."""

    def __init__(self, model_dir: str, dtype: str = "bfloat16", max_seq_len: int = 0, max_batch_tokens: int = 256,
                 kv_cache_mb: Optional[float] = None, page_size: int = 16, num_pages: Optional[int] = None,
                 max_seqs: int = 64, chunk_size: int = 16, max_prefill_entries: int = 999, device: str = "cuda:0",
                 decode_ahead: bool = True, model=None):
        self.core = EngineCore(model_dir, EngineOptions(
            dtype=dtype, max_seq_len=max_seq_len, max_batch_tokens=max_batch_tokens, page_size=page_size,
            num_pages=num_pages, kv_cache_mb=kv_cache_mb, max_seqs=max_seqs, device=device), model=model)
        self.chunk_size = chunk_size
        self.max_batch_tokens = max_batch_tokens
        self.max_prefill_entries = max_prefill_entries
        self.decode_ahead = decode_ahead

    @property
    def vocab_size(self) -> int:
        return self.core.vocab_size

    def new_loop(self) -> BatchMainLoop:
        """A serve loop over this engine (submit / step / run), for callers that stream."""
        return BatchMainLoop(self.core, self.chunk_size, self.max_batch_tokens, self.max_prefill_entries,
                             self.decode_ahead)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64, temperature: float = 1.0,
                 top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, seed: int = 42,
                 eos_token_id=None, return_reasons: bool = False):
        """Continue every prompt (token ids in, token ids out) with continuous batching.
        ``temperature=0`` is greedy.  ``eos_token_id``: an id or several that end a sequence; ``None`` takes them
        from the model's config.json, ``-1`` means none.  Request ``i`` draws from its own stream seeded ``seed + i``
        (as the reference's ``sample_batch``, src/ops/sampling.cpp:341-359)."""
        loop = self.new_loop()
        ids = [loop.submit(p, max_new_tokens, eos_token_id, temperature, top_k, top_p, min_p, seed + i)
               for i, p in enumerate(prompts)]
        loop.run()
        self.last_loop = loop
        outs = [loop.generated_tokens(i) for i in ids]
        if return_reasons:
            return outs, [loop.finish_reason(i) for i in ids]
        return outs

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The step function itself: logits (float32, on the device) at the wanted places."""
        return self.core.step(entries)
