"""A B200-native inference engine for the Qwen2 dense decoder: configuration and registry,
safetensors weights, a paged cache, one step function over mixed batches, a DecodeFirst
scheduler, sampling, and hand-written CUDA kernels for sm_100a."""
from .entry import Engine
from .engine import EngineCore, EngineOptions, StepEntry
from .sampling import SamplingParams
from .weights import write_random_model

__all__ = ["Engine", "EngineCore", "EngineOptions", "StepEntry", "SamplingParams", "write_random_model"]
__version__ = "0.1.0"
