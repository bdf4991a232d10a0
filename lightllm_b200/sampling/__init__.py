from .params import SamplingParams
from .sampler import RequestStream, Sampler

__all__ = ["SamplingParams", "RequestStream", "Sampler"]
