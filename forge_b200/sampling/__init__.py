from .sampler import RequestSampler, SamplerConfig, XorShift64, sample_batch

__all__ = ["RequestSampler", "SamplerConfig", "XorShift64", "sample_batch"]
