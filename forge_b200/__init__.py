"""forge_b200: a single-GPU inference engine for the dense LLaMA decoder on NVIDIA B200 (sm_100a),
from a model folder (config.json + safetensors, or seeded random weights) to generated tokens.

    import forge_b200 as forge
    model = forge.Model(model_dir, device="cuda", dtype="bfloat16")
    model.generate(prompt_ids, max_new_tokens=32, do_sample=False)
"""
from .api import GenerateRequest, InferenceContext, Model, RequestScheduler, RequestStatus, SamplerConfig
from .config import ConfigError, load_config, register_architecture, registered_architectures
from .kernels import (profiler_disable, profiler_enable, profiler_enabled, profiler_print, profiler_reset,
                      profiler_summary)
from .log import Logger
from .weights import WeightError, write_random_model

__version__ = "0.1.0"

__all__ = ["Model", "InferenceContext", "RequestScheduler", "SamplerConfig", "GenerateRequest", "RequestStatus",
           "ConfigError", "WeightError", "load_config", "register_architecture", "registered_architectures",
           "write_random_model", "profiler_enable", "profiler_disable", "profiler_enabled", "profiler_reset",
           "profiler_summary", "profiler_print", "Logger", "__version__"]
