from .base import ConfigError, LayerSpec, ModelPlan, PartSpec
from .llama import LlamaConfig
from .registry import (config_from_dict, load_config, register_architecture, registered_architectures,
                       unregister_architecture)

# LLaMA-architecture checkpoints; Qwen2 files are the same decoder with q/k/v biases on by default
# (the reference routes both names to one engine, src/model/arch_registrations.cpp:46-71).
register_architecture("LlamaForCausalLM", LlamaConfig, replace=True)
register_architecture("Qwen2ForCausalLM", LlamaConfig, replace=True)

__all__ = ["ConfigError", "LayerSpec", "ModelPlan", "PartSpec", "LlamaConfig", "config_from_dict", "load_config",
           "register_architecture", "registered_architectures", "unregister_architecture"]
