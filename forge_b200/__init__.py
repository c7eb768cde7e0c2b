"""forge_b200: a single-GPU inference engine for the dense LLaMA decoder on NVIDIA B200 (sm_100a),
from a model folder (config.json + safetensors, or seeded random weights) to generated tokens.
"""
from .config import ConfigError, load_config, register_architecture, registered_architectures

__version__ = "0.1.0"

__all__ = ["ConfigError", "load_config", "register_architecture", "registered_architectures", "__version__"]
