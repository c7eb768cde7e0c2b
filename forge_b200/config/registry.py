"""One registry from an architecture's name (config.json ``architectures[0]``) to its configuration class.

The reference keeps four singleton maps keyed by architecture and fills them from static objects of one
translation unit (src/model/arch_registrations.cpp:46-71, include/forge/model.h:330-445); here one explicit
table does that job.  A configuration class offers ``from_dict(d, architecture) -> config``,
``config.plan() -> ModelPlan`` and ``config.to_dict()``.
"""
import json
import os

from .base import ConfigError

_ARCHITECTURES = {}


def register_architecture(name, config_cls, replace=False):
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    for attr in ("from_dict", "plan", "to_dict"):
        if not hasattr(config_cls, attr):
            raise ConfigError(f"configuration class for {name!r} lacks '{attr}'")
    _ARCHITECTURES[name] = config_cls


def unregister_architecture(name):
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(d):
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"no model registered for architecture {name!r}; known: {registered_architectures()}")
    return _ARCHITECTURES[name].from_dict(d, architecture=name)


def load_config(model_dir):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)
