"""One registry from an architecture's name (``config.json`` → ``architectures[0]``)
to its typed configuration class and the builder that turns a configuration
into a ``ModelSpec``.

The reference dispatches in ``create_model`` on config features and tensor
presence and never looks at ``architectures`` (src/model/model_factory.cpp:13-34);
here the name is the key, and an unknown name is an error that says so.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Type

from .model_config import ConfigError, ModelConfig, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    build_spec: Callable[[ModelConfig], Any]      # -> parts.base.ModelSpec
    random_tensors: Callable[..., Any] = None     # (config, seed, **opts) -> iterable of (name, shape, kind)


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], build_spec, random_tensors=None,
                          *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise KeyError(f"architecture '{name}' is already registered")
    arch = Architecture(name, config_cls, build_spec, random_tensors)
    _ARCHITECTURES[name] = arch
    return arch


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise ConfigError(f"config.json: unsupported architecture '{name}' (registered: {known})") from None


def registered_architectures() -> List[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def config_from_json(j: Dict[str, Any]) -> ModelConfig:
    """Typed configuration of whatever architecture the json names."""
    return get_architecture(architecture_name(j)).config_cls.from_json(j)


def config_from_dir(model_dir: str) -> ModelConfig:
    return config_from_json(read_config_json(model_dir))


def _ensure_builtin() -> None:
    # the built-in architecture registers itself on import
    from ..models import llama  # noqa: F401
