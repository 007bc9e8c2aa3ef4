"""One registry from an architecture's name (``architectures[0]`` in config.json) to how its model is made.

The reference has no registry: its runner holds a ``Qwen3`` by value (engine/model_runner.h:97) and never
reads ``architectures``.  Here an architecture is an entry with two callables:

* ``parse_config(dict) -> config``   the typed configuration read from config.json's own keys;
* ``build_spec(config) -> ModelSpec``  the model as data: which mixer, feed-forward, norms and position
  encoding every layer has, with sizes as parameters, the tensor names of its weights, and the order in
  which layers run (see ``cppvllm_b200.parts.spec``).

The generic ``CausalLM`` (parts/model.py) builds itself from the ``ModelSpec``; nothing else in the package
knows which architecture it runs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], Any]
    model_types: tuple = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec, model_types=(), replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    arch = Architecture(name, parse_config, build_spec, tuple(model_types))
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_dict: Mapping[str, Any]) -> Architecture:
    """Choose the architecture for a config.json: ``architectures[0]``, else ``model_type``.

    A config.json with neither key is accepted only while exactly one architecture is registered (the
    reference never reads either key, so such files exist)."""
    from .. import models as _models  # noqa: F401  (the package's own architectures register themselves on import)
    archs = config_dict.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        name = str(archs[0])
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
        raise ConfigError(f"config.json: architecture '{name}' is not registered; registered: "
                          f"{registered_architectures()}")
    mt = config_dict.get("model_type")
    if mt is not None:
        for a in _ARCHITECTURES.values():
            if mt in a.model_types:
                return a
        raise ConfigError(f"config.json: model_type '{mt}' matches no registered architecture; registered: "
                          f"{registered_architectures()}")
    if len(_ARCHITECTURES) == 1:
        return next(iter(_ARCHITECTURES.values()))
    raise ConfigError("config.json names no architecture ('architectures' or 'model_type'); registered: "
                      f"{registered_architectures()}")
