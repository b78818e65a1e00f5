"""One registry from an architecture's name to its configuration class and model description.

``config.json`` names its architecture in ``architectures[0]`` (``"Qwen3ForCausalLM"``) and, more
loosely, in ``model_type`` (``"qwen3"``); either finds the entry. The reference keeps the same
association implicitly (``SUPPORTED`` and the ``model_type`` -> ``architectures`` map,
sleuth/formats/hf.py:43,329-331) and refuses an unknown ``model_type`` (hf.py:84-86).

Adding an architecture is one call::

    register_architecture("MyForCausalLM", MyConfig, my_model_spec, model_types=("my",))

where ``MyConfig`` is a dataclass whose fields are the ``config.json`` keys and ``my_model_spec(cfg,
tensor_names=None)`` returns a ``parts.spec.ModelSpec``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .base import ConfigError, read_fields


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    model_spec: Callable


_BY_NAME: dict[str, Architecture] = {}
_BY_MODEL_TYPE: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, model_spec: Callable, model_types=()) -> Architecture:
    arch = Architecture(name, config_class, model_spec)
    _BY_NAME[name] = arch
    for mt in model_types:
        _BY_MODEL_TYPE[mt] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _BY_NAME.pop(name, None)
    for mt in [k for k, v in _BY_MODEL_TYPE.items() if v is arch]:
        del _BY_MODEL_TYPE[mt]


def registered_architectures() -> list[str]:
    return sorted(_BY_NAME)


def find_architecture(config_json: dict) -> Architecture:
    names = config_json.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _BY_NAME:
            return _BY_NAME[n]
    mt = config_json.get("model_type")
    if mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    raise ConfigError(f"config.json names architecture {names or None} (model_type {mt!r}); "
                      f"registered: {registered_architectures()}")


def parse_config(config_json: dict):
    """(architecture entry, typed configuration, keys of config.json nobody read)."""
    arch = find_architecture(config_json)
    d = {k: v for k, v in config_json.items() if k != "architectures"}
    cfg, unread = read_fields(arch.config_class, d)
    return arch, cfg, unread
