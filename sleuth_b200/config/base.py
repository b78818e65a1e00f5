"""Typed reading of a model folder's ``config.json``.

An architecture declares a frozen dataclass whose field names are the keys of its own
``config.json``. ``read_fields`` fills it from the parsed JSON with type checks, defaults and clear
errors; keys the dataclass does not name are kept aside in ``unread`` (a ``config.json`` carries
bookkeeping such as ``transformers_version`` that no formula needs), so nothing is silently
misread and nothing harmless is refused.

The strict dict -> dataclass idea follows sleuth/config.py:57-107 (type coercion where an int may
stand for a float, an error that names the key); the key set and defaults of the Qwen3 family are
those of sleuth/formats/hf.py:83-118.
"""

from __future__ import annotations

import dataclasses
import difflib
import json
import types
import typing
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong type, or asks for something unsupported."""


def _coerce(val: Any, typ: Any, name: str) -> Any:
    origin = typing.get_origin(typ)
    if origin in (typing.Union, types.UnionType):
        errors = []
        for a in typing.get_args(typ):
            try:
                return _coerce(val, a, name)
            except ConfigError as e:
                errors.append(str(e))
        raise ConfigError(f"{name}: {val!r} does not match {typ}")
    if typ is type(None):
        if val is not None:
            raise ConfigError(f"{name}: expected null, got {val!r}")
        return None
    if typ is float:
        if isinstance(val, bool) or not isinstance(val, (int, float)):
            raise ConfigError(f"{name}: expected a number, got {val!r}")
        return float(val)
    if typ is int:
        if isinstance(val, bool) or not isinstance(val, int):
            raise ConfigError(f"{name}: expected an integer, got {val!r}")
        return val
    if typ is bool:
        if not isinstance(val, bool):
            raise ConfigError(f"{name}: expected true or false, got {val!r}")
        return val
    if typ is str:
        if not isinstance(val, str):
            raise ConfigError(f"{name}: expected a string, got {val!r}")
        return val
    if origin in (list, tuple):
        if not isinstance(val, (list, tuple)):
            raise ConfigError(f"{name}: expected a list, got {val!r}")
        args = typing.get_args(typ)
        inner = args[0] if args else Any
        return tuple(_coerce(v, inner, f"{name}[{i}]") if inner is not Any else v for i, v in enumerate(val))
    return val


def read_fields(cls, d: dict, where: str = "config.json"):
    """Build dataclass ``cls`` from the parsed JSON ``d``.

    Every dataclass field is a key of ``d`` (same spelling). A field without a default is required.
    Returns ``(instance, unread)`` where ``unread`` lists the keys of ``d`` that ``cls`` does not name.
    """
    if not isinstance(d, dict):
        raise ConfigError(f"{where}: expected a JSON object, got {type(d).__name__}")
    hints = typing.get_type_hints(cls)
    kwargs = {}
    for f in dataclasses.fields(cls):
        if not f.init:
            continue
        if f.name in d and d[f.name] is not None:
            kwargs[f.name] = _coerce(d[f.name], hints[f.name], f"{where}: {f.name}")
        elif f.name in d and d[f.name] is None and _allows_none(hints[f.name]):
            kwargs[f.name] = None
        elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING:
            close = difflib.get_close_matches(f.name, list(d), n=1)
            hint = f" (it has {close[0]!r}; a misspelling?)" if close else ""
            raise ConfigError(f"{where}: required key {f.name!r} is missing{hint}")
    names = {f.name for f in dataclasses.fields(cls)}
    unread = sorted(k for k in d if k not in names)
    return cls(**kwargs), unread


def _allows_none(typ) -> bool:
    origin = typing.get_origin(typ)
    return origin in (typing.Union, types.UnionType) and type(None) in typing.get_args(typ)


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.exists():
        raise ConfigError(f"{folder}: no config.json (a model folder holds config.json and model.safetensors)")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
