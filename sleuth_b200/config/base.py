"""Typed reading of a model folder's ``config.json``.

An architecture declares a frozen dataclass whose field names are the keys of its own
``config.json``. ``read_fields`` fills it from the parsed JSON with type checks, defaults and clear
errors; keys the dataclass does not name are kept aside in ``unread`` (a ``config.json`` carries
bookkeeping such as ``transformers_version`` that no formula needs), so nothing is silently
misread and nothing harmless is refused.

The reference reads its own TOML run configurations as strictly (sleuth/config.py:57-107: unknown
keys refused with a hint, an integer accepted where a float is wanted, errors that name the key);
here the rules are a table by annotation (``_PLAIN``). The key set and defaults of the Qwen3 family
are those of sleuth/formats/hf.py:83-118.
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


def _is_number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _is_integer(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


# What a JSON value must be for each plain annotation: (test, the words the error uses, how the value is kept).
# JSON has one number type, so an integer may stand where a float is wanted; nothing else converts.
_PLAIN = {
    float: (_is_number, "a number", float),
    int: (_is_integer, "an integer", lambda v: v),
    bool: (lambda v: isinstance(v, bool), "true or false", lambda v: v),
    str: (lambda v: isinstance(v, str), "a string", lambda v: v),
    type(None): (lambda v: v is None, "null", lambda v: v),
}


def _alternatives(annotation) -> tuple:
    """The member types of ``X | Y`` / ``Optional[X]``; the annotation itself otherwise."""
    if typing.get_origin(annotation) in (typing.Union, types.UnionType):
        return typing.get_args(annotation)
    return (annotation,)


def _fit(value: Any, annotation: Any, where: str) -> Any:
    """``value`` as the field annotated ``annotation`` keeps it, or a ConfigError naming ``where``."""
    wanted = []
    for alt in _alternatives(annotation):
        if alt in _PLAIN:
            test, words, keep = _PLAIN[alt]
            if test(value):
                return keep(value)
            wanted.append(words)
        elif typing.get_origin(alt) in (list, tuple):
            if isinstance(value, (list, tuple)):
                item = (typing.get_args(alt) or (Any,))[0]
                return tuple(_fit(v, item, f"{where}[{i}]") for i, v in enumerate(value))
            wanted.append("a list")
        else:
            return value                # Any, or an annotation this reader has no rule for: taken as it is
    raise ConfigError(f"{where}: expected {' or '.join(wanted)}, got {value!r}")


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
            kwargs[f.name] = _fit(d[f.name], hints[f.name], f"{where}: {f.name}")
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
    return type(None) in _alternatives(typ)


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.exists():
        raise ConfigError(f"{folder}: no config.json (a model folder holds config.json and model.safetensors)")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
