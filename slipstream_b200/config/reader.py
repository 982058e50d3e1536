"""A typed reader over the key/value pairs of a ``config.json``.

An architecture's configuration class asks the reader for each key it knows, with the type it expects; the
reader answers with a checked value or raises ``ConfigError`` naming the key.  Keys nobody asked for are the
``leftover``: a configuration keeps them so that writing it back loses nothing.

Accepted values follow the reference reader (slipstream/models/hf_config.py:60-153): whole numbers may be
written as floats (``4096.0``), booleans never count as numbers, a token id may be a list whose first element
is taken, and a second dictionary (``generation_config.json``) stands behind the first for token ids.  The
precision key differs on purpose: the reference also maps ``float16`` / ``fp16`` / ``half``
(hf_config.py:248-262); this engine computes in bfloat16 or float32 only and refuses any other name instead of
silently re-rounding a checkpoint.
"""

from __future__ import annotations

import json
import numbers
from pathlib import Path
from typing import Any

_MISSING = object()

PRECISIONS = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


class ConfigError(ValueError):
    """A ``config.json`` value is missing, mistyped or unsupported."""


def load_json_object(path: Path) -> dict[str, Any]:
    data = json.loads(Path(path).read_text(encoding="utf-8"))
    if not isinstance(data, dict):
        raise ConfigError(f"{path} is not a JSON object")
    return data


class ConfigReader:
    def __init__(self, data: dict[str, Any], behind: dict[str, Any] | None = None, where: str = "config.json") -> None:
        self.data = data
        self.behind = behind or {}
        self.where = where
        self.asked: set[str] = set()

    # ------------------------------------------------------------------ lookups
    def raw(self, key: str, default: Any = _MISSING) -> Any:
        """The stored value; JSON ``null`` counts as absent."""
        self.asked.add(key)
        value = self.data.get(key)
        if value is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where} lacks the required key {key!r}")
            return default
        return value

    def _fail(self, key: str, expected: str, value: Any) -> ConfigError:
        return ConfigError(f"{key} must be {expected}, got {type(value).__name__}: {value!r}")

    def integer(self, key: str, default: Any = _MISSING) -> Any:
        value = self.raw(key, default)
        if value is default:
            return value
        whole = isinstance(value, numbers.Integral) or (isinstance(value, float) and value == int(value))
        if isinstance(value, bool) or not whole:
            raise self._fail(key, "an integer", value)
        return int(value)

    def number(self, key: str, default: Any = _MISSING) -> Any:
        value = self.raw(key, default)
        if value is default:
            return value
        if isinstance(value, bool) or not isinstance(value, numbers.Real):
            raise self._fail(key, "a number", value)
        return float(value)

    def flag(self, key: str, default: Any = _MISSING) -> Any:
        value = self.raw(key, default)
        if value is default:
            return value
        if value is not True and value is not False:
            raise self._fail(key, "true or false", value)
        return value

    def text(self, key: str, default: Any = _MISSING) -> Any:
        value = self.raw(key, default)
        if value is default:
            return value
        if not isinstance(value, str):
            raise self._fail(key, "a string", value)
        return value

    def table(self, *keys: str) -> dict[str, Any] | None:
        """The first of ``keys`` that holds an object, or None."""
        for key in keys:
            value = self.raw(key, None)
            if value is None:
                continue
            if not isinstance(value, dict):
                raise self._fail(key, "an object", value)
            return value
        return None

    def token_id(self, key: str) -> int | None:
        """An id, or the first id of a list; ``generation_config.json`` answers where the model's file does not."""
        self.asked.add(key)
        for source in (self.data, self.behind):
            value = source.get(key)
            while isinstance(value, list) and value:
                value = value[0]
            if isinstance(value, bool):
                raise ConfigError(f"{key} must be a token id, not a boolean")
            if isinstance(value, numbers.Integral):
                return int(value)
        return None

    def precision(self, *keys: str, default: str = "bfloat16") -> str:
        """The dtype the checkpoint was stored in, as one of the engine's two precisions.  An absent key gives the
        default; a name the engine does not compute in is refused."""
        for key in keys:
            value = self.raw(key, None)
            if value is None:
                continue
            name = PRECISIONS.get(value) if isinstance(value, str) else None
            if name is None:
                raise ConfigError(f"{key} {value!r} is not supported: this engine computes in bfloat16 or float32")
            return name
        return default

    def leftover(self, also_known: tuple[str, ...] = ()) -> dict[str, Any]:
        return {k: v for k, v in self.data.items() if k not in self.asked and k not in also_known}
