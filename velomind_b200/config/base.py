"""Typed reading of config.json keys with errors that name the key."""
from __future__ import annotations

import json
import math
import os
from typing import Any, Dict, Iterable, Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong kind, or asks for something unsupported."""


_MISSING = object()


class KeyReader:
    """Wraps the parsed config.json object; every getter checks type and range and names the key on failure."""

    def __init__(self, data: Dict[str, Any], where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: top level is not a JSON object")
        self.data = data
        self.where = where

    def _get(self, key: str, default):
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: missing required key '{key}'")
        return default

    def integer(self, key: str, default=_MISSING, minimum: int = 1) -> int:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{self.where}: key '{key}' must be an integer, found {v!r}")
        v = int(v)
        if v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, found {v}")
        return v

    def number(self, key: str, default=_MISSING, positive: bool = True) -> float:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
            raise ConfigError(f"{self.where}: key '{key}' must be a finite number, found {v!r}")
        if positive and v <= 0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, found {v}")
        return float(v)

    def boolean(self, key: str, default=_MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, found {v!r}")
        return v

    def string(self, key: str, default=_MISSING) -> str:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, found {v!r}")
        return v

    def int_or_list(self, key: str) -> tuple:
        """`eos_token_id`-style keys: absent/null -> (), an int -> (int,), a list of ints -> tuple."""
        v = self.data.get(key)
        if v is None:
            return ()
        items: Iterable = v if isinstance(v, list) else [v]
        out = []
        for x in items:
            if isinstance(x, bool) or not isinstance(x, int):
                raise ConfigError(f"{self.where}: key '{key}' must be an integer or a list of integers, found {v!r}")
            out.append(int(x))
        return tuple(out)

    def absent_or(self, key: str, allowed: Iterable, why: str) -> None:
        """Reject an option this library does not implement instead of ignoring it."""
        if key in self.data and self.data[key] is not None and self.data[key] not in tuple(allowed):
            raise ConfigError(f"{self.where}: key '{key}' = {self.data[key]!r} is not supported ({why})")


def read_config_json(folder_or_file: str) -> Dict[str, Any]:
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    try:
        with open(path, "r", encoding="utf-8") as f:
            data = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level is not a JSON object")
    return data
