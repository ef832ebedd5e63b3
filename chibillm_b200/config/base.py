"""Typed reading of ``config.json`` keys with errors that name the key."""
from __future__ import annotations

import json
import math
import os
from typing import Any, Optional


class ConfigError(ValueError):
    """A configuration problem.  ``code`` is one of the reference's classes of
    error (src/qwen/qwen_configs.h:16-24); the message names the key."""

    def __init__(self, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.code = code


_MISSING = object()


class KeyReader:
    """Reads typed values from a parsed JSON object and remembers which keys
    were looked at."""

    def __init__(self, obj: dict):
        if not isinstance(obj, dict):
            raise ConfigError("invalid_json", "config.json must hold a JSON object")
        self.obj = obj

    def has(self, key: str) -> bool:
        return key in self.obj and self.obj[key] is not None

    def raw(self, key: str, default: Any = _MISSING) -> Any:
        if key not in self.obj:
            if default is _MISSING:
                raise ConfigError("missing_field", f"key '{key}' is required")
            return default
        return self.obj[key]

    def positive_int(self, key: str, default: Any = _MISSING) -> int:
        v = self.raw(key, default)
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ConfigError("invalid_field", f"key '{key}' must be a positive integer, got {v!r}")
        return v

    def optional_positive_int(self, key: str) -> Optional[int]:
        if not self.has(key):
            return None
        return self.positive_int(key)

    def positive_float(self, key: str, default: Any = _MISSING) -> float:
        v = self.raw(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
            raise ConfigError("invalid_field", f"key '{key}' must be a positive finite number, got {v!r}")
        return float(v)

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self.raw(key, default)
        if not isinstance(v, bool):
            raise ConfigError("invalid_field", f"key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self.raw(key, default)
        if not isinstance(v, str):
            raise ConfigError("invalid_field", f"key '{key}' must be a string, got {v!r}")
        return v

    def token_id(self, key: str) -> Optional[int]:
        """A token id, or the first of a list of ids; None when absent."""
        if not self.has(key):
            return None
        v = self.obj[key]
        if isinstance(v, list) and v:
            v = v[0]
        if isinstance(v, bool) or not isinstance(v, int) or v < 0 or v > 2**31 - 1:
            raise ConfigError("invalid_field", f"key '{key}' must be a token id, got {v!r}")
        return v

    def require_value(self, key: str, allowed, code: str = "unsupported_configuration",
                      default: Any = _MISSING) -> Any:
        v = self.raw(key, default)
        if v not in allowed:
            raise ConfigError(code, f"key '{key}' is {v!r}; supported: {sorted(map(repr, allowed))}")
        return v

    def require_null_or_missing(self, key: str) -> None:
        if self.has(key):
            raise ConfigError("unsupported_configuration",
                              f"key '{key}' must be null or absent, got {self.obj[key]!r}")


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
    except OSError as e:
        raise ConfigError("file_read_failed", f"cannot read {path}: {e}") from None
    try:
        obj = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError("invalid_json", f"{path}: {e}") from None
    if not isinstance(obj, dict):
        raise ConfigError("invalid_json", f"{path} must hold a JSON object")
    return obj
