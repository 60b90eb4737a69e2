"""Reading typed values out of a config.json dictionary."""
from __future__ import annotations

from pathlib import Path

from ..errors import FormatError, MissingKey

_MISSING = object()


class ConfigReader:
    """Typed access to the keys of one config.json.

    Every getter names the key in its error, as the engine of MythEclipse/llm
    names the metadata key it misses (apps/engine/src/model.rs:81-83).
    Unknown keys are ignored.
    """

    def __init__(self, raw: dict, where: str = "config.json"):
        if not isinstance(raw, dict):
            raise FormatError(f"{where}: top level is not an object")
        self.raw = raw
        self.where = where

    def _get(self, key, default):
        value = self.raw.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                raise MissingKey(key, self.where)
            return default
        return value

    def integer(self, key, default=_MISSING, minimum=None):
        value = self._get(key, default)
        if value is None:
            return None
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value == int(value):
                value = int(value)
            else:
                raise FormatError(f"{self.where}: '{key}' must be an integer, found {value!r}")
        if minimum is not None and value < minimum:
            raise FormatError(f"{self.where}: '{key}' must be at least {minimum}, found {value}")
        return value

    def number(self, key, default=_MISSING, positive=False):
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise FormatError(f"{self.where}: '{key}' must be a number, found {value!r}")
        value = float(value)
        if positive and not value > 0.0:
            raise FormatError(f"{self.where}: '{key}' must be positive, found {value}")
        return value

    def boolean(self, key, default=_MISSING):
        value = self._get(key, default)
        if not isinstance(value, bool):
            raise FormatError(f"{self.where}: '{key}' must be true or false, found {value!r}")
        return value

    def string(self, key, default=_MISSING):
        value = self._get(key, default)
        if value is not None and not isinstance(value, str):
            raise FormatError(f"{self.where}: '{key}' must be a string, found {value!r}")
        return value

    def mapping(self, key, default=_MISSING):
        value = self._get(key, default)
        if value is not None and not isinstance(value, dict):
            raise FormatError(f"{self.where}: '{key}' must be an object, found {value!r}")
        return value

    def integer_list(self, key, default=_MISSING):
        """An integer or a list of integers, returned as a tuple."""
        value = self._get(key, default)
        if value is None:
            return ()
        if isinstance(value, int) and not isinstance(value, bool):
            return (value,)
        if isinstance(value, (list, tuple)) and all(
                isinstance(v, int) and not isinstance(v, bool) for v in value):
            return tuple(value)
        raise FormatError(f"{self.where}: '{key}' must be an integer or a list of integers")


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FormatError(f"{path}: no such file")
    from .. import native
    raw = native.read_json(path.read_bytes(), str(path))         # the host library's own reader
    if not isinstance(raw, dict):
        raise FormatError(f"{path}: the configuration must be a JSON object")
    return raw
