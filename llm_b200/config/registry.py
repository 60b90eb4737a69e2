"""One registry from an architecture's name to its configuration class.

A configuration class has `from_dict(raw, where)`, `to_dict()` and
`model_spec()`; the model itself is always the generic decoder of
`llm_b200.engine.model`, built from that spec.
"""
from __future__ import annotations

from ..errors import FormatError, Unsupported
from .base import read_config_json

_ARCHITECTURES: dict = {}


def register_architecture(name: str, config_class) -> None:
    _ARCHITECTURES[name] = config_class


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise Unsupported(f"architecture '{name}' is not registered "
                          f"(known: {', '.join(known_architectures())})") from None


def config_from_dict(raw: dict, where: str = "config.json"):
    """Pick the class by `architectures[0]` and parse."""
    archs = raw.get("architectures") if isinstance(raw, dict) else None
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise FormatError(f"{where}: 'architectures' must be a non-empty list of names")
    return config_class_for(archs[0]).from_dict(raw, where)


def load_config(folder):
    return config_from_dict(read_config_json(folder), f"{folder}/config.json")
