"""Configuration dataclasses and their validation.

Mirrors entropack/schemes/config.py:8-111 -- same class names, field names, defaults, error types --
so a config written for the reference validates identically here. Field constraints are carried as
``Annotated`` markers and checked on every compress / decompress call.
"""
from dataclasses import dataclass, fields
from numbers import Real
from typing import Annotated, get_args, get_origin, get_type_hints

__all__ = ["CompressionConfig", "OneOf", "Range", "RawConfig", "config_fields", "validate_config"]


@dataclass
class CompressionConfig:
    """Settings common to every scheme; a concrete subclass selects the scheme."""

    #: ``"auto"`` / ``None`` / ``"b200"`` / ``"cuda"`` all select the one backend that exists here, the
    #: sm_100a kernel library. ``"eager"`` is rejected: there is no CPU lane.
    execution_backend: str | None = "auto"


@dataclass
class RawConfig(CompressionConfig):
    """Store the tensor without entropy coding (also the container of an encode that failed)."""


class Range:
    """Inclusive numeric bound; ``message`` replaces the generated text."""

    def __init__(self, low=None, high=None, *, message: str | None = None):
        self.low, self.high, self.message = low, high, message

    def holds(self, value) -> bool:
        return (self.low is None or value >= self.low) and (self.high is None or value <= self.high)

    def describe(self, name: str) -> str:
        if self.message is not None:
            return self.message
        if self.low is None:
            return f"{name} must be <= {self.high}"
        if self.high is None:
            return f"{name} must be >= {self.low}"
        return f"{name} must be in [{self.low}, {self.high}]"

    def __repr__(self) -> str:
        return f"Range({self.low!r}, {self.high!r})"


class OneOf:
    """Closed set of values; ``silent`` members stand for automatic selection."""

    def __init__(self, choices, *, silent=(), message: str | None = None):
        self.choices, self.silent, self.message = tuple(choices), frozenset(silent), message

    def holds(self, value) -> bool:
        return value in self.silent or value in self.choices

    def describe(self, name: str) -> str:
        return self.message or f"{name} must be one of {self.choices}"

    def __repr__(self) -> str:
        return f"OneOf({list(self.choices)!r})"


_field_cache: dict[type, dict] = {}


def config_fields(cls: type) -> dict:
    if cls not in _field_cache:
        hints = get_type_hints(cls, include_extras=True)
        _field_cache[cls] = {f.name: hints[f.name] for f in fields(cls) if f.name != "execution_backend"}
    return _field_cache[cls]


def _field_rule(hint) -> tuple:
    """(base type, nullable, markers) of an annotated field type such as ``Annotated[int | None, Range(1, None)]``."""
    markers = []
    if get_origin(hint) is Annotated:
        hint, *markers = get_args(hint)
    members = get_args(hint) if get_origin(hint) is not None else (hint,)
    kinds = [kind for kind in members if kind is not type(None)]
    return kinds[0], len(kinds) < len(members), tuple(markers)


_rule_cache: dict[type, list] = {}


def _field_rules(cls: type) -> list:
    """The rules of a config class, worked out from its type hints once (decode paths validate on every call)."""
    if cls not in _rule_cache:
        _rule_cache[cls] = [(name, *_field_rule(hint)) for name, hint in config_fields(cls).items()]
    return _rule_cache[cls]


def _validate_field(name: str, value, base, nullable: bool, markers) -> None:
    noun = "an integer" if base is int else "a bool" if base is bool else "a real number"
    if value is None:
        if nullable:
            return
        raise TypeError(f"{name} must be {noun}")
    if base is int:
        good = isinstance(value, int) and not isinstance(value, bool)
    elif base is bool:
        good = isinstance(value, bool)
    else:
        good = isinstance(value, Real) and not isinstance(value, bool)
    if not good:
        raise TypeError(f"{name} must be {noun}{' or None' if nullable else ''}")
    for marker in markers:
        if not marker.holds(value):
            raise ValueError(marker.describe(name))


def validate_config(config) -> None:
    for name, base, nullable, markers in _field_rules(type(config)):
        _validate_field(name, getattr(config, name), base, nullable, markers)
