"""Typed model configurations and the registry from architecture name to model.

A configuration class mirrors the keys of one architecture's ``config.json``.
The registry maps the name in ``architectures[0]`` (or ``model_type``) to the
pair (configuration class, function that lays the model out from it).  Adding
an architecture means one ``register_architecture`` call; nothing else in the
framework names an architecture.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, ClassVar


class ConfigError(ValueError):
    """A config.json that cannot be read or that describes an impossible model."""


@dataclasses.dataclass
class ModelConfig:
    """Base of the typed configurations.

    Subclasses declare one dataclass field per ``config.json`` key they read.
    A key that is absent or ``null`` takes the field's default, as wlejon/brolm's
    JSON getters do (include/brolm/detail/json.h:88-119).
    """

    architecture: ClassVar[str] = ""
    model_types: ClassVar[tuple[str, ...]] = ()

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"{cls.__name__}: root is not a JSON object")
        kwargs = {}
        for f in dataclasses.fields(cls):
            value = raw.get(f.name)
            if value is None:
                continue
            kwargs[f.name] = _coerce(cls.__name__, f, value)
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    @classmethod
    def from_json_text(cls, text: str) -> "ModelConfig":
        try:
            raw = json.loads(text)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{cls.__name__}: json parse: {e}") from e
        return cls.from_dict(raw)

    @classmethod
    def from_json(cls, path: str) -> "ModelConfig":
        try:
            with open(path, "r", encoding="utf-8") as fh:
                text = fh.read()
        except OSError as e:
            raise ConfigError(f"{cls.__name__}: cannot open '{path}'") from e
        return cls.from_json_text(text)

    @classmethod
    def from_dir(cls, folder: str) -> "ModelConfig":
        return cls.from_json(os.path.join(folder, "config.json"))

    def to_dict(self) -> dict[str, Any]:
        """The config.json content that reads back to an equal configuration."""
        out: dict[str, Any] = {"architectures": [self.architecture]}
        if self.model_types:
            out["model_type"] = self.model_types[0]
        for f in dataclasses.fields(self):
            out[f.name] = getattr(self, f.name)
        return out

    def validate(self) -> None:  # pragma: no cover - overridden
        pass


def _coerce(owner: str, f: dataclasses.Field, value: Any) -> Any:
    kind = f.type if isinstance(f.type, str) else getattr(f.type, "__name__", str(f.type))
    try:
        if kind == "int":
            if isinstance(value, bool) or (isinstance(value, float) and value != int(value)):
                raise TypeError
            return int(value)
        if kind == "float":
            if isinstance(value, bool):
                raise TypeError
            return float(value)
        if kind == "bool":
            if not isinstance(value, bool):
                raise TypeError
            return value
        if kind.startswith("tuple") or kind.startswith("list") or "tuple" in kind:
            if not isinstance(value, (list, tuple)):
                raise TypeError
            return tuple(value)
    except (TypeError, ValueError):
        raise ConfigError(f"{owner}: key '{f.name}' has the wrong type: {value!r}") from None
    return value


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    layout: Callable[[Any], Any]   # configuration -> parts.ModelLayout


_ARCHITECTURES: dict[str, Architecture] = {}
_MODEL_TYPES: dict[str, str] = {}


def register_architecture(config_cls: type, layout: Callable[[Any], Any]) -> None:
    name = config_cls.architecture
    if not name:
        raise ValueError("a configuration class needs an architecture name")
    _ARCHITECTURES[name] = Architecture(name, config_cls, layout)
    for mt in config_cls.model_types:
        _MODEL_TYPES[mt] = name


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(raw: dict[str, Any]) -> Architecture:
    """Pick the architecture a parsed config.json names."""
    names = raw.get("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = raw.get("model_type")
    if mt in _MODEL_TYPES:
        return _ARCHITECTURES[_MODEL_TYPES[mt]]
    raise ConfigError(
        f"no registered architecture for architectures={names!r} model_type={mt!r}; "
        f"registered: {registered_architectures()}")


def load_config(folder_or_file: str) -> ModelConfig:
    """Read config.json and return the typed configuration of its architecture."""
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            text = fh.read()
    except OSError as e:
        raise ConfigError(f"config: cannot open '{path}'") from e
    try:
        raw = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"config: json parse: {e}") from e
    if not isinstance(raw, dict):
        raise ConfigError("config: root is not a JSON object")
    return architecture_of(raw).config_cls.from_dict(raw)
