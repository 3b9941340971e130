"""One table from an architecture's name to its configuration class.

Kapel has a `match model_type` inside its parser and answers "unsupported architecture"
otherwise (crates/kapel-models/src/config.rs:279-294). Here the table is open: a new
architecture registers a class with `from_json(dict)`, `to_json()`, `to_spec()` and
`init_std(name, shape)`, under the names config.json uses (`architectures[0]` and
`model_type`).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Tuple

from .gemma2 import ConfigError, Gemma2Config

_ARCHITECTURES: Dict[str, type] = {}


def register_architecture(config_cls, *names: str) -> None:
    """Registers `config_cls` under each of `names`; a name held by another class is refused."""
    for n in names:
        if n in _ARCHITECTURES and _ARCHITECTURES[n] is not config_cls:
            raise ValueError(f"architecture name {n!r} is already registered")
        _ARCHITECTURES[n] = config_cls


def unregister_architecture(*names: str) -> None:
    for n in names:
        _ARCHITECTURES.pop(n, None)


def architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def config_class_for(raw: dict):
    """The class for a parsed config.json: `architectures[0]` first, then `model_type`."""
    names = []
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs:
        names.append(archs[0])
    if raw.get("model_type") is not None:
        names.append(raw["model_type"])
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(
        f"unsupported architecture {names or 'none named'}; this engine knows {list(architectures())}"
    )


def config_from_json(raw: dict):
    return config_class_for(raw).from_json(raw)


def config_from_dir(folder) -> Tuple[object, dict]:
    """(typed configuration, raw JSON) of a model folder."""
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON ({e})") from None
    return config_from_json(raw), raw


PRESETS = Path(__file__).resolve().parent / "presets"


def presets() -> Tuple[str, ...]:
    """Names of the config.json files that come with the package (`config/presets/NAME.json`)."""
    return tuple(sorted(p.stem for p in PRESETS.glob("*.json")))


def read_config_file(name_or_path) -> dict:
    """The raw JSON of a config.json given by path, or of a preset given by name."""
    path = Path(str(name_or_path))
    if not path.is_file() and (PRESETS / f"{name_or_path}.json").is_file():
        path = PRESETS / f"{name_or_path}.json"
    if path.is_dir():
        path = path / "config.json"
    if not path.is_file():
        raise ConfigError(f"{name_or_path}: neither a config.json nor one of the presets {list(presets())}")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: not a JSON object")
    return raw


register_architecture(Gemma2Config, Gemma2Config.architecture, Gemma2Config.model_type)
