"""One registry from an architecture's name (config.json ``architectures[0]``)
to its typed configuration.  The reference maps ``general.architecture`` to an
enum the same way and refuses unknown names (crates/model/src/lib.rs:37-54).
"""

from __future__ import annotations

import json
from pathlib import Path

from ..errors import ConfigError, UnsupportedArch

_ARCHITECTURES: dict = {}


def register_architecture(name: str, config_cls) -> None:
    """``config_cls`` needs ``from_dict(dict)`` and ``to_spec() -> ModelSpec``."""
    _ARCHITECTURES[name] = config_cls


def architectures() -> list:
    return sorted(_ARCHITECTURES)


def config_class(name: str):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnsupportedArch(name, _ARCHITECTURES) from None


def architecture_name(raw: dict) -> str:
    names = raw.get("architectures")
    if not names or not isinstance(names, (list, tuple)) or not isinstance(names[0], str):
        raise ConfigError("config.json has no 'architectures' entry naming the model")
    return names[0]


def read_config(source):
    """Typed configuration from a model folder, a config.json path or a dict."""
    if isinstance(source, dict):
        raw = source
    else:
        path = Path(source)
        if path.is_dir():
            path = path / "config.json"
        if not path.is_file():
            raise ConfigError(f"no config.json at {path}")
        try:
            raw = json.loads(path.read_text())
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    cfg = config_class(architecture_name(raw)).from_dict(raw)
    # A model folder may carry its authors' sampling settings beside the configuration.
    if not isinstance(source, dict):
        gen = Path(source)
        gen = (gen if gen.is_dir() else gen.parent) / "generation_config.json"
        if gen.is_file() and hasattr(cfg, "generation"):
            try:
                cfg.generation = {k: v for k, v in json.loads(gen.read_text()).items()
                                  if k in ("temperature", "top_k", "top_p", "repetition_penalty")}
            except (json.JSONDecodeError, OSError):
                pass
    return cfg
