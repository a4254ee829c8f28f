"""One registry from an architecture's name (config.json ``architectures[0]``) to its family.

The reference has no such table: one engine class branches on config flags
(src/engine/batched_engine.ts:834,1186,824).  Here a family is a config class
that parses its own config.json keys and yields a :class:`ModelSpec`; the model
itself is assembled from registered parts by ``parts.model.build_model``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

from .specs import ConfigError, ModelSpec


@dataclass(frozen=True)
class Family:
    name: str
    # parse(raw config.json dict) -> typed config with .to_spec() and .to_dict()
    parse: Callable[[Dict[str, Any]], Any]


_FAMILIES: Dict[str, Family] = {}


def register_architecture(name: str, parse: Callable[[Dict[str, Any]], Any]) -> None:
    """Make ``name`` (as written in config.json ``architectures``) loadable."""
    _FAMILIES[name] = Family(name, parse)


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_FAMILIES))


def family_for(raw: Dict[str, Any]) -> Family:
    archs = raw.get("architectures") or []
    if isinstance(archs, str):
        archs = [archs]
    for a in archs:
        if a in _FAMILIES:
            return _FAMILIES[a]
    raise ConfigError(
        f"no registered architecture among {list(archs)!r}; "
        f"registered: {list(registered_architectures())}")


def parse_config(raw: Dict[str, Any]) -> Any:
    """Typed config of whichever family config.json names."""
    return family_for(raw).parse(raw)


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.exists(path):
        raise ConfigError(f"config.json not found at {path}")
    with open(path) as f:
        return json.load(f)


def load_config(model_dir: str) -> Any:
    return parse_config(read_config_json(model_dir))


def _register_builtin() -> None:
    from .qwen3 import Qwen3Config
    register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict)


_register_builtin()
