"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

An architecture is four functions, and nothing else in the package knows a model by name:

    parse_config(dict)            -> a typed, validated configuration
    weight_spec(config)           -> the tensors a checkpoint must hold (names, shapes)
    random_weights(config, seed)  -> a name -> tensor dict with those names and shapes
    build(config, weights, rt)    -> a DecoderModel assembled from parts

The reference keys models by Python module path (kelpie-http/kelpie_http/sdk/serve.py:34-44,
127-129) and states the model contract as `load / attn_specs / forward`
(kelpie-models/kelpie_models/sdk/run.py:283-284); this registry is keyed by the name that
config.json itself carries instead.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable


class ConfigError(ValueError):
    """A configuration that cannot be used: names the key and what is wrong with it."""


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], Any]
    weight_spec: Callable[[Any], list]
    random_weights: Callable[..., dict]
    build: Callable[..., Any]
    config_to_json: Callable[[Any], dict]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    if arch.name in _ARCHITECTURES:
        raise ConfigError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def architecture_of(config_json: dict) -> Architecture:
    """The architecture that a config.json names in `architectures`."""
    names = config_json.get("architectures")
    if not isinstance(names, list) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError(
            f"config.json must name exactly one model in 'architectures', got {names!r}; "
            f"known: {', '.join(known_architectures())}"
        )
    return architecture(names[0])


def read_config_json(model_dir: str | Path) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as err:
        raise ConfigError(f"{path}: not valid JSON ({err})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return data


def load_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """(architecture, typed configuration) of a model folder."""
    data = read_config_json(model_dir)
    arch = architecture_of(data)
    return arch, arch.parse_config(data)
