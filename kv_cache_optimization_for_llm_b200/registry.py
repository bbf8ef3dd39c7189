"""One registry from an architecture's name (``architectures[0]`` or ``architecture`` of config.json) to
its typed configuration and its model description.  Upstream has one hard-wired
model and no registry."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional

from .models.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed configuration
    build_spec: Callable[[Any], ModelSpec]             # typed configuration -> model description
    # (typed configuration, tensor name -> shape of the checkpoint) -> configuration with the sizes
    # filled in that config.json leaves to the tensors' shapes; None: the file says everything
    complete: Optional[Callable[[Any, Mapping[str, Any]], Any]] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec, complete=None) -> None:
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec, complete)


def known_architectures():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def _load_builtin() -> None:
    from .models import llama, nonetar, rezusun, solulix, tevanex  # noqa: F401  (they register themselves)


def resolve_architecture(config_dict: Mapping[str, Any]) -> Architecture:
    _load_builtin()
    archs = config_dict.get("architectures") or []
    if not archs and config_dict.get("architecture"):
        archs = [config_dict["architecture"]]
    if not archs:
        raise ValueError("config.json: 'architectures' (or 'architecture') is missing or empty; known: "
                         + ", ".join(sorted(_ARCHITECTURES)))
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is not registered; known: " + ", ".join(sorted(_ARCHITECTURES)))
    return _ARCHITECTURES[name]
