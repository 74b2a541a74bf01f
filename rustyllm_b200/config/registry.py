"""One registry from an architecture's name to its configuration and model.

Counterpart of the reference's ``architecture_supported`` string list and its
``match arch`` loader dispatch (src/runtime.rs:1087-1135, 1987-2017); an unknown
name is an error that lists the known ones (src/runtime.rs:1236-1245).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Sequence

from .spec import ModelSpec


class UnknownArchitecture(KeyError):
    pass


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed config
    build_spec: Callable[[Any], ModelSpec]             # typed config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(names: Sequence[str], parse_config, build_spec) -> Architecture:
    """Register one architecture under every name config.json may carry for it
    (an entry of ``architectures`` or the ``model_type``)."""
    arch = Architecture(name=names[0], parse_config=parse_config, build_spec=build_spec)
    for n in names:
        _ARCHITECTURES[n] = arch
    return arch


def known_architectures() -> Sequence[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_dict: Mapping[str, Any]) -> Architecture:
    """Pick the architecture by ``architectures[0]``, else by ``model_type``."""
    candidates = []
    archs = config_dict.get("architectures")
    if isinstance(archs, (list, tuple)):
        candidates.extend(a for a in archs if isinstance(a, str))
    mt = config_dict.get("model_type")
    if isinstance(mt, str):
        candidates.append(mt)
    for c in candidates:
        if c in _ARCHITECTURES:
            return _ARCHITECTURES[c]
    raise UnknownArchitecture(
        f"Unsupported architecture: {candidates or '(config.json names none)'}; "
        f"known: {list(known_architectures())}")
