"""Registries of parts by kind.

A model description names each part by a kind string ("rms_norm",
"gqa_attention", "gated_mlp", "rope", "pre_norm", ...); the decoder looks the
kind up here and builds the part from its parameters.  Anything registered under
a new kind - in this package or outside it - can be used in a layer without a
change to the framework's files.
"""
from __future__ import annotations

from typing import Callable, Dict

from ..config.spec import PartSpec

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
    "embedding": {}, "head": {},
}


def register(role: str, kind: str):
    """Class decorator: ``@register("mixer", "gqa_attention")``."""
    if role not in _REGISTRIES:
        raise KeyError(f"unknown role {role!r}; roles: {sorted(_REGISTRIES)}")

    def deco(cls):
        _REGISTRIES[role][kind] = cls
        return cls
    return deco


def register_mixer(kind): return register("mixer", kind)
def register_feed_forward(kind): return register("feed_forward", kind)
def register_norm(kind): return register("norm", kind)
def register_position(kind): return register("position", kind)
def register_block(kind): return register("block", kind)


def build_part(role: str, spec: PartSpec, runtime):
    """Instantiate the part ``spec.kind`` of the given role with its parameters."""
    reg = _REGISTRIES[role]
    if spec.kind not in reg:
        raise KeyError(f"no {role} of kind {spec.kind!r} is registered; known: {sorted(reg)}")
    return reg[spec.kind](runtime=runtime, **spec.params)


def known(role: str):
    return sorted(_REGISTRIES[role])
