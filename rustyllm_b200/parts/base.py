"""Interfaces of the parts a layer is put together from.

A part knows its own sizes and constants (constructor parameters), the parameters
it wants bound (``param_specs``) and how to run on the tokens of one step.  It
does not know which model it is in, which layer it is, or what the other layers
are.  The residual stream is always float32; a part reads a normed copy of it in
the compute dtype and adds its result into the residual in 32-bit.

Roles and what each must provide:

``Norm``
    ``forward(x, out_dtype, rows=None) -> Tensor``: x is the float32 residual
    ``[M, d]``; returns ``[M, d]`` (or ``[len(rows), d]``: only those rows) in
    ``out_dtype``.
``PositionEncoding``
    Used by a mixer; for rotary kinds: ``inv_freq`` (float32 device tensor),
    ``rotary_dim``, ``interleaved``.
``Mixer``
    ``kv_need() -> KVNeed | None`` and ``state_need() -> StateNeed | None``: what
    it wants cached per position, and what fixed-size state per sequence.
    ``forward(xn, residual, step, cache) -> None``: xn ``[M, d]`` compute dtype;
    adds the mixer's output to ``residual`` ``[M, d]`` float32 in place.  ``step``
    is the ``StepState`` (tokens' positions, slots, sequence boundaries);
    ``cache`` is this layer run's ``CacheView`` (key/value pools and page table,
    state area, and whether this layer writes them or only reads another's).
``FeedForward``
    ``forward(xn, residual, step) -> None``: same contract without a cache.
``Block``
    Built from (mixer, mixer_norm, feed_forward, feed_forward_norm);
    ``forward(x, step, cache) -> None`` updates the residual x in place.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..cache.sequence_cache import KVNeed, StateNeed
from ..config.spec import ParamSpec


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model runs."""
    device: torch.device
    compute_dtype: torch.dtype   # torch.float32 (true 32-bit everywhere) or torch.bfloat16


class Part:
    # False for a part whose ``forward`` reads device data on the host (or otherwise
    # cannot be captured in a CUDA graph); the engine then runs every step eagerly.
    graph_capturable: bool = True

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for k, v in tensors.items():
            setattr(self, k, v)

    def sub_parts(self) -> Dict[str, "Part"]:
        """Parts nested in this one (their parameters are bound under ``name.``)."""
        return {}


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step) -> None:
        raise NotImplementedError


class Block(Part):
    def forward(self, x: torch.Tensor, step, cache) -> None:
        raise NotImplementedError
