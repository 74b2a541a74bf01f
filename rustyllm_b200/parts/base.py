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
    ``forward(x, step, cache, pending=None, next_norm=None)`` updates the residual x in
    place.

Norm folding (optional, see ``NormRequest`` / ``NormedInput``): a product that adds into the
residual can start the norm that follows it, and the product behind that norm finishes it,
which saves the norm's own kernel.  Parts that can do so say ``folds_norms = True``; every
other part is called with plain tensors as described above.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..cache.sequence_cache import KVNeed, StateNeed
from ..config.spec import ParamSpec


@dataclass(frozen=True)
class NormRequest:
    """What a product needs to prepare a row norm of its result for whoever reads it
    next: y = x / sqrt(mean(x^2) + eps) * weight."""
    weight: torch.Tensor          # [d] float32
    eps: float


@dataclass
class NormedInput:
    """A row norm that is started but not finished.  ``weighted`` = x * norm weight in the
    compute dtype ([M, d]); ``sumsq`` [M, pieces] float32 = the sum of squares of each row
    of x, in pieces.  The matrix product that reads it multiplies its result rows by
    rsqrt(sum(sumsq[m]) / d + eps), which is the same as normalising its input."""
    weighted: torch.Tensor
    sumsq: torch.Tensor
    eps: float

    @property
    def shape(self):
        return self.weighted.shape

    @property
    def dtype(self):
        return self.weighted.dtype

    @property
    def device(self):
        return self.weighted.device


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

    def request(self) -> Optional[NormRequest]:
        """If this norm is y = x / sqrt(mean(x^2) + eps) * weight, what a neighbouring
        product needs to do it on the way (else ``None``: the norm runs its own kernel)."""
        return None


class PositionEncoding(Part):
    pass


class Mixer(Part):
    # True for a part whose ``forward`` takes the two optional arguments of norm folding:
    # ``xn`` may be a ``NormedInput`` whenever ``takes_normed_input(num_tokens)`` holds, and
    # ``then_norm=NormRequest`` asks its last product to prepare the next norm; it returns
    # the ``NormedInput`` it made or ``None``.  A part that leaves this False is called as
    # ``forward(xn, residual, step, cache)`` with a plain tensor, and the norms around it
    # run their own kernels.
    folds_norms: bool = False

    def takes_normed_input(self, num_tokens: int) -> bool:
        return False

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    folds_norms: bool = False     # as for Mixer; ``forward(xn, residual, step, then_norm=None)``

    def takes_normed_input(self, num_tokens: int) -> bool:
        return False

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step) -> None:
        raise NotImplementedError


class Block(Part):
    # True for a block whose ``forward`` takes ``pending`` and ``next_norm``; a block that
    # leaves this False is called as ``forward(x, step, cache)``.
    folds_norms: bool = False

    def forward(self, x: torch.Tensor, step, cache, pending=None, next_norm=None):
        """Updates the residual x in place.  ``pending``: the block's first norm of x,
        started by the previous block's last product (only given if ``first_norm_request``
        returned a request).  ``next_norm``: what the next block's first norm needs;
        returns the ``NormedInput`` made for it, or ``None``."""
        raise NotImplementedError

    def first_norm_request(self, num_tokens: int) -> Optional[NormRequest]:
        """What a product in front of this block needs to start the block's first norm,
        if the block can take it that way in a step of ``num_tokens`` tokens."""
        return None
