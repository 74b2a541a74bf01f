"""Rotary position encoding: the table of inverse frequencies and how pairs are
formed.  The rotation itself runs inside the mixer's fused rope + cache-write
kernel (csrc/rope_cache.cu).

SimonWaldherr/RustyLLM: ``inv[i] = 1 / (theta^(2i/hd) * factor[i])``
(``build_rope_inv_freq_with_factors``, src/model.rs:3035-3057); interleaved pairs
(2i, 2i+1) in ``apply_rope_qk`` (5562-5603), half-split pairs (i, i + hd/2) in
``apply_rope_qk_neox`` (5606-5647).  The reference's standard path passes no
per-pair factors (src/model.rs:3108); the "llama3" scaling below produces them:
with wavelen = 2*pi/inv, pairs with wavelen < orig/high_freq_factor keep their
frequency, pairs with wavelen > orig/low_freq_factor are divided by ``factor``, and
pairs between are blended linearly in (orig/wavelen - low)/(high - low).
The table is computed once on the host in float64 and rounded to float32.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, Runtime
from .registry import register_position


def rope_inverse_frequencies(theta: float, rotary_dim: int, scaling: Optional[dict]) -> torch.Tensor:
    half = rotary_dim // 2
    inv = [1.0 / (theta ** ((2 * i) / rotary_dim)) for i in range(half)]
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            low_wavelen, high_wavelen = orig / low, orig / high
            for i in range(half):
                wavelen = 2.0 * math.pi / inv[i]
                if wavelen < high_wavelen:
                    continue
                if wavelen > low_wavelen:
                    inv[i] /= factor
                else:
                    smooth = (orig / wavelen - low) / (high - low)
                    inv[i] = (1.0 - smooth) * inv[i] / factor + smooth * inv[i]
        elif kind not in (None, "default"):
            raise ValueError(f"unknown rope scaling {kind!r}")
    return torch.tensor(inv, dtype=torch.float64).to(torch.float32)


@register_position("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, runtime: Runtime, head_dim: int, rotary_dim: int, theta: float,
                 scaling: Optional[dict] = None, pairing: str = "half"):
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing must be 'half' or 'interleaved', got {pairing!r}")
        if rotary_dim % 2 or not (0 <= rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.interleaved = pairing == "interleaved"
        inv = rope_inverse_frequencies(theta, rotary_dim, scaling) if rotary_dim else torch.zeros(1)
        self.inv_freq = inv.to(runtime.device)


@register_position("none")
class NoPositionEncoding(RotaryEmbedding):
    """No position encoding: a rotary part of width 0."""

    def __init__(self, runtime: Runtime, head_dim: int):
        super().__init__(runtime, head_dim=head_dim, rotary_dim=0, theta=1.0)
