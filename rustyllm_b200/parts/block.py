"""Arrangement of a layer's parts.  "pre_norm" is the Llama layer
(SimonWaldherr/RustyLLM src/model.rs:7201-7348): x += mixer(norm(x)); x += ff(norm(x)).
"""
from __future__ import annotations

import torch

from .base import Block, FeedForward, Mixer, Norm, Runtime
from .registry import register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, runtime: Runtime, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward,
                 feed_forward_norm: Norm):
        self.runtime = runtime
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def sub_parts(self):
        return {"mixer": self.mixer, "mixer_norm": self.mixer_norm,
                "feed_forward": self.feed_forward, "feed_forward_norm": self.feed_forward_norm}

    def forward(self, x: torch.Tensor, step, cache) -> None:
        dt = self.runtime.compute_dtype
        self.mixer.forward(self.mixer_norm.forward(x, dt), x, step, cache)
        self.feed_forward.forward(self.feed_forward_norm.forward(x, dt), x, step)
