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

    folds_norms = True

    def first_norm_request(self, num_tokens: int):
        if getattr(self.mixer, "folds_norms", False) and self.mixer.takes_normed_input(num_tokens):
            return self.mixer_norm.request()
        return None

    def forward(self, x: torch.Tensor, step, cache, pending=None, next_norm=None):
        dt = self.runtime.compute_dtype
        # A norm between two matrix products can ride in their epilogues (the product in
        # front starts it, the one behind finishes it) where both parts can; otherwise the
        # norm part runs its own kernel.
        xn = pending if pending is not None else self.mixer_norm.forward(x, dt)
        started = None
        if getattr(self.mixer, "folds_norms", False):
            want = None
            if getattr(self.feed_forward, "folds_norms", False) and self.feed_forward.takes_normed_input(x.shape[0]):
                want = self.feed_forward_norm.request()
            started = self.mixer.forward(xn, x, step, cache, then_norm=want)
        else:
            self.mixer.forward(xn, x, step, cache)
        xn2 = started if started is not None else self.feed_forward_norm.forward(x, dt)
        if getattr(self.feed_forward, "folds_norms", False):
            return self.feed_forward.forward(xn2, x, step, then_norm=next_norm)
        self.feed_forward.forward(xn2, x, step)
        return None
