"""Sampler options and the host random generator, with the reference's names.

SimonWaldherr/RustyLLM src/sampling.rs:30-52 (``SamplerConfig``) and 4-27 (``Rng``).  Meanings are
the reference's; the defaults of the filters are neutral here (top_k 0, top_p 1,
min_p 0, repeat_penalty 1) so that "temperature T" alone means plain softmax
sampling - ``SamplerConfig.reference_defaults()`` gives the reference's values
(temperature 0.7, top_p 0.9, top_k 40, min_p 0, repeat_penalty 1.1).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

RECENT_TOKEN_LIMIT = 64   # window of the repeat penalty, src/runtime.rs:493
MAX_TOP_K = 1024          # the device's top-k kernel sorts its candidates in shared memory


@dataclass
class SamplerConfig:
    temperature: float = 0.7     # < 1e-6: greedy (after the repeat penalty)
    top_p: float = 1.0           # (0, 1]; keep the head whose weight first exceeds top_p * sum
    top_k: int = 0               # active iff 0 < k < vocab; 1 = greedy
    min_p: float = 0.0           # [0, 1); drop tokens below min_p * (weight of the top token)
    repeat_penalty: float = 1.0  # > 0; 1 = off; l > 0 -> l / p, else l * p, per recent occurrence

    @classmethod
    def reference_defaults(cls) -> "SamplerConfig":
        return cls(temperature=0.7, top_p=0.9, top_k=40, min_p=0.0, repeat_penalty=1.1)

    @classmethod
    def greedy(cls) -> "SamplerConfig":
        return cls(temperature=0.0)

    def validate(self) -> None:
        """Ranges and messages of ``GenerationOptions::validate`` (src/runtime.rs:351-368)."""
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError("temperature must be a finite number >= 0.")
        if not math.isfinite(self.top_p) or self.top_p <= 0.0 or self.top_p > 1.0:
            raise ValueError("top_p must be in the range (0, 1].")
        if not math.isfinite(self.repeat_penalty) or self.repeat_penalty <= 0.0:
            raise ValueError("repeat_penalty must be a finite number > 0.")
        if not math.isfinite(self.min_p) or self.min_p < 0.0 or self.min_p >= 1.0:
            raise ValueError("min_p must be in the range [0, 1).")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0.")
        if self.top_k > MAX_TOP_K and not self.is_greedy:
            # the reference takes any 0 < top_k < vocabulary (src/sampling.rs:87); here the candidate
            # set is sorted on the device in shared memory, which bounds it.  Said before a generation
            # starts rather than after its prompt step has run.
            raise ValueError(f"top_k must be at most {MAX_TOP_K} (or 0 for no top-k filter), got {self.top_k}.")

    @property
    def is_greedy(self) -> bool:
        return self.temperature < 1e-6 or self.top_k == 1

    @property
    def needs_candidates(self) -> bool:
        """Whether a sorted candidate set (top-k or top-p) is needed."""
        return not self.is_greedy and (self.top_k > 1 or self.top_p < 1.0)


class Rng:
    """xorshift64 (13, 7, 17); seed 0 means 0xDEADBEEFCAFE1337;
    ``next_f32`` = (state >> 40) / 2^24, uniform in [0, 1).  src/sampling.rs:4-27."""

    _MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = 0xDEADBEEFCAFE1337 if seed == 0 else (seed & self._MASK)

    def next_f32(self) -> float:
        s = self.state
        s ^= (s << 13) & self._MASK
        s ^= s >> 7
        s ^= (s << 17) & self._MASK
        self.state = s
        return (s >> 40) / float(1 << 24)
