"""Sampling on the device: rows of float32 logits in, one token id per row out.

Order of operations of ``sample_with_scratch`` (SimonWaldherr/RustyLLM src/sampling.rs:66-212):
repeat penalty first (also when greedy), then greedy argmax if the temperature is
below 1e-6, else the candidate path (top-k / top-p) or the full-vocabulary softmax
draw with the optional min-p cut.  Each row has its own options, its own uniform
number (from that sequence's host generator) and its own recent-token window, so a
sequence samples the same tokens alone or in any batch.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels as K
from ..staging import PinnedStaging
from .config import RECENT_TOKEN_LIMIT, Rng, SamplerConfig


class SequenceSamplingState:
    """Per-sequence sampler state: options, generator, recent-token window."""

    def __init__(self, config: SamplerConfig, seed: int, prompt: Sequence[int]):
        config.validate()
        self.config = config
        self.rng = Rng(seed)
        # src/runtime.rs:493-521: the last 64 tokens of prompt + output
        self.recent: List[int] = list(prompt[-RECENT_TOKEN_LIMIT:])

    def push(self, token: int) -> None:
        self.recent.append(token)
        if len(self.recent) > RECENT_TOKEN_LIMIT:
            del self.recent[0]


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device
        self._floats = PinnedStaging(device, torch.float32) if device.type == "cuda" else None
        self._ints = PinnedStaging(device, torch.int32) if device.type == "cuda" else None
        self._host_ids: Optional[torch.Tensor] = None      # pinned: the sampled ids come back through it
        self._ids_copied = torch.cuda.Event() if device.type == "cuda" else None

    def _copy_to_host(self, ids: torch.Tensor) -> None:
        n = ids.numel()
        if self._host_ids is None or self._host_ids.numel() < n:
            self._host_ids = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=True)
        self._host_ids[:n].copy_(ids, non_blocking=True)
        self._ids_copied.record()

    def _to_host(self, ids: torch.Tensor) -> List[int]:
        """The sampled ids on the host (waits for the kernels that produced them)."""
        if self._ids_copied is None:
            return ids.tolist()
        self._copy_to_host(ids)
        self._ids_copied.synchronize()
        return self._host_ids[:ids.numel()].tolist()

    @property
    def h2d_bytes(self) -> int:
        return (self._floats.bytes + self._ints.bytes) if self._floats else 0

    def sample(self, logits: torch.Tensor, states: Sequence[SequenceSamplingState]) -> List[int]:
        """logits: float32 [B, V] on the device (modified in place by the repeat
        penalty).  Draws one uniform from the generator of every row that is not
        greedy.  Returns host token ids."""
        return self._to_host(self._sample_on_device(logits, states))

    def sample_begin(self, logits: torch.Tensor, states: Sequence[SequenceSamplingState]) -> "PendingIds":
        """``sample`` in two halves: the kernels and the copy to the host are queued here and
        the ids are waited for in ``PendingIds.wait``, so that the caller can queue the next
        step, fed from ``PendingIds.device_ids``, in between.  One pending result at a time."""
        ids = self._sample_on_device(logits, states)
        if self._ids_copied is not None:
            self._copy_to_host(ids)
        return PendingIds(self, ids)

    def _sample_on_device(self, logits: torch.Tensor, states: Sequence[SequenceSamplingState]) -> torch.Tensor:
        B, V = logits.shape
        assert B == len(states)
        dev = logits.device
        out = torch.empty(B, dtype=torch.int32, device=dev)

        penalties = {s.config.repeat_penalty for s in states}
        if penalties != {1.0}:
            recent = np.zeros((B, RECENT_TOKEN_LIMIT), dtype=np.int32)
            lens = np.zeros(B, dtype=np.int32)
            for b, s in enumerate(states):
                lens[b] = len(s.recent)
                recent[b, :lens[b]] = s.recent
            recent_d = self._ints.upload(recent)
            lens_d = self._ints.upload(lens)
            if len(penalties) == 1:
                K.repeat_penalty(logits, recent_d, lens_d, next(iter(penalties)))
            else:
                for b, s in enumerate(states):   # rows with different penalties: one launch each
                    if s.config.repeat_penalty != 1.0:
                        K.repeat_penalty(logits[b:b + 1], recent_d[b:b + 1], lens_d[b:b + 1],
                                         s.config.repeat_penalty)

        if all(s.config.is_greedy for s in states):
            K.argmax(logits, out)
            return out

        def takes_top_k(c: SamplerConfig) -> bool:
            return not c.is_greedy and 1 < c.top_k < V
        topk = [b for b, s in enumerate(states) if takes_top_k(s.config)]
        topp = [b for b, s in enumerate(states)
                if not s.config.is_greedy and not takes_top_k(s.config) and s.config.top_p < 1.0]
        # one float upload: temperature | uniform | min_p | top-p of the top-k rows | top-p of the top-p rows
        nk, np_ = len(topk), len(topp)
        f = np.zeros(3 * B + nk + np_, dtype=np.float32)
        for b, s in enumerate(states):
            c = s.config
            greedy = c.is_greedy
            f[b] = 0.0 if greedy else c.temperature
            f[B + b] = 0.0 if greedy else s.rng.next_f32()
            f[2 * B + b] = c.min_p
        f[3 * B:3 * B + nk] = [states[b].config.top_p for b in topk]
        f[3 * B + nk:] = [states[b].config.top_p for b in topp]
        fd = self._floats.upload(f)
        temperature, uniform, min_p = fd[:B], fd[B:2 * B], fd[2 * B:3 * B]
        # rows without a candidate set (greedy rows among them) are answered by the softmax kernel,
        # which takes every row of the batch (the others' answers are overwritten below); it is
        # left out when every row has a candidate set
        if nk + np_ < B:
            K.sample_temperature(logits, temperature, uniform, out, min_p if f[2 * B:3 * B].any() else None)
        if topk or topp:
            # one int upload from pinned memory: rows of the top-k path | their k | rows of the top-p path
            idx = self._ints.upload(np.asarray(topk + [states[b].config.top_k for b in topk] + topp, dtype=np.int32))
            K.sample_candidates(logits, temperature, uniform, min_p, out,
                                idx[:nk] if nk else None, idx[nk:2 * nk] if nk else None,
                                fd[3 * B:3 * B + nk] if nk else None,
                                idx[2 * nk:] if np_ else None, fd[3 * B + nk:] if np_ else None)
        return out


class PendingIds:
    """Token ids that a sampler has queued: on the device now, on the host after ``wait``."""

    def __init__(self, sampler: Sampler, device_ids: torch.Tensor):
        self._sampler = sampler
        self.device_ids = device_ids      # int32 [B]

    def wait(self) -> List[int]:
        s = self._sampler
        if s._ids_copied is None:
            return self.device_ids.tolist()
        s._ids_copied.synchronize()
        return s._host_ids[:self.device_ids.numel()].tolist()
