"""Host-to-device copies of a step's small inputs through pinned memory."""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

_NP = {torch.int32: np.int32, torch.float32: np.float32}


class PinnedStaging:
    """A ring of pinned host buffers.  ``upload`` copies a host array into the next
    buffer and from there to the device without blocking; a buffer is reused only
    after the copy that read it has finished, so the host may run ahead of the
    device without changing what an earlier step reads."""

    def __init__(self, device: torch.device, dtype: torch.dtype = torch.int32, depth: int = 4):
        self.device = device
        self.dtype = dtype
        self.depth = depth
        self.bufs: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.views: List[Optional[np.ndarray]] = [None] * depth
        self.i = 0
        self.bytes = 0

    def upload(self, host: np.ndarray) -> torch.Tensor:
        flat = host.reshape(-1)
        n = flat.shape[0]
        k = self.i
        self.i = (self.i + 1) % self.depth
        if self.events[k] is not None:
            self.events[k].synchronize()
        else:
            self.events[k] = torch.cuda.Event()
        if self.bufs[k] is None or self.bufs[k].numel() < n:
            self.bufs[k] = torch.empty(max(n, 1024), dtype=self.dtype, pin_memory=True)
            self.views[k] = self.bufs[k].numpy()
        self.views[k][:n] = flat          # converts to the buffer's type if need be
        dev = self.bufs[k][:n].to(self.device, non_blocking=True)
        self.events[k].record()
        self.bytes += n * self.views[k].itemsize
        return dev.view(host.shape)
