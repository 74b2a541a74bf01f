"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, in 32-bit.

SimonWaldherr/RustyLLM src/model.rs:5429-5437 (``rms_norm_into``): no mean subtraction, no
bias, the weight used as it is (no ``1 + w``).  Used before the mixer, before the
feed-forward and before the head (src/model.rs:7205, 7321, 7351).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..config.spec import ParamSource, ParamSpec
from .base import Norm, NormRequest, Runtime
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, runtime: Runtime, size: int, eps: float, name: str):
        self.runtime = runtime
        self.size = size
        self.eps = float(eps)
        self.name = name
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((ParamSource(self.name, (self.size,)),), role="vector", init="ones")}

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        K.rmsnorm(x, self.weight, out, self.eps, rows)
        return out

    def request(self) -> Optional[NormRequest]:
        return NormRequest(self.weight, self.eps) if self.weight is not None else None
