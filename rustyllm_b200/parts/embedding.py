"""Token embedding and output head.

SimonWaldherr/RustyLLM: ``x = token_embd.row(token)`` (src/model.rs:7193, no scaling) and
``logits = output . rms_norm(x)`` (src/model.rs:7351-7357); an absent output matrix
is the embedding matrix (tied, src/model.rs:3654-3667) - here the head then shares
the embedding's storage instead of cloning it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..config.spec import ParamSource, ParamSpec
from .base import Part, Runtime
from .linear import OUT_F32, linear
from .registry import register


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str):
        self.runtime = runtime
        self.V, self.d, self.name = vocab_size, hidden_size, name
        self.weight: Optional[torch.Tensor] = None
        self.bad_token = torch.zeros(1, dtype=torch.int32, device=runtime.device)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((ParamSource(self.name, (self.V, self.d)),), role="table")}

    def forward(self, step) -> torch.Tensor:
        """The step's tokens (``step.tokens``, int32 [M]) -> float32 residual [M, d].  An embedding
        part is handed the whole step, so that one which also needs the tokens' positions (a
        learned absolute position table) finds them in ``step.positions``."""
        tokens = step.tokens
        x = torch.empty((tokens.numel(), self.d), dtype=torch.float32, device=tokens.device)
        K.embedding(self.weight, tokens, x, self.bad_token)
        return x


@register("head", "lm_head")
class LMHead(Part):
    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str,
                 tied_to: Optional[str] = None):
        self.runtime = runtime
        self.V, self.d, self.name, self.tied_to = vocab_size, hidden_size, name, tied_to
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((ParamSource(self.name, (self.V, self.d)),), role="table",
                                    alias_of=self.tied_to)}

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        """xn: [W, d] compute dtype -> float32 logits [W, V]."""
        logits = torch.empty((xn.shape[0], self.V), dtype=torch.float32, device=xn.device)
        linear(xn, self.weight, logits, OUT_F32)
        return logits
