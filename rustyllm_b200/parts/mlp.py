"""Gated feed-forward (SwiGLU): x += Wdown (silu(Wgate xn) * (Wup xn)).

SimonWaldherr/RustyLLM src/model.rs:7321-7347 with the activation of src/simd.rs:2403-2408
(``g / (1 + exp(-g)) * u``).  Wgate and Wup are one matrix [2I x d] so that one
product serves both (the reference reads a fused ``ffn_up`` of 2I rows, gate rows
first, src/model.rs:3933-3967).  In a bf16 run the rows are interleaved (gate_0, up_0,
gate_1, up_1, ...): a gate and its up value then sit in neighbouring lanes of the
tensor-core product's epilogue, which applies the activation and writes the
[M x I] product directly - the [M x 2I] intermediate is never stored.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import kernels as K
from ..config.spec import ParamSource, ParamSpec
from .base import FeedForward, NormedInput, Runtime
from .linear import OUT_ADD_F32, OUT_SAME, can_fold_norms, linear
from .registry import register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, names: Dict[str, str],
                 activation: str = "silu", bias: bool = False):
        if activation != "silu":
            raise ValueError(f"activation {activation!r} is not supported; known: 'silu'")
        self.runtime = runtime
        self.d, self.I = hidden_size, intermediate_size
        self.names = names
        self.bias = bias
        self.interleaved = runtime.compute_dtype == torch.bfloat16
        self.wgu = self.wdown = self.bgu = self.bdown = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, I, n = self.d, self.I, self.names
        layout = "interleave" if self.interleaved else "concat"
        specs = {
            "wgu": ParamSpec((ParamSource(n["gate"] + ".weight", (I, d)),
                              ParamSource(n["up"] + ".weight", (I, d))), layout=layout),
            "wdown": ParamSpec((ParamSource(n["down"] + ".weight", (d, I)),)),
        }
        if self.bias:
            specs["bgu"] = ParamSpec((ParamSource(n["gate"] + ".bias", (I,)),
                                      ParamSource(n["up"] + ".bias", (I,))), role="vector", layout=layout)
            specs["bdown"] = ParamSpec((ParamSource(n["down"] + ".bias", (d,)),), role="vector")
        return specs

    folds_norms = True

    def takes_normed_input(self, num_tokens: int) -> bool:
        return self.interleaved and can_fold_norms(self.wgu, self.runtime.compute_dtype, num_tokens)

    def forward(self, xn, residual: torch.Tensor, step, then_norm=None):
        M = xn.shape[0]
        h = torch.empty((M, self.I), dtype=xn.dtype, device=xn.device)
        # The activation runs in the product's epilogue: with few tokens the kernel streams
        # weights and the epilogue is idle time anyway; with many, the persistent kernel drains
        # one accumulator while the tensor cores fill the other.
        x = xn.weighted if isinstance(xn, NormedInput) else xn
        if self.interleaved and self.wgu.dtype == torch.bfloat16 and K.gemm_tc_supported(x, self.wgu, None):
            kw = dict(row_sumsq=xn.sumsq, row_eps=xn.eps) if isinstance(xn, NormedInput) else {}
            K.gemm_tc(x, self.wgu, h, K.OUT_SWIGLU, self.bgu, **kw)
        else:
            gu = torch.empty((M, 2 * self.I), dtype=xn.dtype, device=xn.device)
            linear(xn, self.wgu, gu, OUT_SAME, self.bgu)
            K.swiglu(gu, h, interleaved=self.interleaved)
        return linear(h, self.wdown, residual, OUT_ADD_F32, self.bdown, then_norm=then_norm)
