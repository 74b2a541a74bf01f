"""Grouped-query attention over the paged cache: the mixer of the Llama decoder.

Per layer, in the reference's order (SimonWaldherr/RustyLLM src/model.rs:7207-7318):
q = Wq xn, k = Wk xn, v = Wv xn (+ biases if the tensors exist); rotary encoding of
q and k; K[pos] = k, V[pos] = v; per query head h with KV head g = h / (H/G):
softmax over t <= pos of (q_h . K[t, g]) / sqrt(head_dim), times V; then
x += Wo attn.  Here Wq, Wk, Wv are one matrix [(H + 2G) hd x d] so that one product
serves all three, rotation and cache write are one kernel, and all tokens of the
step (several sequences, prompt or single tokens) run together.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import kernels as K
from ..cache.sequence_cache import KVNeed
from ..config.spec import ParamSource, ParamSpec, PartSpec
from .base import Mixer, NormedInput, Runtime
from .linear import OUT_ADD_F32, OUT_SAME, can_fold_norms, linear
from .registry import build_part, register_mixer


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, position: PartSpec, names: Dict[str, str], bias: bool = False,
                 window: Optional[int] = None, value_dim: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} KV heads")
        if head_dim % 2 or not (0 < head_dim <= 256):
            raise ValueError(f"head_dim {head_dim} must be even and at most 256")
        if window is not None and window <= 0:
            raise ValueError("window must be > 0 or None")
        vd = head_dim if value_dim is None else value_dim      # the reference keeps value_dim apart, src/model.rs:33, 67-69
        if vd % 2 or not (0 < vd <= 256):
            raise ValueError(f"value_dim {vd} must be even and at most 256")
        self.vd = vd
        self.runtime = runtime
        self.d, self.H, self.G, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.bias = bias
        self.window = window
        self.names = names
        self.scale = 1.0 / math.sqrt(head_dim)     # src/model.rs:7239
        self.position = build_part("position", position, runtime)
        self.wqkv = self.wo = self.bqkv = self.bo = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, H, G, hd, vd, n = self.d, self.H, self.G, self.hd, self.vd, self.names
        specs = {
            "wqkv": ParamSpec((ParamSource(n["q"] + ".weight", (H * hd, d)),
                               ParamSource(n["k"] + ".weight", (G * hd, d)),
                               ParamSource(n["v"] + ".weight", (G * vd, d)))),
            "wo": ParamSpec((ParamSource(n["o"] + ".weight", (d, H * vd)),)),
        }
        if self.bias:
            specs["bqkv"] = ParamSpec((ParamSource(n["q"] + ".bias", (H * hd,)),
                                       ParamSource(n["k"] + ".bias", (G * hd,)),
                                       ParamSource(n["v"] + ".bias", (G * vd,))), role="vector")
            specs["bo"] = ParamSpec((ParamSource(n["o"] + ".bias", (d,)),), role="vector")
        return specs

    def kv_need(self) -> KVNeed:
        return KVNeed(self.G, self.hd, self.window, None if self.vd == self.hd else self.vd)

    folds_norms = True

    def takes_normed_input(self, num_tokens: int) -> bool:
        return can_fold_norms(self.wqkv, self.runtime.compute_dtype, num_tokens)

    def forward(self, xn, residual: torch.Tensor, step, cache, then_norm=None):
        H, G, hd, vd = self.H, self.G, self.hd, self.vd
        M = xn.shape[0]
        dt = xn.dtype
        qkv = torch.empty((M, (H + G) * hd + G * vd), dtype=dt, device=xn.device)
        group, layer = cache.kv_group, cache.kv_layer
        k_pool, v_pool = group.k_pool(layer), group.v_pool(layer)
        pos = self.position
        x = xn.weighted if isinstance(xn, NormedInput) else xn
        if (dt == torch.bfloat16 and vd == hd and self.wqkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16
                and K.gemm_tc_qkv_rope_supported(x, self.wqkv, H, G, hd, pos.rotary_dim)):
            # few tokens: rotation and cache write ride in the product's epilogue
            kw = dict(row_sumsq=xn.sumsq, row_eps=xn.eps) if isinstance(xn, NormedInput) else {}
            K.gemm_tc_qkv_rope(x, self.wqkv, qkv, self.bqkv, step.positions, step.slot_of_token, group.page_table,
                               pos.inv_freq, pos.interleaved, H, G,
                               k_pool if cache.writes else None, v_pool if cache.writes else None, **kw)
        else:
            linear(xn, self.wqkv, qkv, OUT_SAME, self.bqkv)
            K.rope_kv_write(qkv, step.positions, step.slot_of_token, group.page_table, pos.inv_freq, H, G, hd,
                            pos.rotary_dim, pos.interleaved,
                            k_pool if cache.writes else None, v_pool if cache.writes else None, value_dim=vd)
        attn = torch.empty((M, H * vd), dtype=dt, device=xn.device)
        K.attention(qkv, k_pool, v_pool, group.page_table, step, attn, H, G, hd, self.scale,
                    self.window or 0, value_dim=vd)
        return linear(attn, self.wo, residual, OUT_ADD_F32, self.bo, then_norm=then_norm)
