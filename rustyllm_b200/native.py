"""The native executor of a decoder step (csrc/decoder_forward.cu) from Python: the model's
description is handed over once as plain structs, and a step is then one call that launches
embedding and all layers (another for final norm and head) without the interpreter between
kernels.  It knows the parts the Llama decoder is made of; ``eligible`` says whether a model
(with its cache) consists of those and of nothing else - any other model runs through its
Python parts, which is the same chain of kernels issued more slowly.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import kernels as K

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


class RlLinear(ctypes.Structure):
    _fields_ = [("w", _vp), ("bias", _vp), ("n", _i), ("k", _i)]


class RlNormW(ctypes.Structure):
    _fields_ = [("w", _vp), ("eps", _f)]


class RlLayerDesc(ctypes.Structure):
    _fields_ = [("norm1", RlNormW), ("norm2", RlNormW), ("qkv", RlLinear), ("o", RlLinear), ("gate_up", RlLinear),
                ("down", RlLinear), ("num_heads", _i), ("num_kv_heads", _i), ("head_dim", _i), ("value_dim", _i),
                ("rotary_dim", _i), ("interleaved_rope", _i), ("window", _i), ("scale", _f), ("inv_freq", _vp),
                ("intermediate", _i)]


class RlRunDesc(ctypes.Structure):
    _fields_ = [("layer", _i), ("k_pool", _vp), ("v_pool", _vp), ("page_table", _vp), ("max_pages", _i),
                ("num_pages", _i), ("writes", _i)]


class RlModelDesc(ctypes.Structure):
    _fields_ = [("hidden", _i), ("vocab", _i), ("num_layers", _i), ("num_runs", _i), ("layers", _vp), ("runs", _vp),
                ("embed", _vp), ("final_norm", RlNormW), ("head", RlLinear)]


class RlStepDesc(ctypes.Structure):
    _fields_ = [("M", _i), ("B", _i), ("is_decode", _i), ("tokens", _vp), ("positions", _vp), ("slot_of_token", _vp),
                ("cu_seqlens", _vp), ("seq_slots", _vp), ("kv_lens", _vp), ("tiles_tc", _i), ("tiles_mma", _i),
                ("tile_order", _vp), ("long_context", _i), ("length_spread", _i)]


def _matrix_ok(w: Optional[torch.Tensor]) -> bool:
    return (w is not None and w.dtype == torch.bfloat16 and w.is_cuda and w.is_contiguous() and w.dim() == 2
            and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0)


def _vector_ok(v: Optional[torch.Tensor]) -> bool:
    return v is None or (v.dtype == torch.float32 and v.is_cuda and v.is_contiguous())


def eligible(model, cache) -> bool:
    """Whether every part of the model is one the native executor runs: pre-norm blocks of
    grouped-query attention with a rotary (or no) position encoding and a gated feed-forward,
    RMS norms, token embedding and head, all matrices bfloat16 and addressable by TMA, on a
    bfloat16 cache."""
    from .parts.attention import GQAttention
    from .parts.block import PreNormBlock
    from .parts.embedding import LMHead, TokenEmbedding
    from .parts.mlp import GatedMLP
    from .parts.norm import RMSNorm
    from .parts.rope import RotaryEmbedding
    if model.runtime.compute_dtype != torch.bfloat16 or model.runtime.device.type != "cuda" or cache.dtype != torch.bfloat16:
        return False
    if type(model.embedding) is not TokenEmbedding or type(model.head) is not LMHead or type(model.final_norm) is not RMSNorm:
        return False
    if not (_matrix_ok(model.embedding.weight) and _matrix_ok(model.head.weight) and _vector_ok(model.final_norm.weight)):
        return False
    for b in model.blocks:
        if type(b) is not PreNormBlock or type(b.mixer) is not GQAttention or type(b.feed_forward) is not GatedMLP:
            return False
        if type(b.mixer_norm) is not RMSNorm or type(b.feed_forward_norm) is not RMSNorm or not isinstance(b.mixer.position, RotaryEmbedding):
            return False
        a, f = b.mixer, b.feed_forward
        if not (f.interleaved and _matrix_ok(a.wqkv) and _matrix_ok(a.wo) and _matrix_ok(f.wgu) and _matrix_ok(f.wdown)):
            return False
        if not all(_vector_ok(v) for v in (a.bqkv, a.bo, f.bgu, f.bdown, b.mixer_norm.weight, b.feed_forward_norm.weight)):
            return False
    return True


class NativeDecoder:
    """The structs of one model on one cache, kept alive together with what they point to."""

    def __init__(self, model, cache):
        self.model, self.cache = model, cache
        self.lib = K.library()
        lib = self.lib
        lib.rl_decoder_workspace_bytes.restype = ctypes.c_longlong
        lib.rl_decoder_workspace_bytes.argtypes = [_vp, _i, _i]
        lib.rl_decoder_forward.restype = _i
        lib.rl_decoder_forward.argtypes = [_vp, _vp, _vp, _vp, ctypes.c_longlong, _vp, _vp, _vp]
        lib.rl_decoder_logits.restype = _i
        lib.rl_decoder_logits.argtypes = [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp]
        lib.rl_decoder_last_launches.restype = _i
        lib.rl_decoder_last_launches.argtypes = []
        ptr = lambda t: None if t is None else t.data_ptr()
        lin = lambda w, b: RlLinear(w=w.data_ptr(), bias=ptr(b), n=w.shape[0], k=w.shape[1])
        blocks = model.blocks
        self.layers = (RlLayerDesc * len(blocks))()
        for i, b in enumerate(blocks):
            a, f, pos = b.mixer, b.feed_forward, b.mixer.position
            self.layers[i] = RlLayerDesc(
                norm1=RlNormW(b.mixer_norm.weight.data_ptr(), b.mixer_norm.eps),
                norm2=RlNormW(b.feed_forward_norm.weight.data_ptr(), b.feed_forward_norm.eps),
                qkv=lin(a.wqkv, a.bqkv), o=lin(a.wo, a.bo), gate_up=lin(f.wgu, f.bgu), down=lin(f.wdown, f.bdown),
                num_heads=a.H, num_kv_heads=a.G, head_dim=a.hd, value_dim=a.vd, rotary_dim=pos.rotary_dim,
                interleaved_rope=int(pos.interleaved), window=a.window or 0, scale=a.scale, inv_freq=pos.inv_freq.data_ptr(),
                intermediate=f.I)
        schedule = model.spec.schedule
        self.runs = (RlRunDesc * len(schedule))()
        for r, li in enumerate(schedule):
            entry, writes = model.run_entry[r]
            group, layer = cache.kv_entry(entry)
            self.runs[r] = RlRunDesc(layer=li, k_pool=group.k_pool(layer).data_ptr(), v_pool=group.v_pool(layer).data_ptr(),
                                     page_table=group.page_table.data_ptr(), max_pages=group.page_table.shape[1],
                                     num_pages=group.num_pages, writes=int(writes))
        self.desc = RlModelDesc(
            hidden=model.spec.hidden_size, vocab=model.spec.vocab_size, num_layers=len(blocks), num_runs=len(schedule),
            layers=ctypes.addressof(self.layers), runs=ctypes.addressof(self.runs), embed=model.embedding.weight.data_ptr(),
            final_norm=RlNormW(model.final_norm.weight.data_ptr(), model.final_norm.eps),
            head=lin(model.head.weight, None))
        self._desc_ptr = ctypes.addressof(self.desc)
        self._err = K._tc_error_word(model.runtime.device)
        self._tc_prefill = all(K.attention_prefill_tc_supported(torch.bfloat16, b.mixer.H, b.mixer.G, b.mixer.hd) for b in blocks)

    def forward(self, step) -> torch.Tensor:
        """Embedding and every scheduled layer for the step's tokens: the float32 residual [M, hidden]."""
        M, B = step.num_tokens, step.num_seqs
        dev = self.model.runtime.device
        x = torch.empty((M, self.desc.hidden), dtype=torch.float32, device=dev)
        nbytes = int(self.lib.rl_decoder_workspace_bytes(self._desc_ptr, M, B))
        work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        order = None
        if not step.is_decode and B > 1 and self._tc_prefill:      # the tcgen05 attention starts its heaviest tiles first
            order = step.derived.get("prefill_tile_order")
            if order is None:
                order = step.derived["prefill_tile_order"] = K.prefill_tile_order(step.q_lens, step.kv_lens_host, dev)
        sd = RlStepDesc(M=M, B=B, is_decode=int(step.is_decode), tokens=step.tokens.data_ptr(), positions=step.positions.data_ptr(),
                        slot_of_token=step.slot_of_token.data_ptr(), cu_seqlens=step.cu_seqlens.data_ptr(),
                        seq_slots=step.seq_slots.data_ptr(), kv_lens=step.kv_lens.data_ptr(),
                        tiles_tc=sum(-(-n // K.PREFILL_TC_QTILE) for n in step.q_lens),
                        tiles_mma=sum(-(-n // K.PREFILL_QTILE) for n in step.q_lens),
                        tile_order=None if order is None else order.data_ptr(), long_context=int(step.long_context),
                        length_spread=int(step.length_spread))
        rc = self.lib.rl_decoder_forward(self._desc_ptr, ctypes.addressof(sd), x.data_ptr(), work.data_ptr(), nbytes,
                                         self._err.data_ptr(), self.model.embedding.bad_token.data_ptr(), K._stream())
        K._check(rc, "rl_decoder_forward")
        K._count(int(self.lib.rl_decoder_last_launches()))
        return x

    def logits(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        W = rows.numel()
        dev = x.device
        xn = torch.empty((W, self.desc.hidden), dtype=torch.bfloat16, device=dev)
        out = torch.empty((W, self.desc.vocab), dtype=torch.float32, device=dev)
        rc = self.lib.rl_decoder_logits(self._desc_ptr, x.data_ptr(), rows.data_ptr(), W, xn.data_ptr(), out.data_ptr(),
                                        self._err.data_ptr(), K._stream())
        K._check(rc, "rl_decoder_logits")
        K._count(int(self.lib.rl_decoder_last_launches()))
        return out
