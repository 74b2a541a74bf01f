"""A plain, slow implementation of the Llama dense decoder: whole sequences, no
cache, one function for each part, float64 on the CPU.

It shares no code with the package under test: it reads config.json and
model.safetensors itself and restates the reference's formulas, each function
citing where the reference (SimonWaldherr/RustyLLM, paths inside that project)
computes the same thing.  The reference is Rust and cannot be compiled or
imported in this environment (no cargo/rustc), so this file rests on the
formulas as read from its sources, plus the literal vectors of the reference's
own unit tests restated in tests/test_plain.py.

Two things the reference's standard path does not have are restated from the
architecture's definition instead and are marked "ours": the llama3 frequency
scaling and the half-split pairing used by checkpoints in safetensors layout
(the reference has the pairing itself, as ``apply_rope_qk_neox``).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Minimal reader: header length, JSON header, raw little-endian data."""
    dt = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
          "F64": torch.float64, "I32": torch.int32, "I64": torch.int64}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=dt[info["dtype"]])
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_model_dir(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: v.to(F64) for k, v in w.items()}


# --------------------------------------------------------------------------- parts
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/model.rs:5429-5437 ``rms_norm_into``: ss = sum(x^2)/n;
    y = x * 1/sqrt(ss + eps) * w.  No mean subtraction, weight as is."""
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(ss + eps)) * weight


def rope_inv_freq(theta: float, head_dim: int, scaling: Optional[dict]) -> torch.Tensor:
    """src/model.rs:3035-3057 ``build_rope_inv_freq_with_factors``:
    inv[i] = 1 / (theta^(2i/hd) * factor[i]).

    The per-pair divisor ``factor[i]`` is ours for rope_type "llama3" (the
    reference's standard path passes none, src/model.rs:3108): with
    wavelen = 2*pi/inv, pairs with wavelen < orig/high keep their frequency,
    pairs with wavelen > orig/low are divided by ``factor``, pairs between are
    blended linearly in (orig/wavelen - low)/(high - low)."""
    half = head_dim // 2
    inv = np.array([1.0 / (theta ** ((2 * i) / head_dim)) for i in range(half)], dtype=np.float64)
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        for i in range(half):
            wavelen = 2.0 * math.pi / inv[i]
            if wavelen < orig / high:
                pass
            elif wavelen > orig / low:
                inv[i] = inv[i] / factor
            else:
                s = (orig / wavelen - low) / (high - low)
                inv[i] = (1.0 - s) * inv[i] / factor + s * inv[i]
    # the reference keeps the table in f32 (Vec<f32>)
    return torch.from_numpy(inv.astype(np.float32))


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor):
    """src/model.rs:5575 / 5618: angle = pos as f32 * inv_freq[i] (an f32 product),
    then sin and cos of it."""
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
    ang = ang.to(F64)
    return torch.sin(ang), torch.cos(ang)


def apply_rope_half(x: torch.Tensor, sin: torch.Tensor, cos: torch.Tensor) -> torch.Tensor:
    """src/model.rs:5606-5647 ``apply_rope_qk_neox``: pair (i, i + hd/2);
    x0' = x0*cos - x1*sin, x1' = x0*sin + x1*cos.  x: [T, heads, hd]."""
    half = x.shape[-1] // 2
    x0, x1 = x[..., :half], x[..., half:]
    s, c = sin[:, None, :], cos[:, None, :]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def apply_rope_interleaved(x: torch.Tensor, sin: torch.Tensor, cos: torch.Tensor) -> torch.Tensor:
    """src/model.rs:5562-5603 ``apply_rope_qk``: pair (2i, 2i+1), same rotation."""
    x0, x1 = x[..., 0::2], x[..., 1::2]
    s, c = sin[:, None, :], cos[:, None, :]
    out = torch.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * s
    out[..., 1::2] = x0 * s + x1 * c
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: Optional[int] = None) -> torch.Tensor:
    """src/model.rs:7239-7294 with ``online_attention`` (5807-5869) and the grouping
    of ``online_attention_grouped`` (6034-6198): query head h uses KV head
    g = h / (H/G); score_t = (q_h . k_t,g) / sqrt(hd) for t <= pos (t >= pos+1-W
    under a window W, src/model.rs:7241-7243); softmax over t; out = sum p_t v_t,g.
    The streaming softmax of the reference equals the plain one computed here.
    q: [T, H, hd], k, v: [T, G, hd] -> [T, H, hd]."""
    T, H, hd = q.shape
    G = k.shape[1]
    m = H // G
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    t_idx = torch.arange(T)
    for lo in range(0, T, 1024):          # query rows in blocks, only to bound the score matrix's memory
        rows = t_idx[lo:lo + 1024]
        allowed = t_idx[None, :] <= rows[:, None]
        if window is not None and window > 0:
            allowed &= t_idx[None, :] >= (rows[:, None] + 1 - window)
        for h in range(H):
            g = h // m
            s = (q[lo:lo + 1024, h, :] @ k[:, g, :].T) * scale
            s = s.masked_fill(~allowed, float("-inf"))
            p = torch.softmax(s, dim=-1)
            out[lo:lo + 1024, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """src/simd.rs:2403-2408 ``silu_mul_scalar``: g / (1 + exp(-g)) * up."""
    return gate / (1.0 + torch.exp(-gate)) * up


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """src/model.rs:185-186 ``matvec_into``: out[r] = dot(W[r, :], x); bias added
    only if the tensor exists (``add_bias_if_present``, src/model.rs:5551-5559)."""
    y = x @ w.T
    return y if b is None else y + b


# --------------------------------------------------------------------------- model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
            round_fn: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
            pairing: str = "half", return_hidden: bool = False) -> torch.Tensor:
    """Logits at every position of one whole sequence: [T, V].

    Order of operations of ``forward_into``, src/model.rs:7177-7358, applied to all
    positions at once (the reference runs them one by one against its cache):
    embedding row (7193) -> per layer {rms_norm (7205), q/k/v (7207-7217), rope
    (7230), attention (7239-7294), o-proj + residual (7315-7318), rms_norm (7321),
    gate/up, silu*up, down + residual (7332-7347)} -> final rms_norm and
    output matrix (7351-7357); a missing output matrix is the embedding
    (3654-3667).

    ``round_fn``, if given, is applied where a reduced-precision engine stores
    activations (normed input, q/k/v, attention output, the SwiGLU product); the
    residual sum itself is never rounded.
    """
    r = round_fn if round_fn is not None else (lambda t: t)
    H = cfg["num_attention_heads"]
    G = cfg.get("num_key_value_heads") or H
    d = cfg["hidden_size"]
    hd = cfg.get("head_dim") or d // H
    eps = cfg.get("rms_norm_eps", 1e-5)
    theta = cfg.get("rope_theta", 10000.0)
    scaling = cfg.get("rope_scaling")
    if isinstance(cfg.get("rope_parameters"), dict):
        theta = cfg["rope_parameters"].get("rope_theta", theta)
        scaling = scaling or cfg["rope_parameters"]
    T = len(tokens)
    ids = torch.tensor(list(tokens), dtype=torch.long)
    x = w["model.embed_tokens.weight"][ids]                       # [T, d]
    inv = rope_inv_freq(theta, hd, scaling)
    sin, cos = rope_angles(torch.arange(T), inv)
    rope = apply_rope_half if pairing == "half" else apply_rope_interleaved
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        xn = r(rms_norm(x, w[p + "input_layernorm.weight"], eps))
        q = r(linear(xn, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias")))
        k = r(linear(xn, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias")))
        v = r(linear(xn, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias")))
        q = r(rope(q.view(T, H, hd), sin, cos))
        k = r(rope(k.view(T, G, hd), sin, cos))
        a = r(causal_attention(q, k, v.view(T, G, hd)).reshape(T, H * hd))
        x = x + linear(a, w[p + "self_attn.o_proj.weight"], w.get(p + "self_attn.o_proj.bias"))
        xn2 = r(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
        gate = linear(xn2, w[p + "mlp.gate_proj.weight"], w.get(p + "mlp.gate_proj.bias"))
        up = linear(xn2, w[p + "mlp.up_proj.weight"], w.get(p + "mlp.up_proj.bias"))
        h = r(swiglu(r(gate), r(up)))
        x = x + linear(h, w[p + "mlp.down_proj.weight"], w.get(p + "mlp.down_proj.bias"))
    if return_hidden:
        return x
    xn = r(rms_norm(x, w["model.norm.weight"], eps))
    head = w["lm_head.weight"] if "lm_head.weight" in w and not cfg.get("tie_word_embeddings", False) \
        else w["model.embed_tokens.weight"]
    return linear(xn, head)


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 (nearest even) and widen again: what a store in bf16 does."""
    return t.to(torch.float32).to(torch.bfloat16).to(F64)


# --------------------------------------------------------------------------- sampling
class Rng:
    """src/sampling.rs:4-27: xorshift64 (13, 7, 17); seed 0 -> 0xDEADBEEFCAFE1337;
    next_f32 = (state >> 40) / 2^24."""

    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = 0xDEADBEEFCAFE1337 if seed == 0 else seed & self.MASK

    def next_f32(self) -> float:
        s = self.state
        s ^= (s << 13) & self.MASK
        s ^= s >> 7
        s ^= (s << 17) & self.MASK
        self.state = s
        return float(np.float32(s >> 40) / np.float32(1 << 24))


def apply_repeat_penalty(logits: np.ndarray, recent: Sequence[int], penalty: float) -> None:
    """src/sampling.rs:321-338: for every entry of the recent window (repeats count
    again): v > 0 -> v / p, else v * p; non-finite -> -inf; p == 1 is a no-op."""
    if penalty == 1.0:
        return
    for t in recent:
        if 0 <= t < logits.shape[0]:
            v = logits[t]
            if not np.isfinite(v):
                logits[t] = -np.inf
            elif v > 0:
                logits[t] = np.float32(v / np.float32(penalty))
            else:
                logits[t] = np.float32(v * np.float32(penalty))


def argmax_finite(logits: np.ndarray) -> int:
    """src/sampling.rs:341-356: highest finite logit, first one wins."""
    v = np.where(np.isfinite(logits), logits, -np.inf)
    return int(np.argmax(v))


def sample(logits_in: np.ndarray, temperature: float, rng: Rng, top_k: int = 0, top_p: float = 1.0,
           min_p: float = 0.0, repeat_penalty: float = 1.0, recent: Sequence[int] = ()) -> int:
    """src/sampling.rs:66-212 (``sample_with_scratch``) and 215-306 (``sample_top_k``),
    in f32 like the reference."""
    logits = np.array(logits_in, dtype=np.float32)
    n = logits.shape[0]
    if n == 0:
        return 0
    apply_repeat_penalty(logits, recent, repeat_penalty)
    if temperature < 1e-6:
        return argmax_finite(logits)
    inv_temp = np.float32(1.0) / np.float32(temperature)
    if 0 < top_k < n:
        if top_k == 1:
            return argmax_finite(logits)
        v = np.where(np.isfinite(logits), logits, -np.inf).astype(np.float32)
        # descending by value, ties keep the lower index first (insertion order)
        order = np.lexsort((np.arange(n), -v))[:top_k]
        if not np.isfinite(v[order[0]]):
            return argmax_finite(logits)
        wts = np.exp((v[order] - v[order[0]]) * inv_temp).astype(np.float32)
        total = np.float32(0)
        for x in wts:
            total = np.float32(total + x)
        limit = len(order)
        if min_p > 0:
            thr = np.float32(min_p) * wts[0]
            below = np.nonzero(wts < thr)[0]
            limit = max(int(below[0]) if below.size else len(order), 1)
        cutoff, kept = limit, np.float32(0)
        for x in wts[:limit]:
            kept = np.float32(kept + x)
        if top_p < 1.0:
            c = np.float32(0)
            thr = np.float32(top_p) * total
            for i in range(limit):
                c = np.float32(c + wts[i])
                if c > thr:
                    cutoff, kept = i + 1, c
                    break
        r = np.float32(rng.next_f32()) * kept
        c = np.float32(0)
        for i in range(cutoff):
            c = np.float32(c + wts[i])
            if c > r:
                return int(order[i])
        return int(order[cutoff - 1])
    logits = np.where(np.isfinite(logits), logits, -np.inf).astype(np.float32)
    logits = (logits * inv_temp).astype(np.float32)
    mx = logits.max()
    wts = np.exp(logits - mx).astype(np.float32)
    total = np.float32(0)
    for x in wts:
        total = np.float32(total + x)
    if min_p > 0 and top_p >= 1.0:
        keep = wts >= np.float32(min_p)
        kept = np.float32(0)
        for x in wts[keep]:
            kept = np.float32(kept + x)
        r = np.float32(rng.next_f32()) * kept
        c, last = np.float32(0), 0
        for i in np.nonzero(keep)[0]:
            last = int(i)
            c = np.float32(c + wts[i])
            if c > r:
                return int(i)
        return last
    if top_p < 1.0:
        order = np.lexsort((np.arange(n), -wts))
        sw = wts[order]
        limit = n
        if min_p > 0:
            below = np.nonzero(sw < np.float32(min_p) * sw[0])[0]
            limit = max(int(below[0]) if below.size else n, 1)
        cutoff = limit
        c, thr = np.float32(0), np.float32(top_p) * total
        for i in range(limit):
            c = np.float32(c + sw[i])
            if c > thr:
                cutoff = i + 1
                break
        kept = np.float32(0)
        for x in sw[:cutoff]:
            kept = np.float32(kept + x)
        r = np.float32(rng.next_f32()) * kept
        c = np.float32(0)
        for i in range(cutoff):
            c = np.float32(c + sw[i])
            if c > r:
                return int(order[i])
        return int(order[cutoff - 1])
    r = np.float32(rng.next_f32()) * total
    c = np.float32(0)
    for i in range(n):
        c = np.float32(c + wts[i])
        if c > r:
            return i
    return n - 1


# --------------------------------------------------------------------------- generation
def generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], max_tokens: int,
             temperature: float = 0.0, seed: int = 1, stop_ids: Sequence[int] = (),
             top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repeat_penalty: float = 1.0,
             round_fn=None) -> List[int]:
    """The decode loop of src/runtime.rs:3266-3342 for one sequence, recomputing the
    whole sequence each step: sample from the last logits; a stop token ends the
    run and is neither emitted nor counted (3305-3307); the recent window for the
    repeat penalty is the last 64 tokens of prompt + output (493-521)."""
    seq = list(prompt)
    out: List[int] = []
    rng = Rng(seed)
    while len(out) < max_tokens:
        logits = forward(cfg, w, seq, round_fn=round_fn)[-1].to(torch.float32).numpy()
        tok = sample(logits, temperature, rng, top_k, top_p, min_p, repeat_penalty, recent=seq[-64:])
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
