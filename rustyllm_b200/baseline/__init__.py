"""The timed CPU baseline: a plain float32 C++ implementation of the Llama decoder
(``cpu_llama.cc`` beside this file), one token against a cache, in the reference's order of
operations (SimonWaldherr/RustyLLM src/model.rs:7177-7358).

It stands where a run of the reference itself would stand if the reference could be built
here; its numbers are this library's own CPU reference, never RustyLLM's.  Nothing on the GPU
path imports this module.  The shared object is built with g++ at first use, beside the CUDA
library's build folder, and is named by a hash of its source, its flags and this machine's CPU
features (it is compiled for the machine it runs on).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import sys
import time
from typing import Any, Dict, List, Mapping, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "cpu_llama.cc")
FLAGS = ["-O3", "-march=native", "-fopenmp", "-fno-math-errno", "-std=c++17", "-shared", "-fPIC"]


def _cpu_features() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return line
    except OSError:
        pass
    return "unknown"


def _library_path() -> str:
    from ..csrc.build import _build_root
    h = hashlib.sha256()
    with open(SOURCE, "rb") as f:
        h.update(f.read())
    h.update(" ".join(FLAGS).encode())
    h.update(_cpu_features().encode())
    return os.path.join(_build_root(), f"libcpu_llama_{h.hexdigest()[:16]}.so")


_lib = None


def library() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = _library_path()
    if not os.path.isfile(path):
        print(f"[rustyllm_b200 build] compiling {os.path.basename(SOURCE)} for this machine's CPU ...", file=sys.stderr, flush=True)
        t0 = time.time()
        tmp = path + f".tmp{os.getpid()}"
        p = subprocess.run(["g++"] + FLAGS + [SOURCE, "-o", tmp], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"g++ failed on {SOURCE}:\n{p.stdout}")
        os.replace(tmp, path)
        print(f"[rustyllm_b200 build] built {path} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    lib = ctypes.CDLL(path)
    lib.cpu_llama_new.restype = ctypes.c_void_p
    lib.cpu_llama_new.argtypes = [ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int]
    lib.cpu_llama_free.restype = None
    lib.cpu_llama_free.argtypes = [ctypes.c_void_p]
    lib.cpu_llama_add_layer.restype = ctypes.c_int
    lib.cpu_llama_add_layer.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.cpu_llama_set_globals.restype = ctypes.c_int
    lib.cpu_llama_set_globals.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.cpu_llama_forward.restype = ctypes.c_int
    lib.cpu_llama_forward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.cpu_llama_threads.restype = ctypes.c_int
    lib.cpu_llama_threads.argtypes = []
    _lib = lib
    return lib


def rope_table(theta: float, head_dim: int, scaling: Optional[Mapping[str, Any]]) -> np.ndarray:
    """Inverse frequencies in the reference's form ``1 / (base^(2i/hd) * factor_i)``
    (``build_rope_inv_freq_with_factors``, src/model.rs:3035-3057), computed in float64 and rounded
    once.  Without scaling every factor is 1.  "llama3" scaling, stated as the per-pair divisors a
    GGUF file would carry: with x = original context / wavelength (how many periods fit the original
    context), factor_i = 1 for x > high, ``factor`` for x < low, and in between
    1 / ((1 - s) / factor + s) with s = (x - low) / (high - low)."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    base = np.power(float(theta), 2.0 * i / head_dim)
    div = np.ones_like(base)
    if scaling is not None:
        f, lo, hi = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        x = float(scaling["original_max_position_embeddings"]) / (2.0 * np.pi * base)
        s = (x - lo) / (hi - lo)
        div = np.where(x > hi, 1.0, np.where(x < lo, f, 1.0 / ((1.0 - s) / f + s)))
    return (1.0 / (base * div)).astype(np.float32)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class CpuLlama:
    """The C++ model over float32 arrays that this object keeps alive.

    ``config``: a config.json dictionary of the Llama architecture.  ``tensors``: checkpoint
    name -> array (anything numpy takes).  ``run_layers``: how many layers a token runs through
    (default: the configuration's); when it exceeds the layers ``tensors`` holds, those are used
    in turn, which changes no memory traffic of a timing run and makes its logits meaningless."""

    def __init__(self, config: Mapping[str, Any], tensors: Mapping[str, Any], max_seq: int,
                 run_layers: Optional[int] = None):
        from ..config.llama import LlamaConfig
        cfg = LlamaConfig.from_dict(dict(config))
        if cfg.mlp_bias:
            raise ValueError("the CPU baseline follows the reference, which has no feed-forward biases")
        self.cfg = cfg
        self.lib = library()
        held = 0
        while f"model.layers.{held}.input_layernorm.weight" in tensors:
            held += 1
        if held == 0:
            raise ValueError("no layer tensors given")
        self.run_layers = run_layers or cfg.num_hidden_layers
        inv = rope_table(cfg.rope_theta, cfg.head_dim, cfg.rope_scaling.to_dict() if cfg.rope_scaling else None)
        self._keep: List[np.ndarray] = [_f32(inv)]
        dims = np.asarray([cfg.hidden_size, self.run_layers, cfg.num_attention_heads, cfg.num_key_value_heads,
                           cfg.head_dim, cfg.intermediate_size, cfg.vocab_size, max_seq], dtype=np.int32)
        self.handle = self.lib.cpu_llama_new(dims.ctypes.data, float(cfg.rms_norm_eps), self._keep[0].ctypes.data, 0)
        if not self.handle:
            raise ValueError("the CPU baseline refused these sizes")

        def take(name: str, optional: bool = False) -> Optional[int]:
            if name not in tensors:
                if optional:
                    return None
                raise KeyError(f"tensor {name} is missing")
            a = _f32(tensors[name])
            self._keep.append(a)
            return a.ctypes.data

        for l in range(min(held, self.run_layers)):
            p = f"model.layers.{l}."
            ptrs = [take(p + "input_layernorm.weight"), take(p + "self_attn.q_proj.weight"),
                    take(p + "self_attn.k_proj.weight"), take(p + "self_attn.v_proj.weight"),
                    take(p + "self_attn.q_proj.bias", True), take(p + "self_attn.k_proj.bias", True),
                    take(p + "self_attn.v_proj.bias", True), take(p + "self_attn.o_proj.weight"),
                    take(p + "post_attention_layernorm.weight"), take(p + "mlp.gate_proj.weight"),
                    take(p + "mlp.up_proj.weight"), take(p + "mlp.down_proj.weight")]
            if p + "self_attn.o_proj.bias" in tensors:
                raise ValueError("the CPU baseline follows the reference, which has no output-projection bias")
            arr = (ctypes.c_void_p * 12)(*ptrs)
            if self.lib.cpu_llama_add_layer(self.handle, arr) != 0:
                raise ValueError(f"layer {l} was refused")
        embed = take("model.embed_tokens.weight")
        head = take("lm_head.weight", True) or embed          # absent: tied (src/model.rs:3654-3667)
        if self.lib.cpu_llama_set_globals(self.handle, embed, take("model.norm.weight"), head) != 0:
            raise ValueError("embedding, final norm or head missing")
        self.vocab = cfg.vocab_size

    def forward(self, token: int, pos: int, want_logits: bool = True) -> Optional[np.ndarray]:
        out = np.empty(self.vocab, dtype=np.float32) if want_logits else None
        rc = self.lib.cpu_llama_forward(self.handle, int(token), int(pos), out.ctypes.data if want_logits else None)
        if rc != 0:
            raise ValueError(f"token {token} at position {pos} was refused ({rc})")
        return out

    def logits_of(self, tokens: Sequence[int]) -> np.ndarray:
        """Logits at every position of one sequence fed from position 0: [T, vocab]."""
        return np.stack([self.forward(t, i) for i, t in enumerate(tokens)])

    @property
    def threads(self) -> int:
        return int(self.lib.cpu_llama_threads())

    def close(self) -> None:
        if self.handle:
            self.lib.cpu_llama_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def from_model_dir(model_dir: str, max_seq: Optional[int] = None) -> CpuLlama:
    """The CPU model of a model folder (its own reading of config.json and the safetensors)."""
    import torch
    from ..config.files import read_config_json
    from ..weights.safetensors_io import Checkpoint
    cfg = read_config_json(model_dir)
    ck = Checkpoint(model_dir)
    tensors = {n: ck.tensor(n).to(torch.float32).clone().numpy() for n in ck.names()}   # copies: the file's mapping is closed below
    ck.close()
    return CpuLlama(cfg, tensors, max_seq or int(cfg.get("max_position_embeddings", 2048)))


def time_decode(config: Mapping[str, Any], distinct_layers: int, context: int, tokens: int, seed: int = 0) -> Dict[str, Any]:
    """Decode speed of the CPU baseline at the configuration's full depth with random float32
    weights: ``context`` positions are fed without the head, then ``tokens`` tokens with it are
    timed.  Only ``distinct_layers`` layers' weights are held and used in turn (a layer's
    weights are far larger than the caches, so every pass streams them from memory all the same)."""
    from ..config.llama import LlamaConfig
    cfg = LlamaConfig.from_dict(dict(config))
    rng = np.random.default_rng(seed)
    d, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qd, kvd = cfg.q_size, cfg.kv_size

    block = rng.standard_normal(1 << 22, dtype=np.float32) * np.float32(0.02)

    def w(*shape):
        # a timing run only needs ordinary numbers: one random block, repeated to the tensor's size
        out = np.empty(int(np.prod(shape)), dtype=np.float32)
        for at in range(0, out.size, block.size):
            n = min(block.size, out.size - at)
            out[at:at + n] = block[:n]
        return out.reshape(shape)
    # one table serves as embedding and head (a token reads one row of the embedding, so sharing the
    # array changes nothing that is timed; the head's product streams the whole table either way)
    t = {"model.embed_tokens.weight": w(V, d), "model.norm.weight": np.ones(d, np.float32)}
    for l in range(distinct_layers):
        p = f"model.layers.{l}."
        t.update({p + "input_layernorm.weight": np.ones(d, np.float32), p + "post_attention_layernorm.weight": np.ones(d, np.float32),
                  p + "self_attn.q_proj.weight": w(qd, d), p + "self_attn.k_proj.weight": w(kvd, d),
                  p + "self_attn.v_proj.weight": w(kvd, d), p + "self_attn.o_proj.weight": w(d, qd),
                  p + "mlp.gate_proj.weight": w(I, d), p + "mlp.up_proj.weight": w(I, d), p + "mlp.down_proj.weight": w(d, I)})
    m = CpuLlama(dict(config, attention_bias=False, mlp_bias=False), t, context + tokens + 1)
    ids = rng.integers(0, V, size=context + tokens + 1)
    for i in range(context):
        m.forward(int(ids[i]), i, want_logits=False)
    m.forward(int(ids[context]), context)                       # one untimed token with the head
    t0 = time.perf_counter()
    for i in range(context + 1, context + 1 + tokens):
        m.forward(int(ids[i]), i)
    dt = time.perf_counter() - t0
    out = {"tokens_per_s": tokens / dt, "ms_per_token": dt * 1e3 / tokens, "threads": m.threads, "tokens": tokens,
           "context": context, "layers": cfg.num_hidden_layers, "distinct_layers": distinct_layers, "batch": 1,
           "dtype": "float32", "what": "our CPU reference: plain C++ float32 (OpenMP), not a RustyLLM number"}
    m.close()
    return out
