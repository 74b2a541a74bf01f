"""Random weights from a configuration and a seed: as a model folder (config.json +
model.safetensors) or straight onto the device.

The reference has random weights only in its tests (byte-pattern generators,
src/model.rs:2451-2478, 2842-2870).  Here every checkpoint tensor has its own seed made of
(seed, tensor name), so a tensor's values do not depend on which other tensors exist:
matrices, tables and biases ~ N(0, std), norm weights 1 or, with ``norm_noise``, 1 + N(0, std).
Values are float32 and rounded once to the storage dtype (nearest even).

The numbers are the same wherever they are drawn: element i of a tensor is mean + std * z_i
with z_i = (sum of twelve uniform 16-bit integers - 393,210) / 65,536 (the twelve-uniform
approximation of a standard normal: variance 1, steps of 2^-16, |z| <= 6), the integers being
the 16-bit fields of three splitmix64 outputs over the counter seed + 3 i.  Integer arithmetic,
one float multiply and one float add: ``normal_values`` here (numpy) and the device kernel
(csrc/random_fill.cu) agree bit for bit, so a folder written with ``write_random_model`` and a
model drawn on the device by ``Runner.from_config`` with the same seed hold the same weights.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Any, Dict, Mapping, Optional, Union

import numpy as np
import torch

from ..config.registry import resolve_architecture
from ..config.spec import ParamSpec
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    return (seed * 0x9E3779B97F4A7C15 + zlib.crc32(name.encode("utf-8")) * 0x100000001B3 + 0x1234567) % (1 << 63)


_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def normal_values(seed: int, n: int, mean: float, std: float) -> np.ndarray:
    """Elements 0 .. n-1 of the tensor with this seed, float32 (see the module's text)."""
    out = np.empty(n, dtype=np.float32)
    step = np.float32(std) * np.float32(1.0 / 65536.0)          # a power of two: exact
    s = np.uint64(seed & 0xFFFFFFFFFFFFFFFF)
    f = np.uint64(0xFFFF)
    chunk = 1 << 16                                            # the temporaries of a chunk stay in the cache: 7 times the pace of 4 M
    for at in range(0, n, chunk):
        i = np.arange(at, min(n, at + chunk), dtype=np.uint64)
        total = np.zeros(i.shape[0], dtype=np.int64)
        with np.errstate(over="ignore"):
            base = s + np.uint64(3) * i
            for r in range(3):
                h = _splitmix64(base + np.uint64(r))
                total += ((h & f) + ((h >> np.uint64(16)) & f) + ((h >> np.uint64(32)) & f) + (h >> np.uint64(48))).astype(np.int64)
        z = (total - 393210).astype(np.float32)                   # exact: below 2^20 in magnitude
        out[at:at + i.shape[0]] = np.float32(mean) + z * step     # a multiply, then an add, each rounded
    return out


def draw(name: str, shape, init: str, seed: int, std: float, norm_noise: bool,
         dtype: torch.dtype, device) -> torch.Tensor:
    """One tensor: on a CUDA device by the library's kernel, else on the host; the same numbers."""
    device = torch.device(device)
    if init not in ("zeros", "ones", "normal"):
        raise ValueError(f"unknown init {init!r}")
    if init == "zeros":
        return torch.zeros(shape, dtype=dtype, device=device)
    if init == "ones" and not norm_noise:
        return torch.ones(shape, dtype=dtype, device=device)
    mean = 1.0 if init == "ones" else 0.0
    tseed = _tensor_seed(seed, name)
    if device.type == "cuda":
        from .. import kernels
        if dtype in (torch.float32, torch.bfloat16):
            t = torch.empty(shape, dtype=dtype, device=device)
            kernels.random_fill(t, tseed, mean, std)
            return t
        t = torch.empty(shape, dtype=torch.float32, device=device)
        kernels.random_fill(t, tseed, mean, std)
        return t.to(dtype)
    n = 1
    for d in shape:
        n *= int(d)
    return torch.from_numpy(normal_values(tseed, n, mean, std)).view(*shape).to(dtype)


def _model_param_specs(config_dict: Mapping[str, Any]) -> Dict[str, ParamSpec]:
    from ..models.decoder import DecoderModel
    from ..parts import Runtime
    arch = resolve_architecture(config_dict)
    spec = arch.build_spec(arch.parse_config(config_dict))
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    return model.param_specs()


def write_random_model(model_dir: str, config: Union[Mapping[str, Any], Any], seed: int,
                       dtype: Optional[str] = None, std: float = 0.02, norm_noise: bool = False,
                       device: str = "cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for random weights.

    ``config``: a config.json dictionary or a typed configuration with ``to_dict()``.
    ``dtype``: storage dtype of the file ("bfloat16", "float32", "float16");
    default: the configuration's ``torch_dtype``.  ``device``: where the values are computed
    (a CUDA device is much faster for large models; the values are the same).
    """
    cfg = dict(config.to_dict() if hasattr(config, "to_dict") else config)
    dtype = dtype or cfg.get("torch_dtype", "bfloat16")
    if dtype not in _TORCH_DTYPES:
        raise ValueError(f"dtype {dtype!r} is not one of {sorted(_TORCH_DTYPES)}")
    cfg["torch_dtype"] = dtype
    specs = _model_param_specs(cfg)
    tensors: Dict[str, torch.Tensor] = {}
    for path, ps in specs.items():
        if ps.alias_of is not None:
            continue   # tied: the file holds the shared tensor once
        for src in ps.sources:
            tensors[src.name] = draw(src.name, src.shape, ps.init, seed, std, norm_noise,
                                     _TORCH_DTYPES[dtype], device).cpu()
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir


def random_parameters(specs: Mapping[str, ParamSpec], seed: int, compute_dtype: torch.dtype, device,
                      storage_dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                      norm_noise: bool = False) -> Dict[str, torch.Tensor]:
    """The same draw as ``write_random_model`` followed by loading, without files:
    values are rounded to ``storage_dtype`` as a file would hold them, then kept in
    the run-time dtype of their role.  Generated on ``device``: the same values as the
    folder of the same seed holds."""
    from .loader import place_source, runtime_dtype
    out: Dict[str, torch.Tensor] = {}
    aliases = []
    for path, ps in specs.items():
        if ps.alias_of is not None:
            aliases.append((path, ps.alias_of))
            continue
        dt = runtime_dtype(ps.role, storage_dtype, compute_dtype)
        dest = torch.empty(ps.shape, dtype=dt, device=device)
        for i, src in enumerate(ps.sources):
            place_source(dest, ps, i, draw(src.name, src.shape, ps.init, seed, std, norm_noise, storage_dtype, device).to(dt))
        out[path] = dest
    for path, target in aliases:
        out[path] = out[target]
    return out
