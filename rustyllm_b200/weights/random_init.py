"""Random weights from a configuration and a seed: as a model folder (config.json +
model.safetensors) or straight onto the device.

The reference has random weights only in its tests (byte-pattern generators,
src/model.rs:2451-2478, 2842-2870).  Here every checkpoint tensor is drawn from its
own generator seeded by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist: matrices and tables N(0, std), biases N(0, std), norm
weights 1 or, with ``norm_noise``, 1 + N(0, std).  Values are drawn in float32 and
rounded once to the storage dtype (nearest even).
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Any, Dict, Mapping, Optional, Union

import torch

from ..config.registry import resolve_architecture
from ..config.spec import ParamSpec
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    return (seed * 0x9E3779B97F4A7C15 + zlib.crc32(name.encode("utf-8")) * 0x100000001B3 + 0x1234567) % (1 << 63)


def draw(name: str, shape, init: str, seed: int, std: float, norm_noise: bool,
         dtype: torch.dtype, device) -> torch.Tensor:
    device = torch.device(device)
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if init == "zeros":
        t = torch.zeros(shape, dtype=torch.float32, device=device)
    elif init == "ones":
        t = torch.ones(shape, dtype=torch.float32, device=device)
        if norm_noise:
            t += torch.randn(shape, generator=g, dtype=torch.float32, device=device) * std
    elif init == "normal":
        t = torch.randn(shape, generator=g, dtype=torch.float32, device=device) * std
    else:
        raise ValueError(f"unknown init {init!r}")
    return t.to(dtype)


def _model_param_specs(config_dict: Mapping[str, Any]) -> Dict[str, ParamSpec]:
    from ..models.decoder import DecoderModel
    from ..parts import Runtime
    arch = resolve_architecture(config_dict)
    spec = arch.build_spec(arch.parse_config(config_dict))
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    return model.param_specs()


def write_random_model(model_dir: str, config: Union[Mapping[str, Any], Any], seed: int,
                       dtype: Optional[str] = None, std: float = 0.02, norm_noise: bool = False) -> str:
    """Write ``config.json`` and ``model.safetensors`` for random weights.

    ``config``: a config.json dictionary or a typed configuration with ``to_dict()``.
    ``dtype``: storage dtype of the file ("bfloat16", "float32", "float16");
    default: the configuration's ``torch_dtype``.
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
                                     _TORCH_DTYPES[dtype], "cpu")
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
    the run-time dtype of their role.  Generated on ``device`` (a CUDA generator
    draws other values than the CPU one for the same seed)."""
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
