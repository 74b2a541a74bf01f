"""Binding a checkpoint's tensors to a model's parameters, by name.

Counterpart of the reference's ``load_model`` and its pre-load
``compatibility_report`` (src/model.rs:3573-4048, src/runtime.rs:1263-1406): every
tensor is looked up by name and checked against the shape the configuration
implies before anything is copied.  Where the reference panics on the first
missing tensor (src/model.rs:3208), this loader collects everything that is wrong
- missing tensors, unexpected tensors, wrong shapes, unusable dtypes - into one
``WeightsError``.

Run-time dtypes: matrices and tables take the compute dtype of the run, except
that a tensor the file stores as 32-bit float stays 32-bit (unless the caller asks
for it to be rounded: ``keep_fp32=False``); vectors used in
32-bit math (norm weights, biases) are always float32; integer tables are int32.
Q/K/V and gate/up are concatenated along the rows so one matrix product serves
each (the reference goes the other way and splits fused tensors by rows,
src/model.rs:3795-3857, 3933-3967).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.spec import ParamSpec
from .safetensors_io import Checkpoint

_FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INT_DTYPES = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightsError(ValueError):
    """Everything that is wrong between a checkpoint and the model, at once."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, tuple, tuple]],
                 wrong_dtype: Sequence[Tuple[str, str, str]] = (), where: str = ""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"checkpoint {where!r} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: file has {list(got)}, model needs {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unusable dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n}: file has {got}, model needs {want}" for n, got, want in self.wrong_dtype))
        super().__init__("\n".join(lines))


def runtime_dtype(role: str, file_dtype: torch.dtype, compute_dtype: torch.dtype,
                  keep_fp32: bool = True) -> torch.dtype:
    if role == "int_table":
        return torch.int32
    if role == "vector":
        return torch.float32
    if compute_dtype == torch.float32:
        return torch.float32
    # reduced-precision run: a tensor stored in 32-bit (or wider) stays 32-bit unless the
    # caller asked for it to be rounded
    if keep_fp32 and file_dtype in (torch.float32, torch.float64):
        return torch.float32
    return compute_dtype


def place_source(dest: torch.Tensor, ps: ParamSpec, index: int, tensor: torch.Tensor) -> None:
    """Copy source ``index`` of a parameter into its rows of ``dest`` (concatenated or interleaved)."""
    if ps.layout == "interleave":
        n = len(ps.sources)
        if any(s.shape != ps.sources[0].shape for s in ps.sources):
            raise ValueError("interleaved sources must have equal shapes")
        dest[index::n].copy_(tensor)
    else:
        row = sum(s.shape[0] for s in ps.sources[:index])
        dest[row:row + ps.sources[index].shape[0]].copy_(tensor)


def check_checkpoint(params: Mapping[str, ParamSpec], entries: Mapping[str, object],
                     ignored: Iterable[str] = (), where: str = "") -> None:
    """Compare names, shapes and dtype classes; raise one WeightsError for all faults."""
    missing: List[str] = []
    wrong_shape: List[Tuple[str, tuple, tuple]] = []
    wrong_dtype: List[Tuple[str, str, str]] = []
    used = set()
    for path, ps in params.items():
        present = [s.name in entries for s in ps.sources]
        if ps.alias_of is not None and not any(present):
            continue  # tied: shares another parameter's storage
        if ps.optional_in_file and not any(present):
            continue
        for s, here in zip(ps.sources, present):
            if not here:
                missing.append(s.name)
                continue
            used.add(s.name)
            e = entries[s.name]
            if tuple(e.shape) != tuple(s.shape):
                wrong_shape.append((s.name, tuple(e.shape), tuple(s.shape)))
            if ps.role == "int_table":
                if e.dtype not in _INT_DTYPES:
                    wrong_dtype.append((s.name, str(e.dtype), "an integer type"))
            elif e.dtype not in _FLOAT_DTYPES:
                wrong_dtype.append((s.name, str(e.dtype), "a floating-point type"))
    ignored = set(ignored)
    unexpected = sorted(n for n in entries if n not in used and n not in ignored)
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(sorted(missing), unexpected, wrong_shape, wrong_dtype, where)


def load_parameters(params: Mapping[str, ParamSpec], checkpoint: Checkpoint,
                    compute_dtype: torch.dtype, device: torch.device,
                    ignored: Iterable[str] = (), keep_fp32: bool = True) -> Dict[str, torch.Tensor]:
    """Check first, then copy: returns ``{parameter path: device tensor}``.  ``keep_fp32``:
    whether a matrix stored in 32-bit stays 32-bit in a reduced-precision run."""
    check_checkpoint(params, checkpoint.entries, ignored, checkpoint.model_dir)
    out: Dict[str, torch.Tensor] = {}
    aliases: List[Tuple[str, str]] = []
    for path, ps in params.items():
        present = [s.name in checkpoint.entries for s in ps.sources]
        if not any(present):
            if ps.alias_of is not None:
                aliases.append((path, ps.alias_of))
            continue
        file_dtypes = {checkpoint.entries[s.name].dtype for s in ps.sources}
        widest = torch.float32 if (torch.float32 in file_dtypes or torch.float64 in file_dtypes) \
            else next(iter(file_dtypes))
        dt = runtime_dtype(ps.role, widest, compute_dtype, keep_fp32)
        dest = torch.empty(ps.shape, dtype=dt, device=device)
        for i, s in enumerate(ps.sources):
            t = checkpoint.tensor(s.name)
            # bf16/f16 -> f32 widening is exact; f32 -> bf16 rounds to nearest even
            # (the reference's f32_to_bf16, src/simd.rs:88-96).
            place_source(dest, ps, i, t.to(dt) if t.dtype != dt else t)
        out[path] = dest
    for path, target in aliases:
        if target not in out:
            raise WeightsError([f"{path} (tied to {target}, which was not loaded)"], [], [], (),
                               checkpoint.model_dir)
        out[path] = out[target]
    return out
