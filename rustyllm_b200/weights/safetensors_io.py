"""A reader and a writer for the safetensors container.

Takes the place of the reference's GGUF parser and mmap wrapper
(src/gguf.rs:348-418, src/mmap.rs:23-44): a directory of named tensors with
dtype, shape and byte range, over a memory-mapped file.  Layout: 8-byte
little-endian header length, a JSON header ``{name: {dtype, shape,
data_offsets}}``, then the raw little-endian tensor data.  A model folder holds
``model.safetensors`` or several shards listed by ``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int   # absolute byte offset in the file
    end: int


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are views until copied."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        self.metadata = header.pop("__metadata__", {}) or {}
        base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            dt = _DTYPES.get(info.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {info.get('dtype')!r}")
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=dt).element_size()
            if e - b != want:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans {e - b} bytes, its shape {shape} needs {want}")
            if b < 0 or base + e > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} ends at byte {base + e}, beyond the file size {size} (truncated file?)")
            self.entries[name] = TensorEntry(name, dt, shape, path, base + b, base + e)
        # ACCESS_COPY: private copy-on-write pages, so torch can wrap the buffer
        # as writable without the file ever being modified.
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        n = (e.end - e.begin) // torch.empty((), dtype=e.dtype).element_size()
        t = torch.frombuffer(self._mm, dtype=e.dtype, count=n, offset=e.begin)
        return t.view(e.shape)

    def close(self) -> None:
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass  # views still alive; the mapping goes with them
        self._f.close()


class Checkpoint:
    """All tensors of a model folder by name, over one or several files."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        files: List[str]
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                wm = json.load(f).get("weight_map", {})
            files = sorted({os.path.join(model_dir, v) for v in wm.values()})
        elif os.path.isfile(single):
            files = [single]
        else:
            raise SafetensorsError(
                f"{model_dir!r} holds neither model.safetensors nor model.safetensors.index.json")
        self.files = [SafetensorsFile(p) for p in files]
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for sf in self.files:
            for name, e in sf.entries.items():
                if name in self.entries:
                    raise SafetensorsError(
                        f"tensor {name!r} is in both {self.entries[name].file} and {sf.path}")
                self.entries[name] = e
                self._owner[name] = sf

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    @property
    def total_bytes(self) -> int:
        return sum(os.path.getsize(sf.path) for sf in self.files)

    def close(self) -> None:
        for sf in self.files:
            sf.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write tensors (moved to the host, made contiguous) in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().to("cpu").contiguous()
        if t.dtype not in _DTYPE_NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be written")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for t in blobs:
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
