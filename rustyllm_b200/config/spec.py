"""The description of a model as data: which parts each layer is made of, in
which order layers run, and which cache storage each layer uses.

An architecture turns its typed configuration into a ``ModelSpec``; the generic
decoder (models/decoder.py) builds parts from it by looking each ``PartSpec.kind``
up in the part registries (parts/registry.py).  Nothing in a spec is specific to
one architecture: layers may differ from one another, the ``schedule`` may name a
layer more than once, and a layer may read another layer's cache
(``LayerSpec.cache_from``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and its constructor parameters."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ParamSource:
    """A tensor of the checkpoint, by name, with the shape it must have."""

    name: str
    shape: Tuple[int, ...]


@dataclass(frozen=True)
class ParamSpec:
    """One parameter a part wants bound.

    ``sources`` are concatenated along dimension 0 in the order given (one
    source = taken as is).  ``role`` decides the run-time dtype:
      - "matrix": compute dtype of the run, except that a tensor the file
        stores in 32-bit float stays 32-bit;
      - "vector": always float32 (norm weights, biases: used in 32-bit math);
      - "table": embedding table, treated like "matrix";
      - "int_table": integer data, kept as int32.
    ``alias_of`` names another parameter path ("embedding.weight") whose storage
    this one shares when none of its sources is in the file (tied weights).
    ``layout``: "concat" (sources one after another along dimension 0) or "interleave"
    (sources of equal shape, their rows taken in turn: s0[0], s1[0], s0[1], s1[1], ...).
    ``init`` tells the random-weights mode what to draw: "normal" (N(0, std)),
    "ones" (1, or 1 + N(0, std) when norm noise is asked for) or "zeros".
    """

    sources: Tuple[ParamSource, ...]
    role: str = "matrix"
    alias_of: Optional[str] = None
    optional_in_file: bool = False
    init: str = "normal"
    layout: str = "concat"

    @property
    def shape(self) -> Tuple[int, ...]:
        first = self.sources[0].shape
        rows = sum(s.shape[0] for s in self.sources)
        return (rows,) + tuple(first[1:])


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement of a mixer and a feed-forward with their norms.

    ``cache_from``: index (into ``ModelSpec.layers``) of the layer whose cache
    this layer's mixer reads instead of owning one; ``None`` = its own.
    """

    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[int, ...]            # order in which layers run; may repeat an index
    final_norm: PartSpec
    head: PartSpec
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Tuple[int, ...] = ()
    ignored_tensors: Tuple[str, ...] = ()  # names that may be in the file and are not read

    def validate(self) -> None:
        n = len(self.layers)
        if n == 0:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the schedule of layers is empty")
        for i in self.schedule:
            if not (0 <= i < n):
                raise ValueError(f"schedule names layer {i}, but there are {n} layers")
        for li, layer in enumerate(self.layers):
            src = layer.cache_from
            if src is not None:
                if not (0 <= src < n) or src == li:
                    raise ValueError(f"layer {li}: cache_from={src} is not another layer")
                if self.layers[src].cache_from is not None:
                    raise ValueError(f"layer {li}: cache_from={src} does not own a cache itself")
                first_src = self.schedule.index(src) if src in self.schedule else None
                first_me = self.schedule.index(li) if li in self.schedule else None
                if first_me is not None and (first_src is None or first_src > first_me):
                    raise ValueError(
                        f"layer {li} reads layer {src}'s cache but runs before it in the schedule")
