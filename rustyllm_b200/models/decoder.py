"""A decoder built from a ``ModelSpec``: embedding, layers run in the order the
schedule gives, final norm, head.  Nothing here is specific to one architecture.

Cache entries: every run of a layer in the schedule that owns a cache gets its own
entry (a layer named twice keeps two sets of keys and values, one per run); a layer
with ``cache_from`` reads the entry written by the latest earlier run of that layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..cache.sequence_cache import KVGroup, KVNeed, SequenceCache, StateNeed
from ..config.spec import ModelSpec, ParamSpec
from ..parts import Runtime
from ..parts.base import Part
from ..parts.registry import _REGISTRIES, build_part


@dataclass
class CacheView:
    """What one layer run sees of the cache."""
    kv_group: Optional[KVGroup]
    kv_layer: int
    state: Optional[torch.Tensor]     # [max_slots, nbytes] uint8, or None
    writes: bool                      # False: reads another layer's entry


def _collect_params(prefix: str, part: Part, out: Dict[str, Tuple[Part, str, ParamSpec]]) -> None:
    for name, ps in part.param_specs().items():
        out[f"{prefix}.{name}"] = (part, name, ps)
    for sub_name, sub in part.sub_parts().items():
        _collect_params(f"{prefix}.{sub_name}", sub, out)


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = []
        for ls in spec.layers:
            mixer = build_part("mixer", ls.mixer, runtime)
            mixer_norm = build_part("norm", ls.mixer_norm, runtime)
            ff = build_part("feed_forward", ls.feed_forward, runtime)
            ff_norm = build_part("norm", ls.feed_forward_norm, runtime)
            block_cls = _REGISTRIES["block"].get(ls.block.kind)
            if block_cls is None:
                raise KeyError(f"no block of kind {ls.block.kind!r} is registered")
            self.blocks.append(block_cls(runtime=runtime, mixer=mixer, mixer_norm=mixer_norm,
                                         feed_forward=ff, feed_forward_norm=ff_norm, **ls.block.params))
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.head, runtime)

        # cache entries along the schedule
        self.run_entry: List[Tuple[int, bool]] = []   # per schedule position: (entry, writes)
        self.entry_needs: List[Tuple[Optional[KVNeed], Optional[StateNeed]]] = []
        latest_entry_of_layer: Dict[int, int] = {}
        for li in spec.schedule:
            src = spec.layers[li].cache_from
            if src is None:
                mixer = self.blocks[li].mixer
                self.entry_needs.append((mixer.kv_need(), mixer.state_need()))
                entry = len(self.entry_needs) - 1
                latest_entry_of_layer[li] = entry
                self.run_entry.append((entry, True))
            else:
                self.run_entry.append((latest_entry_of_layer[src], False))

        self._params: Dict[str, Tuple[Part, str, ParamSpec]] = {}
        _collect_params("embedding", self.embedding, self._params)
        for i, b in enumerate(self.blocks):
            _collect_params(f"layers.{i}", b, self._params)
        _collect_params("final_norm", self.final_norm, self._params)
        _collect_params("head", self.head, self._params)

    @property
    def graph_capturable(self) -> bool:
        def ok(part: Part) -> bool:
            return part.graph_capturable and all(ok(p) for p in part.sub_parts().values())
        return all(ok(p) for p in [self.embedding, self.final_norm, self.head] + self.blocks)

    # ------------------------------------------------------------------ parameters
    def param_specs(self) -> Dict[str, ParamSpec]:
        return {path: ps for path, (_, _, ps) in self._params.items()}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        missing = [p for p, (_, _, ps) in self._params.items()
                   if p not in tensors and not ps.optional_in_file]
        if missing:
            raise KeyError(f"parameters without a tensor: {missing}")
        for path, (part, name, _) in self._params.items():
            if path in tensors:
                part.bind({name: tensors[path]})
        self._bound = dict(tensors)

    def parameter_bytes(self) -> int:
        seen, total = set(), 0
        for t in getattr(self, "_bound", {}).values():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ cache
    def kv_needs(self) -> List[Optional[KVNeed]]:
        return [kv for kv, _ in self.entry_needs]

    def state_needs(self) -> List[Optional[StateNeed]]:
        return [st for _, st in self.entry_needs]

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None,
                  max_seq_len: Optional[int] = None, dtype: Optional[torch.dtype] = None) -> SequenceCache:
        return SequenceCache(self.kv_needs(), self.state_needs(), max_tokens,
                             dtype or self.runtime.compute_dtype, self.runtime.device,
                             max_slots=max_slots, max_seq_len=max_seq_len)

    # ------------------------------------------------------------------ running
    use_native = True      # run the step's launch chain in native code where the model consists of parts it knows

    def native_for(self, cache: SequenceCache):
        """The native executor of this model on ``cache`` (csrc/decoder_forward.cu), or ``None``
        if a part of the model is not one it knows: then the Python parts launch the same kernels."""
        if not self.use_native:
            return None
        made = getattr(self, "_native", None)
        if made is None or made[0] is not cache:
            from .. import native
            made = self._native = (cache, native.NativeDecoder(self, cache) if native.eligible(self, cache) else None)
        return made[1]

    def forward(self, step, cache: SequenceCache) -> torch.Tensor:
        """All tokens of the step through all scheduled layers: float32 [M, d]."""
        nat = self.native_for(cache)
        if nat is not None:
            return nat.forward(step)
        x = self.embedding.forward(step)
        schedule = self.spec.schedule
        pending = None      # the next block's first norm, started by the block in front of it
        for pos, li in enumerate(schedule):
            entry, writes = self.run_entry[pos]
            where = cache.entry_group[entry]
            view = CacheView(
                kv_group=cache.groups[where[0]] if where else None,
                kv_layer=where[1] if where else 0,
                state=cache.state_entry(entry),
                writes=writes)
            block = self.blocks[li]
            if block.folds_norms:
                nxt = self.blocks[schedule[pos + 1]] if pos + 1 < len(schedule) else None
                want = nxt.first_norm_request(x.shape[0]) if nxt is not None and nxt.folds_norms else None
                pending = block.forward(x, step, view, pending=pending, next_norm=want)
            else:
                block.forward(x, step, view)
                pending = None
        return x

    def logits(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Final norm and head at the wanted rows only: float32 [len(rows), V]
        (the reference computes the head for the last prompt token only,
        src/runtime.rs:3405-3427)."""
        made = getattr(self, "_native", None)
        if self.use_native and made is not None and made[1] is not None:
            return made[1].logits(x, rows)
        xn = self.final_norm.forward(x, self.runtime.compute_dtype, rows)
        return self.head.forward(xn)
