"""The step function: a batch of sequences, each bringing its next tokens (a whole
prompt, a chunk, or one token), run as one batch from the cache; logits come back
for the wanted places only.

The reference runs one token of one sequence per call (``forward_into(token, pos)``,
src/model.rs:7177-7185; a prompt's last token alone yields logits,
src/runtime.rs:3405-3427).  Here all tokens of the step are packed one sequence
after another - no padding exists, so padding cannot change a result - and every
kernel works from per-token position and slot.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from .. import kernels as K
from ..cache.sequence_cache import SequenceCache
from ..models.decoder import DecoderModel
from ..staging import PinnedStaging


@dataclass
class StepState:
    """Device-side description of one step, shared by every part."""
    num_tokens: int
    num_seqs: int
    tokens: torch.Tensor          # int32 [M]
    positions: torch.Tensor       # int32 [M]  position of each token in its sequence
    slot_of_token: torch.Tensor   # int32 [M]  cache slot of each token's sequence
    cu_seqlens: torch.Tensor      # int32 [B+1] token offsets of the sequences
    seq_slots: torch.Tensor       # int32 [B]
    kv_lens: torch.Tensor         # int32 [B]  sequence lengths after this step
    want_rows: torch.Tensor       # int32 [W]  packed rows whose logits are wanted
    q_lens: List[int]             # host copies
    kv_lens_host: List[int]
    max_q_len: int
    max_kv_len: int
    is_decode: bool               # every sequence brings exactly one token
    # device data that parts derive from the step and that holds for all layers (a part
    # that needs, say, a work plan of the sequences makes it once and leaves it here)
    derived: Dict[object, object] = field(default_factory=dict)
    # the longest sequence holds more than kernels.LONG_CONTEXT tokens.  A part may choose another
    # launch shape by it: captured steps are kept per (number of sequences, this flag, the next).
    long_context: bool = False
    # how far the longest sequence lies above the mean of all (kernels.length_spread: 0 equal,
    # 1 near, 2 far, 3 beyond); 3 where nobody said: the choice that is right for any lengths
    length_spread: int = 3


Want = Union[str, None, Sequence[Sequence[int]]]


class _DecodeGraph:
    """A captured single-token step for a fixed number of sequences.  Its kernels read
    the step's integers from ``static_in`` and leave logits in ``logits``; everything
    they read beyond that (page tables, cache pools, weights) keeps its address."""

    def __init__(self, engine: "Engine", num_seqs: int, long_context: bool = False, length_spread: int = 3):
        B = num_seqs
        self.num_seqs = B
        dev = engine.device
        self.static_in = torch.zeros(7 * B + 1, dtype=torch.int32, device=dev)
        st = engine.step_state(self.static_in, (B, B, B), [1] * B, [1] * B, lengths_class=(long_context, length_spread))
        before = K.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            x = engine.model.forward(st, engine.cache)
            self.logits = engine.model.logits(x, st.want_rows)
        self.launches = K.launch_count - before
        K.launch_count = before    # capturing runs nothing
        # pinned host copies of ``static_in``, taken in turn: a buffer is filled again only
        # after the copy that read it has finished, so the host may run ahead of the device
        n = self.static_in.numel()
        self._host = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._host_np = [h.numpy() for h in self._host]
        self._copied = [torch.cuda.Event() for _ in range(4)]
        self._in_use = [False] * 4
        self._next = 0
        self._rows = np.arange(B + 1, dtype=np.int32)

    def upload(self, tokens, starts, slots) -> int:
        """The integers of a single-token step from the host into ``static_in``; returns
        the bytes copied.  ``tokens`` None: the caller puts them there from the device."""
        B = self.num_seqs
        k = self._next
        self._next = (k + 1) % len(self._host)
        if self._in_use[k]:
            self._copied[k].synchronize()
        a = self._host_np[k]
        a[0:B] = 0 if tokens is None else tokens
        a[B:2 * B] = starts                       # position of the new token
        a[2 * B:3 * B] = slots                    # slot of each token
        a[3 * B:4 * B + 1] = self._rows           # token offsets: one token a sequence
        a[4 * B + 1:5 * B + 1] = slots
        a[5 * B + 1:6 * B + 1] = starts
        a[5 * B + 1:6 * B + 1] += 1               # lengths after the step
        a[6 * B + 1:7 * B + 1] = self._rows[:B]   # wanted rows: every sequence's only token
        self.static_in.copy_(self._host[k], non_blocking=True)
        self._copied[k].record()
        self._in_use[k] = True
        return a.nbytes


class Engine:
    """A model with its cache and the step function over them.

    ``use_graphs``: single-token steps are captured once per batch size and class of the
    sequences' lengths (``lengths_class``) in a CUDA graph and replayed (the first such step
    of a kind runs eagerly, so every kernel has been launched once before it is captured)."""

    def __init__(self, model: DecoderModel, cache: SequenceCache, use_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.device = model.runtime.device
        self.vocab_size = model.spec.vocab_size
        self._staging = PinnedStaging(self.device) if self.device.type == "cuda" else None
        self.h2d_bytes = 0
        self.use_graphs = use_graphs and self.device.type == "cuda" and model.graph_capturable
        self._graphs = {}          # (num_seqs, long context, length spread) -> _DecodeGraph
        self._eager_decodes = {}   # (num_seqs, long context, length spread) -> eager single-token steps run so far

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def warm_up(self, batch_sizes: Sequence[int]) -> None:
        """Capture the single-token step for these batch sizes now instead of at their first
        use in a generation (a capture takes a tenth of a second or more).  Needs that many
        free slots and one page each; leaves the cache as it found it."""
        if not self.use_graphs:
            return
        for B in sorted(set(int(b) for b in batch_sizes)):
            classes = [(False, spread) for spread in ((0,) if B == 1 else (0, 1, 2, 3))]
            if B <= 0 or all((B,) + c in self._graphs for c in classes):
                continue
            slots: List[int] = []
            try:
                for _ in range(B):                             # one by one: a failure part-way frees those taken
                    slots.append(self.alloc_slot())
                self.step(slots, [[0]] * B, None)              # one token each, so that a length exists
                for c in classes:                              # the launches of every class of lengths a batch can have
                    while (B,) + c not in self._graphs:        # an eager step first, then the capture
                        self.step(slots, [[0]] * B, "last", _lengths_class=c)
            finally:
                for s in slots:
                    self.free_slot(s)

    def build_step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], want: Want = "last"):
        """Validate on the host and lay out the step's integer inputs."""
        B = len(slots)
        if B == 0:
            raise ValueError("a step needs at least one sequence")
        if len(tokens) != B:
            raise ValueError(f"{B} slots but {len(tokens)} token lists")
        q_lens = [len(t) for t in tokens]
        starts = [self.cache.length(s) for s in slots]
        M = sum(q_lens)
        flat = np.empty(M, dtype=np.int64)
        positions = np.empty(M, dtype=np.int32)
        slot_of_token = np.empty(M, dtype=np.int32)
        cu = np.zeros(B + 1, dtype=np.int32)
        o = 0
        for b in range(B):
            n = q_lens[b]
            if n == 0:
                raise ValueError(f"sequence {b} of the step brings no token")
            flat[o:o + n] = np.asarray(tokens[b], dtype=np.int64)
            positions[o:o + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
            slot_of_token[o:o + n] = slots[b]
            o += n
            cu[b + 1] = o
        if flat.min() < 0 or flat.max() >= self.vocab_size:
            bad = int(flat[(flat < 0) | (flat >= self.vocab_size)][0])
            raise ValueError(f"token id {bad} lies outside the vocabulary [0, {self.vocab_size})")
        if want is None:
            rows: List[int] = []
        elif isinstance(want, str):
            if want == "last":
                rows = [int(cu[b + 1]) - 1 for b in range(B)]
            elif want == "all":
                rows = list(range(M))
            else:
                raise ValueError(f"want must be 'last', 'all', None or lists of places, got {want!r}")
        else:
            if len(want) != B:
                raise ValueError(f"{B} sequences but {len(want)} lists of wanted places")
            rows = []
            for b in range(B):
                for w in want[b]:
                    if not (0 <= w < q_lens[b]):
                        raise ValueError(f"sequence {b}: wanted place {w} is not among its {q_lens[b]} tokens")
                    rows.append(int(cu[b]) + int(w))
        kv_lens = [starts[b] + q_lens[b] for b in range(B)]
        packed = np.concatenate([
            flat.astype(np.int32), positions, slot_of_token, cu,
            np.asarray(slots, dtype=np.int32), np.asarray(kv_lens, dtype=np.int32),
            np.asarray(rows, dtype=np.int32)])
        return packed, (M, B, len(rows)), q_lens, kv_lens

    @staticmethod
    def lengths_class(kv_lens: Sequence[int]):
        """What of the sequences' lengths a kernel's launch shape may depend on (``StepState.long_context``,
        ``StepState.length_spread``); captured steps are kept by it."""
        return max(kv_lens) > K.LONG_CONTEXT, K.length_spread(kv_lens)

    def step_state(self, packed_dev: torch.Tensor, sizes, q_lens, kv_lens, lengths_class=None) -> StepState:
        M, B, W = sizes
        long_context, spread = lengths_class if lengths_class is not None else self.lengths_class(kv_lens)
        o = 0
        def take(n):
            nonlocal o
            t = packed_dev[o:o + n]
            o += n
            return t
        tokens, positions, slot_of_token = take(M), take(M), take(M)
        cu, seq_slots, kv = take(B + 1), take(B), take(B)
        rows = take(W)
        return StepState(M, B, tokens, positions, slot_of_token, cu, seq_slots, kv, rows,
                         list(q_lens), list(kv_lens), max(q_lens), max(kv_lens),
                         all(n == 1 for n in q_lens), long_context=long_context, length_spread=spread)

    def step_borrowed(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], want: Want = "last") -> Optional[torch.Tensor]:
        """``step`` for a caller that is done with the logits before its next step (the
        generation loop samples from them at once): a captured step then hands out the
        graph's own output buffer instead of a copy."""
        return self.step(slots, tokens, want, _borrow=True)

    def step_fed_from_device(self, slots: Sequence[int], token_ids: torch.Tensor) -> Optional[torch.Tensor]:
        """A single-token step of ``slots`` whose tokens are on the device already
        (``token_ids``: int32 [len(slots)], as a sampler leaves them), queued without waiting
        for them: the host may learn the ids while the step runs.  Ids a sampler wrote lie
        inside the vocabulary, so nothing is checked.  Returns the logits of the last (only)
        tokens in the captured step's own buffer, overwritten by its next run - or ``None``
        when no captured step for this many sequences exists yet and nothing was run."""
        B = len(slots)
        starts = [self.cache.length(s) for s in slots]
        g = self._graphs.get((B,) + self.lengths_class([n + 1 for n in starts])) if self.use_graphs and B > 0 else None
        if g is None:
            return None
        if token_ids.dtype != torch.int32 or token_ids.numel() != B:
            raise ValueError(f"token_ids must hold {B} int32 ids")
        ones = [1] * B
        self.cache.prepare(slots, ones)
        self.h2d_bytes += g.upload(None, starts, slots)
        g.static_in[:B].copy_(token_ids, non_blocking=True)
        g.graph.replay()
        K.launch_count += g.launches
        self.cache.commit(slots, ones)
        return g.logits

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], want: Want = "last",
             _borrow: bool = False, _lengths_class=None) -> Optional[torch.Tensor]:
        """Run the given tokens of the given sequences as one batch from the cache.

        ``slots[b]`` holds sequence b, whose next tokens are ``tokens[b]`` (they take
        positions ``length(slot) ..``).  ``want``: "last" (each sequence's last
        token), "all", ``None``, or per sequence the places among its tokens.
        Returns float32 logits ``[wanted, vocab]`` on the device in the order of the
        sequences and of their wanted places (``None`` if nothing is wanted).
        """
        B = len(slots)
        decode = (self.use_graphs and B > 0 and len(tokens) == B and isinstance(want, str) and want == "last"
                  and all(len(t) == 1 for t in tokens))
        if decode:
            starts = [self.cache.length(s) for s in slots]
            key = (B,) + (_lengths_class or self.lengths_class([n + 1 for n in starts]))
            g = self._graphs.get(key)
            if g is None and self._eager_decodes.get(key, 0) >= 1:
                g = self._graphs[key] = _DecodeGraph(self, B, key[1], key[2])
            if g is not None:
                # the short way for the step that generation repeats: same checks, same layout
                # of the integers as build_step, no intermediate arrays
                toks = [t[0] for t in tokens]
                if min(toks) < 0 or max(toks) >= self.vocab_size:
                    bad = next(t for t in toks if t < 0 or t >= self.vocab_size)
                    raise ValueError(f"token id {bad} lies outside the vocabulary [0, {self.vocab_size})")
                ones = [1] * B
                self.cache.prepare(slots, ones)
                self.h2d_bytes += g.upload(toks, starts, slots)
                g.graph.replay()
                K.launch_count += g.launches
                self.cache.commit(slots, ones)
                return g.logits if _borrow else g.logits.clone()   # the graph's own buffer is overwritten by its next replay
            self._eager_decodes[key] = self._eager_decodes.get(key, 0) + 1
        packed, sizes, q_lens, kv_lens = self.build_step(slots, tokens, want)
        self.cache.prepare(slots, q_lens)
        if self._staging is not None:
            dev = self._staging.upload(packed)
        else:
            dev = torch.from_numpy(packed).to(self.device)
        self.h2d_bytes += packed.nbytes
        st = self.step_state(dev, sizes, q_lens, kv_lens, _lengths_class)
        x = self.model.forward(st, self.cache)
        self.cache.commit(slots, q_lens)
        if sizes[2] == 0:
            return None
        return self.model.logits(x, st.want_rows)
