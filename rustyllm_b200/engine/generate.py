"""The generation loop above the step function: batches of unequal prompts, stop
tokens, sequences that end earlier, and as many batches one after another as there
are requests.

Per sequence the order of events is the reference's (``generate_chat_stream``,
SimonWaldherr/RustyLLM src/runtime.rs:3266-3342): the first token is sampled from the prompt's
last logits; a sampled stop token ends the sequence and is neither emitted nor
counted (3305-3307); the token is emitted and counted; the sequence ends when
``max_tokens`` are out or the context is full (3336-3338); otherwise the token is
fed back for the next logits - so N tokens cost one prompt step and N-1 single-token
steps.  Stop *strings* of the reference (3312-3325) become stop sequences of token
ids here (no tokenizer in this library): a match at the tail of the output ends
the sequence and is cut from it.

The loop only needs ``alloc_slot / free_slot / step`` of an engine and ``sample`` of
a sampler, so its decisions are tested on the CPU against stand-ins.

Running ahead.  The host learns a step's tokens only after the device has sampled
them, and the device would wait meanwhile for the host to queue the next step.  Where
the engine has ``step_fed_from_device`` and the sampler ``sample_begin``, the loop
queues the next step - fed with the sampled ids where they lie on the device - before
it waits for the ids, whenever no live sequence can end for a reason the host knows
beforehand (its token count, its context).  A sequence that then turns out to have
drawn a stop token has run one step too many: its logits are dropped and its slot is
freed as usual, and the other sequences' rows are taken from that step.  Tokens,
finish reasons and the order of ``on_token`` calls are those of the plain loop.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..kernels import PAGE_SIZE
from ..sampling.config import SamplerConfig
from ..sampling.sampler import SequenceSamplingState


@dataclass
class GenerationOptions:
    """SimonWaldherr/RustyLLM src/runtime.rs:94-111, minus the text-side fields."""
    max_tokens: int = 256
    sampler: SamplerConfig = field(default_factory=SamplerConfig)
    seed: int = 0                       # 0: from the clock (src/runtime.rs:3205-3213)
    stop_token_ids: Sequence[int] = ()  # in addition to the model's end-of-sequence ids
    stop_sequences: Sequence[Sequence[int]] = ()
    ignore_eos: bool = False            # benchmarks: run to max_tokens
    max_context: Optional[int] = None   # cap of the context (reference: --max-context)
    run_ahead: bool = True              # queue a step before the host has read the previous one's tokens
    prefill_step_tokens: int = 16384    # most prompt tokens one step runs (bounds the step's activation memory)

    def validate(self) -> None:
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be greater than 0.")
        if self.max_context is not None and self.max_context <= 0:
            raise ValueError("--max-context must be greater than 0.")
        if self.prefill_step_tokens <= 0:
            raise ValueError("prefill_step_tokens must be greater than 0.")
        self.sampler.validate()
        for s in self.stop_sequences:
            if len(s) == 0:
                raise ValueError("a stop sequence must hold at least one token id")


@dataclass
class GenerationStats:
    """SimonWaldherr/RustyLLM src/runtime.rs:393-403; times in seconds."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_time: float = 0.0
    decode_time: float = 0.0
    total_time: float = 0.0
    cached_tokens: int = 0
    steps: int = 0


@dataclass
class GenerationResult:
    token_ids: List[int]
    stats: GenerationStats
    finish_reason: str = ""    # "stop" | "length" | "context" | "stop_sequence"


def _ends_with(seq: List[int], tail: Sequence[int]) -> bool:
    n = len(tail)
    return n <= len(seq) and seq[-n:] == list(tail)


def pages_for(prompt_len: int, max_tokens: int) -> int:
    """Cache pages one request can come to hold: its prompt plus all but the last of
    its generated tokens (the last one is never fed back)."""
    return -(-(prompt_len + max_tokens - 1) // PAGE_SIZE)


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, max_batch: int, free_pages: int,
                 max_seq_len: int) -> List[List[int]]:
    """Cut the requests, in order, into batches that fit the slots and the pages."""
    batches: List[List[int]] = []
    cur: List[int] = []
    cur_pages = 0
    for i, p in enumerate(prompt_lens):
        if p <= 0:
            raise ValueError(f"request {i}: No prompt provided.")
        if p > max_seq_len:
            raise ValueError(f"request {i}: prompt of {p} tokens exceeds the context of {max_seq_len}")
        need = pages_for(p, min(max_tokens, max_seq_len - p + 1))
        if need > free_pages:
            raise ValueError(f"request {i} alone needs {need} cache pages, the cache has {free_pages}")
        if cur and (len(cur) >= max_batch or cur_pages + need > free_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


def prompt_portions(prompt_lens: Sequence[int], step_tokens: int) -> List[List[tuple]]:
    """Cut the prompts of a batch, in order, into steps of at most ``step_tokens`` tokens.
    Each step is a list of ``(sequence, first token, one past the last token)``; a long prompt
    goes on in the next step where the last one left it, and short prompts share a step."""
    steps: List[List[tuple]] = []
    cur: List[tuple] = []
    room = step_tokens
    for i, n in enumerate(prompt_lens):
        at = 0
        while at < n:
            take = min(n - at, room)
            cur.append((i, at, at + take))
            at += take
            room -= take
            if room == 0:
                steps.append(cur)
                cur, room = [], step_tokens
    if cur:
        steps.append(cur)
    return steps


def run_prompts(engine, slots: Sequence[int], prompts: Sequence[Sequence[int]], step_tokens: int):
    """The prompts of a batch through the step function, in as few steps as ``step_tokens``
    allows; returns the logits at every prompt's last token, in the order of the batch.
    (The reference feeds a prompt in chunks too and takes logits from its last token only,
    ``prefill_prompt_tokens``, SimonWaldherr/RustyLLM src/runtime.rs:3368-3428.)"""
    steps = prompt_portions([len(p) for p in prompts], step_tokens)
    if len(steps) == 1:
        return engine.step(list(slots), [list(p) for p in prompts], "last")
    rows = [None] * len(prompts)
    for portions in steps:
        want = [[hi - lo - 1] if hi == len(prompts[i]) else [] for i, lo, hi in portions]
        logits = engine.step([slots[i] for i, _, _ in portions], [list(prompts[i][lo:hi]) for i, lo, hi in portions],
                             want if any(want) else None)
        r = 0
        for (i, _, _), w in zip(portions, want):
            if w:
                rows[i] = logits[r]
                r += 1
    return _stack_rows(rows)


def _stack_rows(rows):
    first = rows[0]
    if hasattr(first, "new_empty"):        # device tensors: one [B, V] tensor, as a single step returns
        import torch
        return torch.stack(list(rows))
    return list(rows)


def generate_batch(engine, sampler, prompts: Sequence[Sequence[int]], options: GenerationOptions,
                   seeds: Sequence[int], stop_ids: Sequence[int], max_seq_len: int,
                   on_token: Optional[Callable[[int, int], None]] = None,
                   sync: Callable[[], None] = lambda: None) -> List[GenerationResult]:
    """One batch: its prompts in one step (or, beyond ``options.prefill_step_tokens`` tokens, in
    several), then one token per live sequence per step."""
    B = len(prompts)
    t_start = time.perf_counter()
    stop = set(() if options.ignore_eos else stop_ids) | set(options.stop_token_ids)
    cache_len = [min(max_seq_len, len(p) + options.max_tokens + 1) for p in prompts]  # src/runtime.rs:3184-3185
    states = [SequenceSamplingState(options.sampler, seeds[i], prompts[i]) for i in range(B)]
    out: List[List[int]] = [[] for _ in range(B)]
    reason = [""] * B
    pos = [len(p) for p in prompts]
    slots: List[Optional[int]] = []
    # the logits of a step are sampled from before the next step runs: no copy of them is needed
    step = getattr(engine, "step_borrowed", engine.step)
    step_ahead = getattr(engine, "step_fed_from_device", None) if options.run_ahead else None
    sample_begin = getattr(sampler, "sample_begin", None)
    try:
        for _ in range(B):
            slots.append(engine.alloc_slot())
        logits = run_prompts(engine, slots, prompts, options.prefill_step_tokens)
        sync()
        t_prefill = time.perf_counter()
        steps = 1
        live = list(range(B))
        while live:
            ahead = None
            if (step_ahead is not None and sample_begin is not None
                    and all(len(out[i]) + 1 < options.max_tokens and pos[i] < cache_len[i] for i in live)):
                # only a stop token or a stop sequence can end a sequence now: run the next step at once
                pending = sample_begin(logits, [states[i] for i in live])
                ahead = step_ahead([slots[i] for i in live], pending.device_ids)
                toks = pending.wait()
            else:
                toks = sampler.sample(logits, [states[i] for i in live])
            nxt, feed, kept_rows = [], [], []
            for row, i in enumerate(live):
                tok = int(toks[row])
                if tok in stop:
                    reason[i] = "stop"
                else:
                    out[i].append(tok)
                    states[i].push(tok)
                    hit = next((s for s in options.stop_sequences if _ends_with(out[i], s)), None)
                    if hit is not None:
                        del out[i][len(out[i]) - len(hit):]
                        reason[i] = "stop_sequence"
                    else:
                        if on_token is not None:
                            on_token(i, tok)
                        if len(out[i]) >= options.max_tokens:
                            reason[i] = "length"
                        elif pos[i] >= cache_len[i]:
                            reason[i] = "context"
                if reason[i]:
                    engine.free_slot(slots[i])   # ends earlier: its slot and pages go back at once
                    slots[i] = None
                else:
                    nxt.append(i)
                    feed.append([tok])
                    kept_rows.append(row)
            ran = len(live)
            live = nxt
            if not live:
                break
            if ahead is None:
                logits = step([slots[i] for i in live], feed, "last")
            else:
                logits = ahead if len(live) == ran else ahead[kept_rows]
            for i in live:
                pos[i] += 1
            steps += 1
        sync()
        t_end = time.perf_counter()
    finally:
        for s in slots:
            if s is not None:
                engine.free_slot(s)
    results = []
    for i in range(B):
        results.append(GenerationResult(
            token_ids=out[i],
            stats=GenerationStats(prompt_tokens=len(prompts[i]), generated_tokens=len(out[i]),
                                  prefill_time=t_prefill - t_start, decode_time=t_end - t_prefill,
                                  total_time=t_end - t_start, cached_tokens=0, steps=steps),
            finish_reason=reason[i]))
    return results
