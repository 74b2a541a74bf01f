"""Decisions of the generation loop, against stand-ins for the engine and the sampler (no GPU)."""
import pytest
import torch

from rustyllm_b200.engine.generate import (GenerationOptions, generate_batch, pages_for, plan_batches,
                                           prompt_portions)
from rustyllm_b200.sampling.config import Rng, SamplerConfig


class ScriptedEngine:
    """Each sequence's next token is a function of (its prompt, how many tokens it has been fed)."""

    def __init__(self, script, max_slots=8):
        self.script = script
        self.free = list(range(max_slots))[::-1]
        self.held = {}
        self.calls = []

    def alloc_slot(self):
        s = self.free.pop()
        self.held[s] = []
        return s

    def free_slot(self, s):
        assert s in self.held, "slot freed twice"
        del self.held[s]
        self.free.append(s)

    def step(self, slots, tokens, want):
        self.calls.append((list(slots), [list(t) for t in tokens]))
        rows = []
        for b, (s, t) in enumerate(zip(slots, tokens)):
            self.held[s].extend(t)
            if want == "last" or (want is not None and want[b] == [len(t) - 1]):
                rows.append(self.script(self.held[s]))
            else:
                assert want is None or want[b] == [], "a prompt portion wants its last token or nothing"
        return torch.tensor(rows) if rows else None


class PickSampler:
    def sample(self, logits, states):
        for st in states:
            if not st.config.is_greedy:
                st.rng.next_f32()
        return [int(x) for x in logits.tolist()]


class AheadEngine(ScriptedEngine):
    """Also takes a step whose tokens it is handed as a tensor (the device's copy of the ids)."""

    def __init__(self, script, max_slots=8):
        super().__init__(script, max_slots)
        self.ahead_calls = 0

    def step_fed_from_device(self, slots, token_ids):
        if self.ahead_calls == 0:          # like the engine before it has captured a step
            self.ahead_calls = 1
            return None
        self.ahead_calls += 1
        return self.step(slots, [[int(t)] for t in token_ids.tolist()], "last")


class Pending:
    def __init__(self, ids):
        self.device_ids = torch.tensor(ids, dtype=torch.int32)
        self.waited = False

    def wait(self):
        self.waited = True
        return self.device_ids.tolist()


class AheadSampler(PickSampler):
    def sample_begin(self, logits, states):
        return Pending(self.sample(logits, states))


def run(script, prompts, **opt):
    eng = ScriptedEngine(script)
    stop_ids = opt.pop("eos", (99,))
    max_seq = opt.pop("max_seq_len", 1000)
    opts = GenerationOptions(sampler=SamplerConfig.greedy(), **opt)
    opts.validate()
    seen = []
    res = generate_batch(eng, PickSampler(), prompts, opts, [1] * len(prompts), stop_ids, max_seq,
                         on_token=lambda i, t: seen.append((i, t)))
    assert eng.held == {}, "every slot goes back"
    return eng, res, seen


def test_first_token_comes_from_the_prompt_step_and_the_last_is_not_fed_back():
    eng, res, _ = run(lambda held: len(held), [[5, 6, 7]], max_tokens=4)
    assert res[0].token_ids == [3, 4, 5, 6] and res[0].finish_reason == "length"
    # 1 prompt step + 3 single-token steps for 4 tokens
    assert len(eng.calls) == 4 and eng.calls[0][1] == [[5, 6, 7]] and eng.calls[-1][1] == [[5]]
    assert res[0].stats.prompt_tokens == 3 and res[0].stats.generated_tokens == 4 and res[0].stats.steps == 4


def test_stop_token_is_neither_emitted_nor_counted():
    eng, res, seen = run(lambda held: 99 if len(held) == 5 else 10 + len(held), [[1, 2, 3]], max_tokens=10)
    assert res[0].token_ids == [13, 14] and res[0].finish_reason == "stop"
    assert seen == [(0, 13), (0, 14)]


def test_ignore_eos_and_extra_stop_ids():
    _, res, _ = run(lambda held: 99, [[1]], max_tokens=3, ignore_eos=True)
    assert res[0].token_ids == [99, 99, 99]
    _, res, _ = run(lambda held: 42, [[1]], max_tokens=3, stop_token_ids=(42,))
    assert res[0].token_ids == [] and res[0].finish_reason == "stop"


def test_shorter_sequences_leave_the_batch_and_the_others_go_on():
    # sequence with prompt [p] stops after p tokens
    def script(held):
        p = held[0]
        return 99 if len(held) - 1 >= p else 50
    eng, res, _ = run(script, [[3], [1], [2]], max_tokens=10)
    assert [r.token_ids for r in res] == [[50, 50, 50], [50], [50, 50]]
    sizes = [len(c[0]) for c in eng.calls]
    assert sizes == [3, 3, 2, 1]
    # freed at once: the slot of the shortest one is free while the others run
    assert all(r.finish_reason == "stop" for r in res)


def test_stop_sequence_of_ids_is_cut_from_the_output():
    _, res, seen = run(lambda held: len(held), [[0, 0]], max_tokens=10, stop_sequences=[[4, 5]])
    assert res[0].token_ids == [2, 3] and res[0].finish_reason == "stop_sequence"
    assert (0, 5) not in seen


def test_context_limit_ends_a_sequence():
    # context of 5 positions, prompt of 3: positions 3 and 4 can still be written
    eng, res, _ = run(lambda held: 7, [[1, 2, 3]], max_tokens=10, max_seq_len=5)
    assert res[0].finish_reason == "context"
    assert res[0].token_ids == [7, 7, 7]
    assert sum(len(t[0]) for _, t in eng.calls) == 5


def test_prompts_are_cut_into_steps_of_bounded_size():
    assert prompt_portions([5, 3], 100) == [[(0, 0, 5), (1, 0, 3)]]
    assert prompt_portions([5, 3], 4) == [[(0, 0, 4)], [(0, 4, 5), (1, 0, 3)]]
    assert prompt_portions([2, 7, 1], 3) == [[(0, 0, 2), (1, 0, 1)], [(1, 1, 4)], [(1, 4, 7)], [(2, 0, 1)]]
    for lens, n in (([64, 130, 1], 64), ([9, 9, 9], 1), ([1], 5)):
        steps = prompt_portions(lens, n)
        assert all(0 < sum(hi - lo for _, lo, hi in st) <= n for st in steps)
        for i, total in enumerate(lens):      # every token once, in order
            mine = [(lo, hi) for st in steps for j, lo, hi in st if j == i]
            assert mine[0][0] == 0 and mine[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(mine, mine[1:]))


@pytest.mark.parametrize("step_tokens", [1, 2, 3, 64])
def test_a_prompt_step_in_portions_changes_nothing(step_tokens):
    script = lambda held: 99 if len(held) >= 9 else sum(held) % 50
    prompts = [[5, 6, 7], [1], [2, 3, 4, 5, 6], [8, 8]]
    _, whole, seen_whole = run(script, prompts, max_tokens=6)
    eng, res, seen = run(script, prompts, max_tokens=6, prefill_step_tokens=step_tokens)
    assert [r.token_ids for r in res] == [r.token_ids for r in whole]
    assert [r.finish_reason for r in res] == [r.finish_reason for r in whole] and seen == seen_whole
    fed = [sum(len(t) for t in c[1]) for c in eng.calls]
    n_prompt_steps = -(-sum(len(p) for p in prompts) // step_tokens) if step_tokens < 11 else 1
    assert all(f <= max(step_tokens, len(prompts)) for f in fed[:n_prompt_steps])
    with pytest.raises(ValueError, match="prefill_step_tokens"):
        GenerationOptions(prefill_step_tokens=0).validate()


SCENARIOS = [
    (lambda held: len(held), [[5, 6, 7]], dict(max_tokens=4)),
    (lambda held: 99 if len(held) == 5 else 10 + len(held), [[1, 2, 3]], dict(max_tokens=10)),
    (lambda held: 99 if len(held) - 1 >= held[0] else 50, [[3], [1], [2], [7], [5]], dict(max_tokens=6)),
    (lambda held: 99 if len(held) - 1 >= held[0] else 50, [[6], [2], [9], [4]], dict(max_tokens=30)),
    (lambda held: len(held), [[0, 0], [0]], dict(max_tokens=10, stop_sequences=[[4, 5]])),
    (lambda held: 7, [[1, 2, 3], [1]], dict(max_tokens=10, max_seq_len=5)),
    (lambda held: 42, [[1]], dict(max_tokens=3, stop_token_ids=(42,))),
]


@pytest.mark.parametrize("case", range(len(SCENARIOS)))
def test_running_ahead_changes_no_token_reason_or_callback(case):
    script, prompts, opt = SCENARIOS[case]
    _, plain, seen_plain = run(script, prompts, **dict(opt))
    opt = dict(opt)
    stop_ids = opt.pop("eos", (99,))
    max_seq = opt.pop("max_seq_len", 1000)
    opts = GenerationOptions(sampler=SamplerConfig(temperature=0.5), **opt)
    eng, seen = AheadEngine(script), []
    res = generate_batch(eng, AheadSampler(), prompts, opts, [1] * len(prompts), stop_ids, max_seq,
                         on_token=lambda i, t: seen.append((i, t)))
    assert eng.held == {}, "every slot goes back, none twice"
    assert [r.token_ids for r in res] == [r.token_ids for r in plain]
    assert [r.finish_reason for r in res] == [r.finish_reason for r in plain]
    assert seen == seen_plain
    # and with running ahead switched off the engine is never asked for it
    opts.run_ahead = False
    eng2 = AheadEngine(script)
    res2 = generate_batch(eng2, AheadSampler(), prompts, opts, [1] * len(prompts), stop_ids, max_seq)
    assert eng2.ahead_calls == 0 and [r.token_ids for r in res2] == [r.token_ids for r in plain]


def test_running_ahead_feeds_an_ended_sequence_once_more_and_no_further():
    # sequence [p] draws its stop token after p tokens; only a stop token is unknown beforehand
    script = lambda held: 99 if len(held) - 1 >= held[0] else 50
    eng = AheadEngine(script)
    opts = GenerationOptions(sampler=SamplerConfig.greedy(), max_tokens=30)
    res = generate_batch(eng, AheadSampler(), [[4], [2]], opts, [1, 1], (99,), 1000)
    assert [r.token_ids for r in res] == [[50] * 4, [50] * 2]
    sizes = [len(c[0]) for c in eng.calls]
    # prompt step; plain step (nothing captured yet); then steps run ahead: the one queued while
    # sequence 1 drew its stop token still holds it, the next does not
    assert sizes == [2, 2, 2, 2, 1, 1]
    assert eng.calls[3][1][1] == [99]          # the dropped step was fed the stop token itself
    assert eng.calls[5][1][0] == [99]          # and so was the last one, whose logits nobody reads
    assert eng.ahead_calls == 5


def test_options_are_validated_like_the_reference():
    with pytest.raises(ValueError, match="max_tokens"):
        GenerationOptions(max_tokens=0).validate()
    with pytest.raises(ValueError, match="top_p"):
        GenerationOptions(sampler=SamplerConfig(top_p=0.0)).validate()
    with pytest.raises(ValueError, match="min_p"):
        GenerationOptions(sampler=SamplerConfig(min_p=1.0)).validate()
    with pytest.raises(ValueError, match="repeat_penalty"):
        GenerationOptions(sampler=SamplerConfig(repeat_penalty=0.0)).validate()
    with pytest.raises(ValueError, match="temperature"):
        GenerationOptions(sampler=SamplerConfig(temperature=-1.0)).validate()
    # the device sorts at most 1,024 candidates: said before a generation starts, not in its middle
    with pytest.raises(ValueError, match="top_k must be at most 1024"):
        GenerationOptions(sampler=SamplerConfig(top_k=1025)).validate()
    GenerationOptions(sampler=SamplerConfig(top_k=1024)).validate()
    GenerationOptions(sampler=SamplerConfig(temperature=0.0, top_k=5000)).validate()    # greedy: no candidate set


def test_batches_are_cut_by_slots_and_by_pages():
    assert pages_for(64, 1) == 1 and pages_for(64, 2) == 2 and pages_for(1, 64) == 1
    assert plan_batches([10] * 5, 8, max_batch=2, free_pages=100, max_seq_len=512) == [[0, 1], [2, 3], [4]]
    # each request can hold 100 + 29 tokens = 3 pages; 7 pages hold two of them
    assert plan_batches([100] * 5, 30, max_batch=8, free_pages=7, max_seq_len=512) == [[0, 1], [2, 3], [4]]
    with pytest.raises(ValueError, match="alone needs"):
        plan_batches([1000], 30, 8, free_pages=3, max_seq_len=4096)
    with pytest.raises(ValueError, match="exceeds the context"):
        plan_batches([600], 30, 8, free_pages=300, max_seq_len=512)
    with pytest.raises(ValueError, match="No prompt"):
        plan_batches([0], 30, 8, free_pages=300, max_seq_len=512)


def test_rng_matches_the_reference_generator():
    r = Rng(0)
    assert r.state == 0xDEADBEEFCAFE1337
    r = Rng(1)
    # xorshift64 (13, 7, 17) from state 1, computed by hand
    s = 1
    s ^= (s << 13) & (2**64 - 1); s ^= s >> 7; s ^= (s << 17) & (2**64 - 1)
    assert r.next_f32() == (s >> 40) / 2**24
    vals = [Rng(12345).next_f32() for _ in range(3)]
    assert vals[0] == vals[1] == vals[2] and 0.0 <= vals[0] < 1.0


def test_classes_of_a_batchs_lengths():
    """Equal (the longest within 16 tokens of the mean), near (within 768), far (within 4,096, and
    the longest no more than a twentieth of all tokens) and the rest; one sequence is always equal.  A step's launches may depend on the class, so captured steps are kept by it."""
    from rustyllm_b200 import kernels as K
    assert K.length_spread([1]) == 0 and K.length_spread([100000]) == 0
    assert K.length_spread([500, 500, 500]) == 0
    assert K.length_spread([516, 500, 500, 500]) == 0          # 12 above the mean of 504
    assert K.length_spread([532, 500]) == 0 and K.length_spread([534, 500]) == 1
    assert K.length_spread([2036, 500]) == 1 and K.length_spread([2038, 500]) == 3
    assert K.length_spread([1] * 63 + [781]) == 1 and K.length_spread([1] * 63 + [782]) == 3
    assert K.length_spread([8692, 500]) == 3                      # near enough, but nearly all tokens are its own
    assert K.length_spread([2000] + [1000] * 39) == 2 and K.length_spread([2000] + [900] * 39) == 3
    assert K.length_spread([5000] + [4000] * 60) == 2 and K.length_spread([8200] + [4000] * 60) == 3
