"""Generation through the entry point against the plain implementation's loop."""
import numpy as np
import pytest
import torch

import plain_llama as P
from gpu_helpers import load_runner, random_tokens
from tiny_configs import TINY

pytestmark = pytest.mark.gpu


def _plain(d):
    return P.load_model_dir(d)


def test_greedy_batch_of_unequal_prompts_matches_the_plain_loop(model_dirs):
    """Tiny A: prompts of 5/11/17 tokens, 8 tokens each, greedy, 32-bit."""
    from rustyllm_b200 import GenerationOptions, SamplerConfig
    d, cfg = model_dirs["A"]
    r = load_runner(d, "float32")
    prompts = [random_tokens(256, n, 40 + n) for n in (5, 11, 17)]
    res = r.generate(prompts, GenerationOptions(max_tokens=8, sampler=SamplerConfig.greedy(), seed=1))
    pc, pw = _plain(d)
    for p, got in zip(prompts, res):
        want = P.generate(pc, pw, p, 8, temperature=0.0, stop_ids=[255])
        assert got.token_ids == want
        assert got.stats.prompt_tokens == len(p) and got.stats.generated_tokens == len(want)
    alone = r.generate(prompts[1], GenerationOptions(max_tokens=8, sampler=SamplerConfig.greedy(), seed=1))
    assert alone.token_ids == res[1].token_ids
    r.cache.check()
    assert r.cache.free_pages == r.cache.num_pages


def test_temperature_batch_matches_the_plain_sampler_with_the_same_seeds(model_dirs):
    """Tiny B: prompts of 1/7/23/40 tokens, 12 tokens each, temperature 0.8, fixed seeds, 32-bit."""
    from rustyllm_b200 import GenerationOptions, SamplerConfig
    d, cfg = model_dirs["B"]
    r = load_runner(d, "float32")
    prompts = [random_tokens(384, n, 50 + n) for n in (1, 7, 23, 40)]
    opts = GenerationOptions(max_tokens=12, sampler=SamplerConfig(temperature=0.8), seed=77)
    res = r.generate(prompts, opts)
    pc, pw = _plain(d)
    for i, (p, got) in enumerate(zip(prompts, res)):
        want = P.generate(pc, pw, p, 12, temperature=0.8, seed=77 + i, stop_ids=[382, 383])
        assert got.token_ids == want, f"sequence {i}"
    # the same sequence alone, with its own seed, samples the same tokens
    alone = r.generate(prompts[2], opts, seeds=[79])
    assert alone.token_ids == res[2].token_ids


def test_greedy_in_bfloat16_agrees_with_the_plain_loop_where_the_margin_is_clear(model_dirs):
    """In bf16 a near-tie between two logits may flip; compare up to the first step whose
    plain margin is smaller than the bf16 tolerance, and require at least a few steps."""
    from rustyllm_b200 import GenerationOptions, SamplerConfig
    d, cfg = model_dirs["C"]
    r = load_runner(d, "bfloat16")
    pc, pw = _plain(d)
    checked = 0
    for seed in range(4):
        p = random_tokens(307, 20 + seed, 60 + seed)
        got = r.generate(p, GenerationOptions(max_tokens=10, sampler=SamplerConfig.greedy(), seed=1)).token_ids
        seq = list(p)
        for t in got:
            logits = P.forward(pc, pw, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if (top2[0] - top2[1]) < 0.05 * logits.pow(2).mean().sqrt():
                break
            assert t == int(torch.argmax(logits))
            seq.append(t); checked += 1
    assert checked >= 10


def test_stop_tokens_and_batches_one_after_another(model_dirs):
    from rustyllm_b200 import GenerationOptions, Runner, SamplerConfig
    d, cfg = model_dirs["A"]
    r, info = Runner.from_path(d, dtype="float32", max_cache_tokens=64 * 3, max_batch=2)
    assert info.file_size_bytes > 0 and info.load_time > 0 and r.architecture() == "LlamaForCausalLM"
    prompts = [random_tokens(256, n, 70 + n) for n in (3, 30, 9, 14, 2)]
    greedy = GenerationOptions(max_tokens=6, sampler=SamplerConfig.greedy(), seed=1)
    res = r.generate(prompts, greedy)            # 5 requests through 2 slots: three batches
    assert [len(x.token_ids) for x in res] == [6] * 5
    # make the third token of request 1 a stop token: it ends there, the token is not emitted
    stop = res[1].token_ids[2]
    res2 = r.generate(prompts, GenerationOptions(max_tokens=6, sampler=SamplerConfig.greedy(), seed=1,
                                                 stop_token_ids=(stop,)))
    assert res2[1].token_ids == res[1].token_ids[:2] and res2[1].finish_reason == "stop"
    for a, b in zip(res, res2):
        cut = a.token_ids.index(stop) if stop in a.token_ids else len(a.token_ids)
        assert b.token_ids == a.token_ids[:cut]
    streamed = []
    one = r.generate_stream(prompts[0], greedy, streamed.append)
    assert streamed == one.token_ids == res[0].token_ids
    r.cache.check()
    assert r.cache.free_pages == r.cache.num_pages and r.cache.slots.free_count == 2


@pytest.mark.parametrize("name,cache_tokens,max_batch", [("A", 64 * 6, 3), ("B", 64 * 16, 5), ("B", 64 * 40, 16)])
def test_many_random_requests_through_a_small_cache(model_dirs, name, cache_tokens, max_batch):
    """Dozens of requests of random lengths and a random token budget through caches far too small
    for them at once: batches follow one another, sequences end early (tiny B stops at two ids),
    slots and pages are taken again.  Greedy in 32-bit, every sequence token for token as the
    plain loop makes it; the cache is whole afterwards."""
    import random
    from rustyllm_b200 import GenerationOptions, Runner, SamplerConfig
    d, cfg = model_dirs[name]
    pc, pw = _plain(d)
    V, maxpos = cfg["vocab_size"], cfg["max_position_embeddings"]
    eos = cfg.get("eos_token_id")
    stop = eos if isinstance(eos, list) else [eos]
    rng = random.Random(cache_tokens)
    r, _ = Runner.from_path(d, dtype="float32", max_cache_tokens=cache_tokens, max_batch=max_batch)
    for _ in range(2):
        n, budget = rng.randrange(4, 24), rng.randrange(1, 28)
        prompts = [random_tokens(V, rng.randrange(1, min(maxpos - 30, cache_tokens // 2)), rng.randrange(1 << 30)) for _ in range(n)]
        res = r.generate(prompts, GenerationOptions(max_tokens=budget, sampler=SamplerConfig.greedy(), seed=3))
        for p, got in zip(prompts, res):
            want = P.generate(pc, pw, p, min(budget, maxpos - len(p)), temperature=0.0, stop_ids=stop)
            assert got.token_ids == want, f"a prompt of {len(p)} tokens among {n} requests"
        r.cache.check()
        assert r.cache.free_pages == r.cache.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_of_the_host_generates_the_same_tokens(model_dirs, dtype):
    """The loop queues a step before it has read the previous step's tokens; with stop tokens
    that end sequences in the middle of a batch, filters and a repeat penalty, several batches
    one after another, the tokens are those of the loop that waits every step."""
    from rustyllm_b200 import GenerationOptions, Runner, SamplerConfig
    from rustyllm_b200 import kernels as K
    d, cfg = model_dirs["B"]
    r, _ = Runner.from_path(d, dtype=dtype, max_cache_tokens=64 * 8, max_batch=4)
    prompts = [random_tokens(384, n, 90 + n) for n in (4, 33, 9, 61, 2, 17, 26)]
    for sampler in (SamplerConfig.greedy(), SamplerConfig(temperature=0.9),
                    SamplerConfig(temperature=0.7, top_p=0.9, top_k=40, repeat_penalty=1.1)):
        base = GenerationOptions(max_tokens=24, sampler=sampler, seed=5, run_ahead=False)
        first = r.generate(prompts, base)
        # stop tokens taken from what was generated: some sequences end early, at different steps
        stops = tuple({first[1].token_ids[5], first[3].token_ids[11], first[5].token_ids[2]})
        for stop_ids in ((), stops):
            waits = r.generate(prompts, GenerationOptions(max_tokens=24, sampler=sampler, seed=5, run_ahead=False,
                                                          stop_token_ids=stop_ids))
            launches = K.launch_count
            ahead = r.generate(prompts, GenerationOptions(max_tokens=24, sampler=sampler, seed=5, run_ahead=True,
                                                          stop_token_ids=stop_ids))
            assert [x.token_ids for x in ahead] == [x.token_ids for x in waits]
            assert [x.finish_reason for x in ahead] == [x.finish_reason for x in waits]
            assert K.launch_count > launches
        assert any(x.finish_reason == "stop" for x in waits) and any(x.finish_reason == "length" for x in waits)
        r.cache.check()
        assert r.cache.free_pages == r.cache.num_pages and r.cache.slots.free_count == 4


def test_warm_up_captures_the_decode_steps_and_changes_no_token(model_dirs):
    from rustyllm_b200 import GenerationOptions, Runner, SamplerConfig
    d, cfg = model_dirs["A"]
    prompts = [random_tokens(256, n, 20 + n) for n in (6, 19, 3)]
    opts = GenerationOptions(max_tokens=7, sampler=SamplerConfig(temperature=0.8), seed=9)
    cold, _ = Runner.from_path(d, dtype="bfloat16", max_cache_tokens=64 * 6, max_batch=3)
    want = [r.token_ids for r in cold.generate(prompts, opts)]
    warm, _ = Runner.from_path(d, dtype="bfloat16", max_cache_tokens=64 * 6, max_batch=3)
    warm.warm_up([1, 2, 3, 3])
    assert sorted(warm.engine._graphs) == [(1, False, 0)] + [(n, False, spread) for n in (2, 3) for spread in (0, 1, 2, 3)]
    warm.cache.check()
    assert warm.cache.free_pages == warm.cache.num_pages and warm.cache.slots.free_count == 3
    assert [r.token_ids for r in warm.generate(prompts, opts)] == want


def test_random_weights_without_files_and_layer_override():
    from rustyllm_b200 import GenerationOptions, Runner, SamplerConfig
    r = Runner.from_config(TINY["B"]["config"], seed=3, dtype="bfloat16", max_cache_tokens=64 * 4, max_batch=2,
                           num_layers=2)
    assert r.config.num_hidden_layers == 2 and len(r.model.blocks) == 2
    out = r.generate([1, 2, 3], GenerationOptions(max_tokens=4, sampler=SamplerConfig.greedy(), ignore_eos=True))
    assert len(out.token_ids) == 4 and all(0 <= t < 384 for t in out.token_ids)
    r2 = Runner.from_config(TINY["B"]["config"], seed=3, dtype="bfloat16", max_cache_tokens=64 * 4, max_batch=2,
                            num_layers=2)
    assert r2.generate([1, 2, 3], GenerationOptions(max_tokens=4, sampler=SamplerConfig.greedy(), ignore_eos=True)).token_ids == out.token_ids


def test_command_line_generates_benchmarks_and_times_kernels(model_dirs, capsys, tmp_path):
    import json
    from rustyllm_b200 import cli
    d, cfg = model_dirs["D"]
    pc, pw = _plain(d)
    prompt = random_tokens(320, 9, 81)
    assert cli.main([d, "--dtype", "float32", "-p", " ".join(map(str, prompt)), "-n", "5", "-t", "0", "-v"]) == 0
    cap = capsys.readouterr()
    assert [int(t) for t in cap.out.split()] == P.generate(pc, pw, prompt, 5)
    assert "Prompt: 9 tokens" in cap.err and "Generated: 5 tokens" in cap.err and "Decode:" in cap.err
    pf = tmp_path / "prompts.txt"
    pf.write_text("1 2 3\n4,5,6,7\n")
    assert cli.main([d, "--prompt-file", str(pf), "-n", "3", "-t", "0", "--ignore-eos"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2 and all(len(l.split()) == 3 for l in lines)
    assert cli.main([d, "--bench-json", "--bench-runs", "2", "--batch", "3", "--prompt-len", "20", "-n", "4", "--seed", "5",
                     "--ignore-eos", "--bench-output"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["type"] == "rusty-llm.benchmark" and rep["architecture"] == "LlamaForCausalLM" and rep["runs"] == 2
    assert rep["results"][0]["prompt_tokens"] == 60 and rep["results"][0]["generated_tokens"] == 12
    assert rep["summary"]["aggregate_decode_tok_s"] > 0 and len(rep["results"][1]["token_ids"]) == 3
    assert cli.main([d, "--random", "--kernel-bench-json", "--kernel-bench-runs", "3"]) == 0
    rows = {r["name"]: r for r in json.loads(capsys.readouterr().out)["rows"]}
    for name in ("attn_norm.rms", "attn_qkv.fused", "ffn_gate_up.fused", "ffn_activation.silu_mul", "output", "attn_scan.ctx128"):
        assert rows[name]["avg_us"] > 0
