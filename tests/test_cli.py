"""The command line's options and the parts of it that need no GPU."""
import pytest

from rustyllm_b200 import cli


def test_reference_option_names_are_accepted():
    p = cli.build_parser()
    a = p.parse_args(["m", "-p", "1 2 3", "-n", "7", "-t", "0.5", "--top-p", "0.8", "--top-k", "5", "--min-p", "0.1",
                      "--repeat-penalty", "1.2", "--seed", "9", "--stop", "4", "--stop", "5,6", "--max-context", "64",
                      "--kv-cache-dtype", "bf16", "--bench-json", "--bench-runs", "2", "--bench-output",
                      "--kernel-bench-runs", "3", "-v"])
    o = cli._options(a)
    assert (o.max_tokens, o.seed, o.max_context) == (7, 9, 64)
    s = o.sampler
    assert (s.temperature, s.top_p, s.top_k, s.min_p, s.repeat_penalty) == (0.5, 0.8, 5, 0.1, 1.2)
    assert tuple(o.stop_token_ids) == (4,) and tuple(o.stop_sequences) == ((5, 6),)
    assert a.model_pos == "m" and a.bench_json and a.bench_runs == 2 and a.verbose


def test_defaults_and_reference_sampler():
    a = cli.build_parser().parse_args(["m", "--prompt", "1"])
    o = cli._options(a)
    assert o.max_tokens == 256 and o.sampler.temperature == 0.7           # the reference's
    assert (o.sampler.top_p, o.sampler.top_k, o.sampler.repeat_penalty) == (1.0, 0, 1.0)   # neutral filters
    o = cli._options(cli.build_parser().parse_args(["m", "--prompt", "1", "--reference-sampler"]))
    assert (o.sampler.top_p, o.sampler.top_k, o.sampler.repeat_penalty) == (0.9, 40, 1.1)


def test_bad_values_are_refused():
    with pytest.raises(ValueError, match="top_p"):
        cli._options(cli.build_parser().parse_args(["m", "--prompt", "1", "--top-p", "0"]))
    with pytest.raises(SystemExit):
        cli._ids("hello world")
    assert cli.main(["m"]) == 2                       # no prompt
    assert cli.main([]) == 2                          # no model


def test_inspect_and_list_tensors(model_dirs, capsys):
    d, _ = model_dirs["B"]
    assert cli.main([d, "--inspect", "--list-tensors"]) == 0
    out = capsys.readouterr().out
    assert "architecture: LlamaForCausalLM" in out and "compatibility: supported" in out
    assert "model.layers.2.mlp.down_proj.weight" in out and "hidden_size: 96" in out


def test_benchmark_prompt_lengths_and_other_spellings():
    import random
    p = cli.build_parser()
    a = p.parse_args(["m", "--json", "--runs", "2", "--batch", "16", "--prompt-len-range", "64,1024",
                      "--decode-tokens", "256", "--context", "2048", "--seed", "3"])
    assert a.bench_json and a.bench_runs == 2 and a.max_tokens == 256 and a.max_context == 2048
    lens = cli.synthetic_prompt_lengths(a, random.Random(3))
    assert len(lens) == 16 and all(64 <= n < 1024 for n in lens) and len(set(lens)) > 8
    assert lens == cli.synthetic_prompt_lengths(a, random.Random(3))        # seeded
    a = p.parse_args(["m", "--bench", "--batch", "3", "--prompt-len", "40"])
    assert cli.synthetic_prompt_lengths(a, random.Random(1)) == [40, 40, 40]
    for bad in ("5", "9,3", "0,4", "a,b"):
        with pytest.raises(SystemExit):
            cli.synthetic_prompt_lengths(p.parse_args(["m", "--bench", "--prompt-len-range", bad]), random.Random(1))
