"""The C++ float32 CPU baseline (rustyllm_b200/baseline) against the plain implementation: two
restatements of the reference's formulas by different routes (one token at a time against a cache
in C++ float32; whole sequences without a cache in float64) must agree to float32 rounding."""
import numpy as np
import pytest
import torch

import plain_llama as P
from rustyllm_b200 import baseline
from tiny_configs import TINY


@pytest.mark.parametrize("name", ["A", "B"])
def test_cpu_baseline_matches_the_plain_implementation(model_dirs, name):
    d, cfg = model_dirs[name]
    m = baseline.from_model_dir(d)
    pc, pw = P.load_model_dir(d)
    g = torch.Generator().manual_seed(11)
    for n in (1, 23, 70):
        toks = torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
        got = torch.from_numpy(m.logits_of(toks)).double()          # a new sequence starts again at position 0
        ref = P.forward(pc, pw, toks)
        rel = ((got - ref).abs() / ref.pow(2).mean(-1, keepdim=True).sqrt()).max().item()
        assert rel < 3e-5, f"{name}, {n} tokens: {rel:.2e}"
    m.close()


def test_rope_tables_agree_between_the_three_statements():
    """Product (parts/rope.py), plain implementation and the baseline's divisor form."""
    from rustyllm_b200.parts.rope import rope_inverse_frequencies
    cases = [(10000.0, 16, None), (500000.0, 32, TINY["B"]["config"]["rope_scaling"]),
             (500000.0, 128, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 8192}),
             (500000.0, 64, {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192})]
    for theta, hd, sc in cases:
        a = rope_inverse_frequencies(theta, hd, sc).double().numpy()
        b = baseline.rope_table(theta, hd, sc).astype(np.float64)
        c = np.asarray(P.rope_inv_freq(theta, hd, sc), dtype=np.float64)
        assert np.allclose(a, b, rtol=2e-7, atol=0) and np.allclose(a, c, rtol=2e-7, atol=0)
        if sc is not None:       # the scaling does something: low frequencies are divided by the factor
            plain = baseline.rope_table(theta, hd, None).astype(np.float64)
            assert np.isclose(b[-1], plain[-1] / sc["factor"], rtol=1e-6) and np.isclose(b[0], plain[0])


def test_timing_run_reports_what_it_ran():
    cfg = dict(TINY["A"]["config"], num_hidden_layers=6)
    r = baseline.time_decode(cfg, distinct_layers=2, context=5, tokens=3)
    assert r["layers"] == 6 and r["distinct_layers"] == 2 and r["tokens"] == 3 and r["tokens_per_s"] > 0
    assert "not a RustyLLM number" in r["what"]
