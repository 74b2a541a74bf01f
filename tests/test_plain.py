"""The plain implementation against the reference's own literal test vectors and
against itself (no GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P
from sampler_cases import CASES
from tiny_configs import TINY


def test_half_split_rope_literal():
    # SimonWaldherr/RustyLLM src/model.rs:1952-1965: q=[1,2,3,4], k=[5,6,7,8], inv=[pi/2, 0], pos=1
    inv = torch.tensor([math.pi / 2, 0.0], dtype=torch.float32)
    sin, cos = P.rope_angles(torch.tensor([1]), inv)
    q = P.apply_rope_half(torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=P.F64), sin, cos)[0, 0]
    k = P.apply_rope_half(torch.tensor([[[5.0, 6.0, 7.0, 8.0]]], dtype=P.F64), sin, cos)[0, 0]
    assert torch.allclose(q, torch.tensor([-3.0, 2.0, 1.0, 4.0], dtype=P.F64), atol=1e-5)
    assert abs(k[0] + 7.0) < 1e-5 and abs(k[2] - 5.0) < 1e-5


def test_inverse_frequencies():
    # src/model.rs:1945-1949: theta 10000, head 4 -> inv[0] = 1; inv[1] = 1/100
    inv = P.rope_inv_freq(10000.0, 4, None)
    assert abs(inv[0] - 1.0) < 1e-6 and abs(inv[1] - 0.01) < 1e-8
    sc = TINY["B"]["config"]["rope_scaling"]
    plain = P.rope_inv_freq(500000.0, 32, None)
    scaled = P.rope_inv_freq(500000.0, 32, sc)
    wavelen = 2 * math.pi / plain.double()
    hi, lo = 64 / 4.0, 64 / 1.0
    for i in range(16):
        if wavelen[i] < hi:
            assert scaled[i] == plain[i]
        elif wavelen[i] > lo:
            assert abs(scaled[i] - plain[i] / 8.0) < 1e-9
        else:
            assert plain[i] / 8.0 < scaled[i] < plain[i]
    assert (wavelen < hi).any() and (wavelen > lo).any() and ((wavelen >= hi) & (wavelen <= lo)).any()


def test_interleaved_equals_half_split_after_permuting_rows(model_dirs):
    """The reference's comment at src/model.rs:5520-5523: GGUF files permute q/k rows so
    that interleaved pairs reproduce the half-split model."""
    d, cfg = model_dirs["A"]
    cfgd, w = P.load_model_dir(d)
    hd, H, G = 16, 4, 2
    perm_head = torch.tensor([i // 2 + (i % 2) * (hd // 2) for i in range(hd)])   # new row 2i <- i, 2i+1 <- i + hd/2
    w2 = dict(w)
    for l in range(2):
        for name, heads in (("q_proj", H), ("k_proj", G)):
            key = f"model.layers.{l}.self_attn.{name}.weight"
            idx = torch.cat([h * hd + perm_head for h in range(heads)])
            w2[key] = w[key][idx]
    toks = [3, 77, 200, 5, 5, 91, 17]
    a = P.forward(cfgd, w, toks, pairing="half")
    b = P.forward(cfgd, w2, toks, pairing="interleaved")
    assert torch.allclose(a, b, atol=1e-12)


def test_rms_norm_and_swiglu_values():
    x = torch.tensor([[3.0, 4.0]], dtype=P.F64)
    y = P.rms_norm(x, torch.tensor([1.0, 2.0], dtype=P.F64), 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]], dtype=P.F64))
    g = torch.tensor([0.0, 1.0, -2.0], dtype=P.F64)
    u = torch.tensor([5.0, 2.0, 3.0], dtype=P.F64)
    want = torch.tensor([0.0, 2.0 / (1 + math.exp(-1.0)), -6.0 / (1 + math.exp(2.0))], dtype=P.F64)
    assert torch.allclose(P.swiglu(g, u), want)


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    T, H, G, hd = 6, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=P.F64) for n in (H, G, G))
    out = P.causal_attention(q, k, v)
    # position 0 sees only itself
    assert torch.allclose(out[0, 3], v[0, 1])
    # streaming softmax of the reference (src/model.rs:5807-5869) for one head and position
    h, pos, g = 2, 4, 1
    mx, den, acc = -math.inf, 0.0, torch.zeros(hd, dtype=P.F64)
    for t in range(pos + 1):
        s = float(q[pos, h] @ k[t, g]) / math.sqrt(hd)
        if s > mx:
            r = math.exp(mx - s) if math.isfinite(mx) else 0.0
            acc = acc * r + v[t, g]; den = den * r + 1.0; mx = s
        else:
            wgt = math.exp(s - mx); acc = acc + wgt * v[t, g]; den += wgt
    assert torch.allclose(out[pos, h], acc / den, atol=1e-12)
    # a window of 2 sees the last two positions only
    win = P.causal_attention(q, k, v, window=2)
    s = torch.tensor([float(q[3, 0] @ k[t, 0]) / math.sqrt(hd) for t in (2, 3)], dtype=P.F64)
    p = torch.softmax(s, 0)
    assert torch.allclose(win[3, 0], p[0] * v[2, 0] + p[1] * v[3, 0])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_later_tokens_do_not_change_earlier_logits(model_dirs, name):
    d, _ = model_dirs[name]
    cfg, w = P.load_model_dir(d)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg["vocab_size"], (12,), generator=g).tolist()
    full = P.forward(cfg, w, toks)
    part = P.forward(cfg, w, toks[:7])
    assert full.shape == (12, cfg["vocab_size"])
    assert torch.allclose(full[:7], part, atol=1e-12)
    assert torch.isfinite(full).all() and full.std() > 1e-3


def test_tied_head_uses_the_embedding(model_dirs):
    d, _ = model_dirs["B"]
    cfg, w = P.load_model_dir(d)
    assert "lm_head.weight" not in w and cfg["tie_word_embeddings"]
    hid = P.forward(cfg, w, [1, 2, 3], return_hidden=True)
    logits = P.forward(cfg, w, [1, 2, 3])
    xn = P.rms_norm(hid, w["model.norm.weight"], cfg["rms_norm_eps"])
    assert torch.allclose(logits, xn @ w["model.embed_tokens.weight"].T)


def test_rng_and_repeat_penalty_literals():
    # src/sampling.rs:365-383
    l = np.array([4.0, -4.0, 2.0], dtype=np.float32)
    P.apply_repeat_penalty(l, [0, 1], 2.0)
    assert l.tolist() == [2.0, -8.0, 2.0]
    l = np.array([1.0, 2.0], dtype=np.float32)
    P.apply_repeat_penalty(l, [5, 99], 2.0)
    assert l.tolist() == [1.0, 2.0]
    assert P.Rng(0).state == 0xDEADBEEFCAFE1337
    assert P.sample(np.zeros(0, dtype=np.float32), 0.7, P.Rng(7)) == 0   # 420-428


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_sampler_cases_of_the_reference(case):
    _, opt, seed, draws, logits, recent, allowed, must = case
    rng = P.Rng(seed)
    seen = set()
    for _ in range(draws):
        t = P.sample(np.array(logits, dtype=np.float32), opt["temperature"], rng, opt["top_k"], opt["top_p"],
                     opt["min_p"], opt["repeat_penalty"], recent)
        assert t in allowed
        seen.add(t)
    assert must <= seen


def test_temperature_sampling_follows_the_distribution():
    logits = np.array([0.0, math.log(3.0)], dtype=np.float32)
    rng = P.Rng(11)
    n = 4000
    ones = sum(P.sample(logits, 1.0, rng) for _ in range(n))
    assert abs(ones / n - 0.75) < 0.03


def test_greedy_generation_stops_at_a_stop_token(model_dirs):
    d, _ = model_dirs["A"]
    cfg, w = P.load_model_dir(d)
    out = P.generate(cfg, w, [1, 2, 3, 4, 5], max_tokens=6)
    assert len(out) == 6
    stopped = P.generate(cfg, w, [1, 2, 3, 4, 5], max_tokens=6, stop_ids=[out[2]])
    assert stopped == out[:2]
