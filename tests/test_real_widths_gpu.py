"""Layers of real width (two of them, a small vocabulary), for the three Llama shapes the
measurements name: the 32-bit engine against the plain implementation, and the bfloat16
engine against what rounding every stored activation to bfloat16 does to the plain
implementation itself.

At these widths (products over 2048 to 14336 terms, 32 heads) the rounding noise of a
bfloat16 run is about 1 % of a logit row's scale, twice what the tiny configurations show,
so the bound is not a constant here: the plain implementation is run twice, exactly and
with its activations rounded to bfloat16 where a reduced-precision engine stores them, and
the engine may not be noisier than that by more than a quarter.  This carries the tiny
configurations' agreement to the shapes the tensor-core kernels were written for: products
split over clusters, rotation in the QKV epilogue, folded norms, tcgen05 and mma.sync
prefill attention with 32 heads, decode attention with 1 and 4 heads a KV head."""
import pytest
import torch

import plain_llama as P
from gpu_helpers import random_tokens

pytestmark = pytest.mark.gpu

SHAPES = {
    # Llama-3.1-8B layers: GQA 32/8, head 128, llama3 rope scaling
    "llama31_8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       intermediate_size=14336, rope_theta=500000.0, tie_word_embeddings=False,
                       rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}),
    # Llama-2-7B layers: MHA 32/32, head 128, intermediate 11008
    "llama2_7b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=32, head_dim=128,
                      intermediate_size=11008, rope_theta=10000.0, tie_word_embeddings=False),
    # Llama-3.2-1B layers: GQA 32/8, head 64, tied embeddings
    "llama32_1b": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                       intermediate_size=8192, rope_theta=500000.0, tie_word_embeddings=True,
                       rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}),
}


def _plain_weights(model, cfg):
    """The 32-bit engine's bound parameters under the checkpoint names the plain implementation reads."""
    H, G, hd, I = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    f = lambda t: t.detach().to("cpu", torch.float64)
    w = {"model.embed_tokens.weight": f(model.embedding.weight), "model.norm.weight": f(model.final_norm.weight)}
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = f(model.head.weight)
    for i, blk in enumerate(model.blocks):
        p = f"model.layers.{i}."
        qkv, gu = f(blk.mixer.wqkv), f(blk.feed_forward.wgu)          # rows: q, k, v / gate, up (32-bit run: not interleaved)
        w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"] = \
            qkv[:H * hd], qkv[H * hd:(H + G) * hd], qkv[(H + G) * hd:]
        w[p + "self_attn.o_proj.weight"] = f(blk.mixer.wo)
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = gu[:I], gu[I:]
        w[p + "mlp.down_proj.weight"] = f(blk.feed_forward.wdown)
        w[p + "input_layernorm.weight"] = f(blk.mixer_norm.weight)
        w[p + "post_attention_layernorm.weight"] = f(blk.feed_forward_norm.weight)
    return w


@pytest.mark.parametrize("name", list(SHAPES))
def test_engines_at_real_widths(name):
    from rustyllm_b200 import Runner, kernels
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=1536, num_hidden_layers=2,
               max_position_embeddings=1024, rms_norm_eps=1e-5, **SHAPES[name])
    lens, steps = [130, 40, 1], 6
    seqs = [random_tokens(cfg["vocab_size"], n + steps, 40 + i) for i, n in enumerate(lens)]
    got, weights = {}, None
    for dtype in ("float32", "bfloat16"):
        r = Runner.from_config(cfg, seed=5, dtype=dtype, storage_dtype="bfloat16", max_cache_tokens=64 * 16, max_batch=4)
        assert not r.model.blocks[0].feed_forward.interleaved or dtype == "bfloat16"
        if dtype == "float32":
            weights = _plain_weights(r.model, cfg)
        eng = r.engine
        slots = [eng.alloc_slot() for _ in lens]
        first = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")        # unequal prompts in one step
        per_seq, o = [], 0
        for n in lens:
            per_seq.append([first[o:o + n]]); o += n
        for t in range(steps):                                                     # then one token each
            out = eng.step(slots, [[s[n + t]] for s, n in zip(seqs, lens)], "last")
            for b in range(3):
                per_seq[b].append(out[b:b + 1])
        for s in slots:
            eng.free_slot(s)
        kernels.check_device_errors()
        got[dtype] = torch.cat([torch.cat(rows) for rows in per_seq])
        del r, eng
        torch.cuda.empty_cache()
    exact = torch.cat([P.forward(cfg, weights, s) for s in seqs])
    rounded = torch.cat([P.forward(cfg, weights, s, round_fn=P.bf16_round) for s in seqs])
    scale = exact.pow(2).mean(-1, keepdim=True).sqrt()
    # 32-bit engine: a float32 sum of K terms is off by about 2^-24 sqrt(K) of its scale (a random
    # walk of roundings), and 4 products a layer plus the head lie behind a logit; eight times that
    # covers the largest of a few hundred thousand logits.  (The constant of the tiny
    # configurations, 3e-5, is this expression at their widths.)
    k_max, depth = max(cfg["intermediate_size"], cfg["hidden_size"]), 4 * cfg["num_hidden_layers"] + 1
    f32_bound = 8 * 2.0 ** -24 * (k_max * depth) ** 0.5
    f32_err = ((got["float32"].double().cpu() - exact).abs() / scale).max().item()
    assert f32_err <= f32_bound, f"{name}: 32-bit engine against plain: max |diff| / rms(row) = {f32_err:.2e} > {f32_bound:.2e}"
    noise = ((rounded - exact) / scale).pow(2).mean().sqrt().item()        # what bf16 storage costs the plain implementation
    err = (got["bfloat16"].double().cpu() - exact).abs() / scale
    rms, worst = err.pow(2).mean().sqrt().item(), err.max().item()
    assert 2e-3 < noise < 3e-2, f"{name}: rounding noise of the plain implementation {noise:.2e} is not what this test was sized for"
    assert rms <= 1.25 * noise, f"{name}: bf16 engine rms error {rms:.2e} of a row's scale, rounding noise alone is {noise:.2e}"
    assert worst <= 6.5 * noise, f"{name}: bf16 engine worst error {worst:.2e}, rounding noise (rms) is {noise:.2e}"


def test_a_written_folder_and_a_drawn_model_of_one_seed_are_the_same_model(tmp_path):
    """Llama-3.1-8B's widths, two layers: the folder that ``write_random_model`` writes for a seed,
    loaded by name (concatenated Q/K/V, interleaved gate and up rows at an intermediate size of
    14,336), against the model ``Runner.from_config`` draws on the device for the same seed: the
    same tensors bit for bit, hence the same logits.  (The drawn model is held to the plain
    implementation above; this carries that to the loader at real widths.)"""
    from rustyllm_b200 import Runner, write_random_model
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=1536, num_hidden_layers=2,
               max_position_embeddings=1024, rms_norm_eps=1e-5, torch_dtype="bfloat16", **SHAPES["llama31_8b"])
    d = write_random_model(str(tmp_path / "m"), cfg, seed=5, dtype="bfloat16", device="cuda:0")
    loaded, info = Runner.from_path(d, dtype="bfloat16", max_cache_tokens=64 * 8, max_batch=2)
    drawn = Runner.from_config(cfg, seed=5, dtype="bfloat16", max_cache_tokens=64 * 8, max_batch=2)
    assert info.fp32_matrices == 0
    for a, b in zip(loaded.model.blocks, drawn.model.blocks):
        for name in ("wqkv", "wo"):
            assert torch.equal(getattr(a.mixer, name), getattr(b.mixer, name)), name
        for name in ("wgu", "wdown"):
            assert torch.equal(getattr(a.feed_forward, name), getattr(b.feed_forward, name)), name
    assert torch.equal(loaded.model.embedding.weight, drawn.model.embedding.weight)
    toks = random_tokens(cfg["vocab_size"], 70, 3)
    out = []
    for r in (loaded, drawn):
        s = r.engine.alloc_slot()
        out.append(r.engine.step([s], [toks], "all"))
        r.engine.free_slot(s)
    assert torch.equal(out[0], out[1])
