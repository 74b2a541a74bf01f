"""Configurations drawn at random, every size free: head sizes in steps of 16 and two that are
not (18, 50), any number of KV heads and of query heads to a KV head (1 to 17), hidden,
intermediate and vocabulary sizes that are odd, prime or powers of two, one to three layers,
every rope variant, tied or untied head, biases.  The engine in 32-bit and in bfloat16 against
the plain implementation: a prompt whole, single tokens behind it, a batch of unequal prompts
(137, 9, 70 and 1 tokens) and single tokens behind those.  Whatever kernel a shape falls to -
tensor cores, the any-shape kernels, folded or separate norms - the logits have to agree."""
import os
import random

import pytest
import torch

import plain_llama as P
from gpu_helpers import assert_close_logits, random_tokens

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    hd = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 192, 256, 18, 50])
    G = rng.choice([1, 1, 2, 3, 4, 5])
    m = rng.choice([1, 1, 2, 3, 4, 7, 8, 16, 17])
    while G * m > 40:
        m = max(1, m // 2)
    hidden = rng.choice([rng.randrange(24, 400), 8 * rng.randrange(4, 80), 64 * rng.randrange(1, 9)])
    inter = rng.choice([rng.randrange(17, 500), 8 * rng.randrange(4, 100), 128 * rng.randrange(1, 6)])
    vocab = rng.choice([rng.randrange(40, 2000), 128 * rng.randrange(1, 12)])
    scaling = None
    if rng.random() < 0.5:
        scaling = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]), "low_freq_factor": 1.0,
                   "high_freq_factor": rng.choice([2.0, 4.0]),
                   "original_max_position_embeddings": rng.choice([32, 64, 8192])}
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": vocab, "hidden_size": hidden,
            "intermediate_size": inter, "num_hidden_layers": rng.choice([1, 2, 3]), "num_attention_heads": G * m,
            "num_key_value_heads": G, "head_dim": hd, "max_position_embeddings": 512,
            "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-6]), "rope_theta": rng.choice([10000.0, 500000.0, 25000.0]),
            "rope_scaling": scaling, "tie_word_embeddings": rng.random() < 0.5,
            "attention_bias": rng.random() < 0.3, "mlp_bias": rng.random() < 0.3}


@pytest.mark.parametrize("seed", [0, 3, 5, 6, 10, 12, 13, 15, 19, 20, 24, 27, 29, 38, 57, 101])
def test_a_random_configuration_in_both_dtypes(tmp_path, seed):
    from rustyllm_b200 import Runner, kernels, write_random_model
    cfg = draw_config(seed)
    d = write_random_model(os.path.join(str(tmp_path), "m"), cfg, seed=seed, dtype="bfloat16", norm_noise=True)
    pcfg, w = P.load_model_dir(d)
    lens = [137, 9, 70, 1]
    seqs = [random_tokens(cfg["vocab_size"], n + 6, 100 * seed + i) for i, n in enumerate(lens)]
    refs = [P.forward(pcfg, w, s) for s in seqs]
    what = f"seed {seed}: " + ", ".join(f"{k}={cfg[k]}" for k in ("hidden_size", "intermediate_size", "vocab_size",
                                                                   "num_attention_heads", "num_key_value_heads", "head_dim"))
    for dtype in ("float32", "bfloat16"):
        r, _ = Runner.from_path(d, dtype=dtype, max_cache_tokens=64 * 16, max_batch=4)
        eng = r.engine
        s = eng.alloc_slot()
        whole = eng.step([s], [seqs[0][:137]], "all")
        assert_close_logits(whole, refs[0][:137], dtype, what + ": alone, whole")
        dec = [eng.step([s], [[t]], "last") for t in seqs[0][137:]]
        assert_close_logits(torch.cat(dec), refs[0][137:], dtype, what + ": alone, single tokens")
        eng.free_slot(s)
        slots = [eng.alloc_slot() for _ in lens]
        first = eng.step(slots, [q[:n] for q, n in zip(seqs, lens)], "last")
        assert_close_logits(first, torch.stack([refs[b][n - 1] for b, n in enumerate(lens)]), dtype, what + ": batch, prompts")
        for t in range(6):
            out = eng.step(slots, [[q[n + t]] for q, n in zip(seqs, lens)], "last")
            assert_close_logits(out, torch.stack([refs[b][n + t] for b, n in enumerate(lens)]), dtype,
                                what + f": batch, single token {t}")
        for sl in slots:
            eng.free_slot(sl)
        kernels.check_device_errors()
        r.cache.check()
