"""The schedules the measurements run, against the plain implementation in 32-bit and in
bfloat16: contexts of 4,000 to 8,700 positions (llama3 rope scaling with the real models'
constants), a batch of 64 unequal sequences through the packed prompt step and the captured
single-token steps with sequences leaving and a second batch taking their slots, and steps that
mix sequences in the middle of decoding with fresh prompts and with prompt portions."""
import pytest
import torch

from gpu_helpers import assert_close_logits, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _runner(d, dtype, tokens, batch):
    from rustyllm_b200 import Runner
    r, info = Runner.from_path(d, dtype=dtype, max_cache_tokens=tokens, max_batch=batch)
    assert info.fp32_matrices == 0
    return r


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["F", "G"])
def test_a_long_prompt_whole_in_portions_and_decoding_across_a_page_edge(model_dirs, name, dtype):
    """4,200 prompt tokens whole and in portions of unequal size, then 64 single-token steps that
    cross position 4,224 (the edge between the 66th and the 67th page of the slot)."""
    d, cfg = model_dirs[name]
    toks = random_tokens(cfg["vocab_size"], 4264, 31)
    ref = plain_logits(d, toks)
    r = _runner(d, dtype, 64 * 140, 2)
    eng = r.engine
    places = [0, 1, 63, 64, 2047, 2048, 4095, 4096, 4199]
    s = eng.alloc_slot()
    whole = eng.step([s], [toks[:4200]], [places])
    assert_close_logits(whole, ref[places], dtype, f"{name} 4,200 tokens whole")
    eng.free_slot(s)
    s2 = eng.alloc_slot()
    rows, at = [], 0
    for n in (1000, 37, 2059, 1, 1103):
        rows.append(eng.step([s2], [toks[at:at + n]], [[0, n - 1]] if n > 1 else [[0]]))
        at += n
    assert at == 4200
    want = [0, 999, 1000, 1036, 1037, 3095, 3096, 3097, 4199]
    assert_close_logits(torch.cat(rows), ref[want], dtype, f"{name} 4,200 tokens in portions")
    dec = [eng.step([s2], [[t]], "last") for t in toks[4200:]]
    assert_close_logits(torch.cat(dec), ref[4200:], dtype, f"{name} single tokens from 4,200 to 4,263")
    eng.free_slot(s2)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["F", "G"])
def test_a_sequence_pushed_to_position_8700(model_dirs, name, dtype):
    """Beyond the original context of the rope scaling (8,192) and up to the last position the
    1B benchmark reaches (8,703): prompt in portions, logits at a handful of places, then single
    tokens; a short sequence decodes beside it so that the step is a batch of very unequal lengths."""
    d, cfg = model_dirs[name]
    V = cfg["vocab_size"]
    long, short = random_tokens(V, 8704, 41), random_tokens(V, 60, 42)
    ref_long, ref_short = plain_logits(d, long), plain_logits(d, short)
    r = _runner(d, dtype, 64 * 140, 2)
    eng = r.engine
    a, b = eng.alloc_slot(), eng.alloc_slot()
    rows, at = [], 0
    for n in (3000, 3000, 2660):
        rows.append(eng.step([a], [long[at:at + n]], [[0, n // 2, n - 1]]))
        at += n
    want = [0, 1500, 2999, 3000, 4500, 5999, 6000, 7330, 8659]
    assert_close_logits(torch.cat(rows), ref_long[want], dtype, f"{name} portions up to 8,660")
    eng.step([b], [short[:16]], None)
    got_a, got_b = [], []
    for i in range(44):
        out = eng.step([a, b], [[long[8660 + i]], [short[16 + i]]], "last")
        got_a.append(out[0:1]); got_b.append(out[1:2])
    assert_close_logits(torch.cat(got_a), ref_long[8660:8704], dtype, f"{name} single tokens to position 8,703")
    assert_close_logits(torch.cat(got_b), ref_short[16:60], dtype, f"{name} the short sequence beside it")
    eng.free_slot(a); eng.free_slot(b)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["F", "G"])
def test_one_sequence_decoding_across_the_long_context_mark(model_dirs, name, dtype):
    """A sequence alone, single tokens from position 6,100 to 6,199: up to ``kernels.LONG_CONTEXT``
    cached tokens its attention runs as one cluster of eight chunks, beyond as sixteen chunks and a
    combining kernel, each side with a captured step of its own."""
    from rustyllm_b200 import kernels
    assert 6100 < kernels.LONG_CONTEXT < 6190
    d, cfg = model_dirs[name]
    long = random_tokens(cfg["vocab_size"], 8704, 41)
    ref = plain_logits(d, long)
    r = _runner(d, dtype, 64 * 100, 1)
    eng = r.engine
    s = eng.alloc_slot()
    for at in range(0, 6100, 3050):
        eng.step([s], [long[at:at + 3050]], None)
    got = [eng.step([s], [[t]], "last") for t in long[6100:6200]]
    assert_close_logits(torch.cat(got), ref[6100:6200], dtype, f"{name} single tokens from 6,100 to 6,199")
    if eng.use_graphs:
        assert sorted(eng._graphs) == [(1, False, 0), (1, True, 0)]
    eng.free_slot(s)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,batch", [("F", 5), ("G", 16), ("F", 80), ("F", 160)])
def test_batches_of_equal_near_and_far_lengths_take_their_own_decode_steps(model_dirs, name, batch, dtype):
    """Batches by the class of their lengths - equal, near one another (the longest within 768 tokens
    of the mean), far (within 4,096, and no sequence more than a twentieth of all tokens) and the
    rest - decode through captured steps of their own: with equal chunks a sequence (a cluster, one
    kernel a layer) or whole sequences where that serves them, with chunks dealt by length and a
    combining kernel where not.  5 sequences have 8 chunks each, a cluster's size, so the near batch
    clusters too; 16 have 7, rounded to 4 in a cluster, which only a batch of equal lengths takes; 80
    sequences of two KV heads would be more clusters of two than the GPU holds at once, so equal and
    near ones run whole, a CTA a sequence and KV head; 160 are more whole sequences than the GPU
    holds at once and run whole, the longest first (one more launch a step, which orders them),
    far ones too."""
    from rustyllm_b200 import kernels
    d, cfg = model_dirs[name]
    V, layers, G, hd = cfg["vocab_size"], cfg["num_hidden_layers"], cfg["num_key_value_heads"], cfg["head_dim"]
    steps = 4
    batches = {0: [70 if batch > 100 else 300] * batch,
               1: [150 + (450 * i) // (batch - 1) for i in range(batch)],
               3: [2400] + [40 + i % 50 for i in range(batch - 1)]}
    if batch == 80:
        batches[2] = [260] * 76 + [1100] * 4
    if batch == 160:
        del batches[1]
        batches[2] = [150] * 77 + [1000] * 2 + [150] * 79 + [1000] * 2
    r = _runner(d, dtype, max(sum(-(-(n + steps) // 64) * 64 for n in lens) for lens in batches.values()), batch)
    eng = r.engine
    launches = {}
    for spread, lens in sorted(batches.items()):
        assert len(lens) == batch
        assert kernels.length_spread([n + 1 for n in lens]) == spread == kernels.length_spread([n + steps for n in lens])
        seqs = [random_tokens(V, n + steps, 50 * spread + i) for i, n in enumerate(lens)]
        refs = [plain_logits(d, q) for q in seqs]
        slots = [eng.alloc_slot() for _ in lens]
        first = eng.step(slots, [q[:n] for q, n in zip(seqs, lens)], "last")
        assert_close_logits(first, torch.stack([refs[b][n - 1] for b, n in enumerate(lens)]), dtype, f"{name} spread {spread}: prompts")
        for t in range(steps):
            before = kernels.launch_count
            out = eng.step(slots, [[q[n + t]] for q, n in zip(seqs, lens)], "last")
            launches[spread] = kernels.launch_count - before
            assert_close_logits(out, torch.stack([refs[b][n + t] for b, n in enumerate(lens)]), dtype,
                                f"{name} spread {spread}: single token {t}")
        for sl in slots:
            eng.free_slot(sl)
    r.cache.check()
    kernels.check_device_errors()
    if eng.use_graphs:
        assert sorted(eng._graphs) == sorted((batch, max(lens) > kernels.LONG_CONTEXT, spread) for spread, lens in batches.items())
    if dtype == "bfloat16":
        cluster = {spread: kernels.decode_cluster_size(batch, G, hd, False, spread) for spread in sorted(batches)}
        assert cluster == {5: {0: 8, 1: 8, 3: 0}, 16: {0: 4, 1: 0, 3: 0}, 80: {0: 1, 1: 1, 2: 0, 3: 0}, 160: {0: 1, 2: 1, 3: 0}}[batch]
        # dealt chunks: a plan a step and a combining kernel a layer more than a cluster or whole sequences,
        # which are put in order by one launch a step where they are more than the GPU holds at once
        ordered = 1 if kernels.decode_order_wanted(batch, G, hd) else 0
        assert ordered == (1 if batch == 160 else 0)
        assert launches == {c: launches[3] - (layers + 1 - ordered if cluster[c] else 0) for c in launches}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["F", "B"])
def test_a_batch_of_64_unequal_sequences_then_another_in_their_slots(model_dirs, name, dtype):
    """64 prompts of 1 to 600 tokens (B: to 244) in one packed step, ten single-token steps
    (captured once a batch size), sequences leaving after 1 to 10 of them, then a second batch of
    64 other lengths in the slots and pages the first gave back."""
    d, cfg = model_dirs[name]
    V, top = cfg["vocab_size"], min(600, cfg["max_position_embeddings"] - 12)
    r = _runner(d, dtype, 64 * (top // 64 + 2) * 64, 64)
    eng = r.engine
    g = torch.Generator().manual_seed(3)
    for batch_no in range(2):
        lens = (torch.randperm(top, generator=g)[:64] + 1).tolist()
        lens[batch_no * 7] = 1; lens[63 - batch_no] = top               # the extremes are always there
        steps_of = [(i * 7 + batch_no) % 10 + 1 for i in range(64)]      # single-token steps before sequence i leaves
        seqs = [random_tokens(V, n + k, 1000 * batch_no + i) for i, (n, k) in enumerate(zip(lens, steps_of))]
        slots = [eng.alloc_slot() for _ in range(64)]
        assert sorted(slots) == list(range(64))
        first = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "last")
        got = [[first[i:i + 1]] for i in range(64)]
        live, fed = list(range(64)), list(lens)
        while live:
            out = eng.step([slots[i] for i in live], [[seqs[i][fed[i]]] for i in live], "last")
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1]); fed[i] += 1
            for i in [i for i in live if fed[i] >= len(seqs[i])]:
                eng.free_slot(slots[i])
                live.remove(i)
        for i in range(64):
            assert_close_logits(torch.cat(got[i]), plain_logits(d, seqs[i])[lens[i] - 1:], dtype,
                                f"{name} batch {batch_no} sequence {i} ({lens[i]} + {steps_of[i]} tokens)")
        r.cache.check()
    assert r.cache.free_pages == r.cache.num_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "E", "H"])
def test_a_step_that_mixes_decoding_sequences_fresh_prompts_and_a_prompt_portion(model_dirs, name, dtype):
    """Three sequences in the middle of decoding (one token each), two fresh prompts and the
    second portion of a third, all in one step: what a generation loop that feeds long prompts
    in portions produces.  Every token's logits against the sequence run whole."""
    d, cfg = model_dirs[name]
    V = cfg["vocab_size"]
    seqs = [random_tokens(V, n, 500 + i) for i, n in enumerate([90, 20, 131, 70, 5, 150])]
    r = _runner(d, dtype, 64 * 24, 8)
    eng = r.engine
    slots = [eng.alloc_slot() for _ in seqs]
    # sequences 0-2: a prompt step, then two single-token steps of their own
    got = {i: [] for i in range(6)}
    cut = [80, 10, 128]
    out = eng.step(slots[:3], [seqs[i][:cut[i]] for i in range(3)], "all")
    o = 0
    for i in range(3):
        got[i].append(out[o:o + cut[i]]); o += cut[i]
    fed = cut + [0, 0, 0]
    for _ in range(2):
        out = eng.step(slots[:3], [[seqs[i][fed[i]]] for i in range(3)], "last")
        for i in range(3):
            got[i].append(out[i:i + 1]); fed[i] += 1
    # sequence 5: the first portion of its prompt
    got[5].append(eng.step([slots[5]], [seqs[5][:100]], "all")); fed[5] = 100
    # the mixed step
    feed = [[seqs[0][fed[0]]], [seqs[1][fed[1]]], [seqs[2][fed[2]]], seqs[3], seqs[4], seqs[5][100:]]
    out = eng.step(slots, feed, "all")
    o = 0
    for i, f in enumerate(feed):
        got[i].append(out[o:o + len(f)]); o += len(f); fed[i] += len(f)
    # and the decoding sequences go on alone afterwards
    while any(fed[i] < len(seqs[i]) for i in range(3)):
        live = [i for i in range(3) if fed[i] < len(seqs[i])]
        out = eng.step([slots[i] for i in live], [[seqs[i][fed[i]]] for i in live], "last")
        for row, i in enumerate(live):
            got[i].append(out[row:row + 1]); fed[i] += 1
    for i, s in enumerate(seqs):
        assert_close_logits(torch.cat(got[i]), plain_logits(d, s), dtype, f"{name} mixed step, sequence {i}")
    for s in slots:
        eng.free_slot(s)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_with_the_prompt_step_in_portions(model_dirs, dtype):
    """Prompt steps of at most 1, 2 and 64 tokens (a portion then ends on a page's edge) generate
    the tokens of the prompt step run whole."""
    from rustyllm_b200 import GenerationOptions, SamplerConfig
    d, cfg = model_dirs["E"]
    V = cfg["vocab_size"]
    prompts = [random_tokens(V, n, 600 + n) for n in (64, 3, 130, 1)]
    r = _runner(d, dtype, 64 * 16, 4)
    opt = lambda n: GenerationOptions(max_tokens=6, sampler=SamplerConfig(temperature=0.7), seed=5, prefill_step_tokens=n)
    whole = [x.token_ids for x in r.generate(prompts, opt(16384))]
    for n in (64, 2, 1):
        got = [x.token_ids for x in r.generate(prompts, opt(n))]
        if dtype == "float32":
            assert got == whole, f"portions of {n}"
        else:
            # other kernels run for other step sizes; in bfloat16 a sampled token may differ where
            # two candidates' cumulative weights lie within rounding of the uniform number
            same = sum(a == b for a, b in zip(got, whole))
            assert same >= 3, f"portions of {n}: {got} vs {whole}"
    r.cache.check()
    assert r.cache.free_pages == r.cache.num_pages


def test_the_8b_shape_at_full_depth_in_32_bit_and_in_bfloat16():
    """Llama-3.1-8B's configuration, all 32 layers, random weights of one seed stored as bfloat16:
    the 32-bit engine and the bfloat16 engine on the same unequal batch and a few single-token
    steps.  No plain run at this size; the bound comes from the same two engines at 2 layers (where
    the plain implementation vouches for both, test_real_widths_gpu.py): rounding noise adds up
    like a random walk over the layers, so 32 layers may show sqrt(16) times the error of 2, and
    half as much again is allowed."""
    from rustyllm_b200 import Runner, kernels
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 4096,
           "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8,
           "head_dim": 128, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192}, "tie_word_embeddings": False}
    lens, steps = [70, 5, 131], 4
    seqs = [random_tokens(cfg["vocab_size"], n + steps, 80 + i) for i, n in enumerate(lens)]
    err = {}
    for layers in (2, 32):
        got = {}
        for dtype in ("float32", "bfloat16"):
            r = Runner.from_config(cfg, seed=9, dtype=dtype, storage_dtype="bfloat16", num_layers=layers,
                                   max_cache_tokens=64 * 12, max_batch=4)
            eng = r.engine
            slots = [eng.alloc_slot() for _ in lens]
            rows = [eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "last")]
            for t in range(steps):
                rows.append(eng.step(slots, [[s[n + t]] for s, n in zip(seqs, lens)], "last"))
            kernels.check_device_errors()
            got[dtype] = torch.cat(rows).double().cpu()
            del r, eng
            torch.cuda.empty_cache()
        exact = got["float32"]
        assert torch.isfinite(got["bfloat16"]).all() and torch.isfinite(exact).all()
        e = (got["bfloat16"] - exact).abs() / exact.pow(2).mean(-1, keepdim=True).sqrt()
        err[layers] = (e.pow(2).mean().sqrt().item(), e.max().item())
    print(f"8B shape, bf16 against 32-bit engine, rms / worst error of a row's scale: 2 layers {err[2]}, 32 layers {err[32]}")
    assert 1e-3 < err[2][0] < 3e-2, f"2 layers: rms error {err[2][0]:.2e} is not what this test was sized for"
    assert err[32][0] <= 1.5 * 4.0 * err[2][0], f"32 layers: rms {err[32][0]:.2e} against {err[2][0]:.2e} at 2 layers"
    assert err[32][1] <= 6.5 * 1.5 * 4.0 * err[2][0], f"32 layers: worst {err[32][1]:.2e}"
