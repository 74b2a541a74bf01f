"""The engine against the plain implementation, in 32-bit and in bfloat16: whole
requests, the last 32 tokens one by one, batches of unequal lengths whose shorter
requests end earlier with slots used again, long decoding, first tokens."""
import pytest
import torch

from gpu_helpers import assert_close_logits, load_runner, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
CONFIGS = ["A", "B", "C", "D", "E", "H"]


def _vocab(cfg):
    return cfg["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_each_request_alone_and_whole(model_dirs, name, dtype):
    d, cfg = model_dirs[name]
    r = load_runner(d, dtype)
    for seed, n in enumerate([1, 2, 17, 64, 65, 100]):
        toks = random_tokens(_vocab(cfg), n, 100 + seed)
        s = r.engine.alloc_slot()
        got = r.engine.step([s], [toks], "all")
        r.engine.free_slot(s)
        assert_close_logits(got, plain_logits(d, toks), dtype, f"{name} whole n={n}")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_last_32_tokens_one_by_one(model_dirs, name, dtype):
    d, cfg = model_dirs[name]
    r = load_runner(d, dtype)
    for n in (33, 90, 128):
        if n > cfg["max_position_embeddings"]:
            continue
        toks = random_tokens(_vocab(cfg), n, 200 + n)
        ref = plain_logits(d, toks)
        s = r.engine.alloc_slot()
        head = r.engine.step([s], [toks[:n - 32]], "all")
        rows = [head]
        for t in toks[n - 32:]:
            rows.append(r.engine.step([s], [[t]], "last"))
        r.engine.free_slot(s)
        assert_close_logits(torch.cat(rows), ref, dtype, f"{name} last-32 n={n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_unequal_batches_one_after_another_reuse_slots(model_dirs, name, dtype):
    """Two batches through a cache that only just holds one of them: the second batch
    gets the slots and pages the first gave back (with its stale contents)."""
    d, cfg = model_dirs[name]
    from rustyllm_b200 import Runner
    r, _ = Runner.from_path(d, dtype=dtype, max_cache_tokens=64 * 6, max_batch=4)
    eng = r.engine
    V = _vocab(cfg)
    for batch_no, (lens, total) in enumerate([([5, 70, 17, 1], [13, 100, 17, 30]),
                                              ([64, 3, 40], [66, 90, 41])]):
        seqs = [random_tokens(V, t, 300 + 10 * batch_no + i) for i, t in enumerate(total)]
        slots = [eng.alloc_slot() for _ in seqs]
        if batch_no == 1:
            assert sorted(slots) == [0, 1, 2], "slots of the first batch are used again"
        got = [[] for _ in seqs]
        out = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        o = 0
        for i, n in enumerate(lens):
            got[i].append(out[o:o + n]); o += n
        fed = list(lens)
        live = [i for i in range(len(seqs)) if fed[i] < total[i]]
        for i in range(len(seqs)):
            if i not in live:
                eng.free_slot(slots[i])
        while live:
            out = eng.step([slots[i] for i in live], [[seqs[i][fed[i]]] for i in live], "last")
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1]); fed[i] += 1
            done = [i for i in live if fed[i] >= total[i]]
            for i in done:
                eng.free_slot(slots[i])          # ends earlier: leaves the batch
            live = [i for i in live if i not in done]
        for i, s in enumerate(seqs):
            assert_close_logits(torch.cat(got[i]), plain_logits(d, s), dtype, f"{name} batch {batch_no} seq {i}")
        r.cache.check()
    assert r.cache.free_pages == r.cache.num_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D", "E"])
def test_long_decoding_across_pages(model_dirs, name, dtype):
    d, cfg = model_dirs[name]
    r = load_runner(d, dtype)
    toks = random_tokens(_vocab(cfg), 300, 7)
    ref = plain_logits(d, toks)
    s = r.engine.alloc_slot()
    rows = [r.engine.step([s], [toks[:3]], "all")]
    for t in toks[3:]:
        rows.append(r.engine.step([s], [[t]], "last"))
    r.engine.free_slot(s)
    assert_close_logits(torch.cat(rows), ref, dtype, f"{name} long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    d, cfg = model_dirs[name]
    r = load_runner(d, dtype)
    toks = random_tokens(_vocab(cfg), 4, 9)
    ref = plain_logits(d, toks)
    s = r.engine.alloc_slot()
    rows = [r.engine.step([s], [[t]], "last") for t in toks]     # position 0 is a step of its own
    r.engine.free_slot(s)
    assert_close_logits(torch.cat(rows), ref, dtype, f"{name} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunked_prompt_and_wanted_places(model_dirs, dtype):
    """A prompt cut into chunks of unequal size, and logits asked for at chosen places only."""
    d, cfg = model_dirs["B"]
    r = load_runner(d, dtype)
    toks = random_tokens(_vocab(cfg), 150, 11)
    ref = plain_logits(d, toks)
    s = r.engine.alloc_slot()
    a = r.engine.step([s], [toks[:70]], [[0, 69]])
    assert r.engine.step([s], [toks[70:71]], None) is None
    b = r.engine.step([s], [toks[71:150]], [[3, 78]])
    r.engine.free_slot(s)
    assert_close_logits(torch.cat([a, b]), ref[[0, 69, 74, 149]], dtype, "B chunks")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_reused_slot_does_not_see_its_former_contents(model_dirs, dtype):
    d, cfg = model_dirs["A"]
    r = load_runner(d, dtype)
    long = random_tokens(_vocab(cfg), 120, 21)
    short = random_tokens(_vocab(cfg), 9, 22)
    s = r.engine.alloc_slot()
    r.engine.step([s], [long], None)
    r.engine.free_slot(s)
    s2 = r.engine.alloc_slot()
    assert s2 == s
    got = r.engine.step([s2], [short], "all")
    r.engine.free_slot(s2)
    assert_close_logits(got, plain_logits(d, short), dtype, "A reused slot")


def test_bad_requests_are_refused_before_anything_runs(model_dirs):
    d, cfg = model_dirs["A"]
    r = load_runner(d, "float32")
    s = r.engine.alloc_slot()
    with pytest.raises(ValueError, match="outside the vocabulary"):
        r.engine.step([s], [[1, 256]], "last")
    with pytest.raises(ValueError, match="wanted place"):
        r.engine.step([s], [[1, 2]], [[2]])
    from rustyllm_b200.cache.allocators import CacheFull
    with pytest.raises(CacheFull):
        r.engine.step([s], [[0] * 129], "last")       # max_position_embeddings is 128
    assert r.cache.length(s) == 0
    r.engine.free_slot(s)


@pytest.mark.parametrize("name", ["B", "C", "D", "E"])
def test_folded_norms_save_launches_and_give_the_norm_kernels_results(model_dirs, name, monkeypatch):
    """In a bf16 step of up to 64 tokens every RMSNorm between two matrix products rides in
    their epilogues; with that switched off the norm kernels run.  Same logits either way
    (to bf16 rounding), 2 * layers - 1 launches apart."""
    from rustyllm_b200 import kernels
    from rustyllm_b200.parts import linear
    d, cfg = model_dirs[name]
    toks = random_tokens(_vocab(cfg), 40, 7)
    ref = plain_logits(d, toks)
    out, launches = {}, {}
    for mode, limit in (("folded", linear.FOLD_NORMS_UP_TO), ("kernels", 0)):
        monkeypatch.setattr(linear, "FOLD_NORMS_UP_TO", limit)
        r = load_runner(d, "bfloat16")
        monkeypatch.setattr(type(r.model), "use_native", False)      # the Python parts read the limit; the native executor has its own
        s = r.engine.alloc_slot()
        before = kernels.launch_count
        out[mode] = r.engine.step([s], [toks], "all")
        launches[mode] = kernels.launch_count - before
        r.engine.free_slot(s)
        assert_close_logits(out[mode], ref, "bfloat16", f"{name} {mode}")
    assert launches["kernels"] - launches["folded"] == 2 * cfg["num_hidden_layers"] - 1
    assert not torch.equal(out["folded"], out["kernels"])      # the other order of roundings shows


@pytest.mark.parametrize("name", ["B", "C", "D", "E", "F", "H"])
def test_native_executor_and_python_parts_launch_the_same_chain(model_dirs, name, monkeypatch):
    """The step's launch chain in native code (csrc/decoder_forward.cu) against the Python parts:
    the same kernels with the same arguments, so the same bits - for a packed prompt step of
    unequal lengths, a step of few tokens (norms folded into the products), a mixed step and
    single-token steps, eager and captured."""
    from rustyllm_b200 import Runner, kernels
    d, cfg = model_dirs[name]
    V = _vocab(cfg)
    seqs = [random_tokens(V, n, 700 + i) for i, n in enumerate([150, 9, 70])]
    out = {}
    for mode in ("native", "python"):
        monkeypatch.setattr("rustyllm_b200.models.decoder.DecoderModel.use_native", mode == "native")
        r, _ = Runner.from_path(d, dtype="bfloat16", max_cache_tokens=64 * 12, max_batch=4)
        eng = r.engine
        assert (r.model.native_for(r.cache) is not None) == (mode == "native")
        slots = [eng.alloc_slot() for _ in seqs]
        before = kernels.launch_count
        got = [eng.step(slots, [s[:n] for s, n in zip(seqs, (140, 3, 64))], "all")]          # 207 tokens: norm kernels
        got.append(eng.step(slots[1:], [seqs[1][3:8], seqs[2][64:69]], "all"))               # 10 tokens: folded norms
        got.append(eng.step(slots, [seqs[0][140:149], seqs[1][8:9], seqs[2][69:70]], "last"))   # mixed
        for _ in range(3):                                                                    # eager, then captured
            got.append(eng.step([slots[0]], [[seqs[0][149]]], "last"))
            eng.cache.lengths[slots[0]] -= 1                                                  # feed the same position again
        out[mode] = (torch.cat(got), kernels.launch_count - before)
        for s in slots:
            eng.free_slot(s)
        kernels.check_device_errors()
    assert torch.equal(out["native"][0], out["python"][0])
    assert out["native"][1] == out["python"][1], "both count the same launches"
    ref = plain_logits(d, seqs[0])
    assert_close_logits(out["native"][0][:140], ref[:140], "bfloat16", f"{name} native prompt")
