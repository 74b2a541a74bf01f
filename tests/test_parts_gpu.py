"""Each part alone, built through the registry from its parameters, against the plain formulas."""
import math

import pytest
import torch

import plain_llama as P
from gpu_helpers import BF16_REL_MAX, BF16_REL_MEAN

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _runtime(dtype):
    from rustyllm_b200.parts import Runtime
    return Runtime(DEV, dtype)


def _rand(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _step(positions, slots_per_token, cu, slots, kv_lens):
    from rustyllm_b200.engine.step import StepState
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    q_lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
    return StepState(len(positions), len(slots), i32([0] * len(positions)), i32(positions), i32(slots_per_token),
                     i32(cu), i32(slots), i32(kv_lens), i32([]), q_lens, kv_lens, max(q_lens), max(kv_lens),
                     all(q == 1 for q in q_lens))


def close(got, ref, dtype):
    """Error against the rms of the reference.  32-bit: at most 2e-5.  bf16: the bound
    used for logits throughout these tests (gpu_helpers): every stored intermediate
    carries a relative rounding error of up to 2^-8, a few dozen of them add up in
    each output, and the maximum is taken over thousands of outputs - at most 3e-2,
    and 6e-3 on average."""
    got, ref = got.double().cpu(), ref.double().cpu()
    rms = ref.pow(2).mean().sqrt().item()
    err = (got - ref).abs() / rms
    if dtype == torch.float32:
        assert err.max().item() <= 2e-5, f"max |diff| / rms = {err.max().item():.3e}"
    else:
        assert err.max().item() <= BF16_REL_MAX, f"max |diff| / rms = {err.max().item():.3e}"
        assert err.mean().item() <= BF16_REL_MEAN, f"mean |diff| / rms = {err.mean().item():.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from rustyllm_b200.config.spec import PartSpec
    from rustyllm_b200.parts import build_part
    n = build_part("norm", PartSpec("rms_norm", {"size": 100, "eps": 1e-4, "name": "n.weight"}), _runtime(dtype))
    assert n.param_specs()["weight"].sources[0].name == "n.weight" and n.param_specs()["weight"].role == "vector"
    n.bind({"weight": _rand(100, seed=1) + 1})
    x = _rand(6, 100, seed=2, scale=4)
    got = n.forward(x, dtype)
    assert got.dtype == dtype
    close(got, P.rms_norm(x.double().cpu(), n.weight.double().cpu(), 1e-4), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bias", [False, True])
def test_feed_forward_part(dtype, bias):
    from rustyllm_b200.config.spec import PartSpec
    from rustyllm_b200.parts import build_part
    d, I, M = 72, 200, 9
    ff = build_part("feed_forward", PartSpec("gated_mlp", {
        "hidden_size": d, "intermediate_size": I, "bias": bias,
        "names": {"gate": "g", "up": "u", "down": "dn"}}), _runtime(dtype))
    specs = ff.param_specs()
    assert [s.name for s in specs["wgu"].sources] == ["g.weight", "u.weight"] and specs["wgu"].shape == (2 * I, d)
    assert ("bgu" in specs) == bias
    # a bf16 run interleaves gate and up rows (the activation runs in the product's epilogue)
    assert specs["wgu"].layout == ("interleave" if dtype == torch.bfloat16 else "concat")
    w = {"wgu": _rand(2 * I, d, seed=3, scale=0.2, dtype=dtype), "wdown": _rand(d, I, seed=4, scale=0.2, dtype=dtype)}
    if bias:
        w.update(bgu=_rand(2 * I, seed=5, scale=0.1), bdown=_rand(d, seed=6, scale=0.1))
    bound = dict(w)
    if dtype == torch.bfloat16:      # what the loader would hand over: rows taken in turn
        for name in ("wgu", "bgu"):
            if name in w:
                t = torch.empty_like(w[name]); t[0::2] = w[name][:I]; t[1::2] = w[name][I:]; bound[name] = t
    ff.bind(bound)
    xn = _rand(M, d, seed=7, dtype=dtype)
    res = _rand(M, d, seed=8)
    out = res.clone()
    ff.forward(xn, out, None)
    x64 = xn.double().cpu()
    gu = x64 @ w["wgu"].double().cpu().T + (w["bgu"].double().cpu() if bias else 0)
    h = P.swiglu(gu[:, :I], gu[:, I:])
    ref = res.double().cpu() + h @ w["wdown"].double().cpu().T + (w["bdown"].double().cpu() if bias else 0)
    close(out, ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,bias,pairing", [(4, 2, 16, False, "half"), (3, 1, 32, True, "interleaved"), (6, 3, 48, False, "half")])
def test_attention_part_prompt_then_single_tokens(dtype, H, G, hd, bias, pairing):
    """The mixer alone with a cache of its own: two sequences' prompts in one step, then
    one token each; equal to plain causal attention over the whole sequences."""
    from rustyllm_b200.cache.sequence_cache import SequenceCache
    from rustyllm_b200.config.spec import PartSpec
    from rustyllm_b200.models.decoder import CacheView
    from rustyllm_b200.parts import build_part
    d = 56
    rope = PartSpec("rope", {"head_dim": hd, "rotary_dim": hd, "theta": 10000.0, "scaling": None, "pairing": pairing})
    att = build_part("mixer", PartSpec("gqa_attention", {
        "hidden_size": d, "num_heads": H, "num_kv_heads": G, "head_dim": hd, "bias": bias, "window": None,
        "position": rope, "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}), _runtime(dtype))
    need = att.kv_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (G, hd, None) and att.state_need() is None
    # weights scaled so that scores are of order one (a softmax that is not razor sharp:
    # with scores of 20 and more, bf16 rounding of q and k alone would move the result)
    w = {"wqkv": _rand((H + 2 * G) * hd, d, seed=1, scale=0.12, dtype=dtype), "wo": _rand(d, H * hd, seed=2, scale=0.3, dtype=dtype)}
    if bias:
        w.update(bqkv=_rand((H + 2 * G) * hd, seed=3, scale=0.2), bo=_rand(d, seed=4, scale=0.2))
    att.bind(w)
    cache = SequenceCache([need], [None], 64 * 6, dtype, DEV, max_slots=3)
    s0, s1 = cache.alloc_slot(), cache.alloc_slot()
    lens = [70, 9]
    xs = [_rand(n + 2, d, seed=10 + i, dtype=dtype) for i, n in enumerate(lens)]   # prompt + 2 more tokens each
    view = CacheView(cache.groups[0], 0, None, True)

    def run(chunks, starts):
        slots = [s0, s1]
        counts = [c.shape[0] for c in chunks]
        cache.prepare(slots, counts)
        pos, sot, cu = [], [], [0]
        for b, c in enumerate(chunks):
            pos += list(range(starts[b], starts[b] + c.shape[0])); sot += [slots[b]] * c.shape[0]; cu.append(len(pos))
        st = _step(pos, sot, cu, slots, [starts[b] + counts[b] for b in range(2)])
        res = torch.zeros(len(pos), d, device=DEV)
        att.forward(torch.cat(chunks), res, st, view)
        cache.commit(slots, counts)
        return [res[cu[b]:cu[b + 1]] for b in range(2)]

    got = [[], []]
    for b, o in enumerate(run([xs[0][:70], xs[1][:9]], [0, 0])):
        got[b].append(o)
    for t in range(2):
        for b, o in enumerate(run([xs[0][70 + t:71 + t], xs[1][9 + t:10 + t]], [70 + t, 9 + t])):
            got[b].append(o)
    inv = att.position.inv_freq.cpu()
    for b in range(2):
        x = xs[b].double().cpu()
        T = x.shape[0]
        qkv = x @ w["wqkv"].double().cpu().T + (w["bqkv"].double().cpu() if bias else 0)
        q, k, v = qkv[:, :H * hd].view(T, H, hd), qkv[:, H * hd:(H + G) * hd].view(T, G, hd), qkv[:, (H + G) * hd:].view(T, G, hd)
        sin, cos = P.rope_angles(torch.arange(T), inv)
        f = P.apply_rope_half if pairing == "half" else P.apply_rope_interleaved
        a = P.causal_attention(f(q, sin, cos), f(k, sin, cos), v).reshape(T, H * hd)
        ref = a @ w["wo"].double().cpu().T + (w["bo"].double().cpu() if bias else 0)
        close(torch.cat(got[b]), ref, dtype)


def test_rope_part_tables():
    from rustyllm_b200.config.spec import PartSpec
    from rustyllm_b200.parts import build_part
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    r = build_part("position", PartSpec("rope", {"head_dim": 32, "rotary_dim": 32, "theta": 500000.0, "scaling": sc,
                                                   "pairing": "half"}), _runtime(torch.float32))
    assert torch.equal(r.inv_freq.cpu(), P.rope_inv_freq(500000.0, 32, sc))
    n = build_part("position", PartSpec("none", {"head_dim": 32}), _runtime(torch.float32))
    assert n.rotary_dim == 0
    with pytest.raises(ValueError, match="pairing"):
        build_part("position", PartSpec("rope", {"head_dim": 8, "rotary_dim": 8, "theta": 1e4, "pairing": "odd"}),
                   _runtime(torch.float32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from rustyllm_b200.config.spec import PartSpec
    from rustyllm_b200.parts import build_part
    rt = _runtime(dtype)
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 307, "hidden_size": 40, "name": "e"}), rt)
    head = build_part("head", PartSpec("lm_head", {"vocab_size": 307, "hidden_size": 40, "name": "h", "tied_to": "embedding.weight"}), rt)
    assert head.param_specs()["weight"].alias_of == "embedding.weight"
    table = _rand(307, 40, seed=1, dtype=dtype)
    emb.bind({"weight": table}); head.bind({"weight": table})
    ids = torch.tensor([306, 0, 5], dtype=torch.int32, device=DEV)
    from types import SimpleNamespace
    x = emb.forward(SimpleNamespace(tokens=ids))         # an embedding part is handed the step
    assert x.dtype == torch.float32 and torch.equal(x, table[ids.long()].float())
    xn = _rand(4, 40, seed=2, dtype=dtype)
    logits = head.forward(xn)
    assert logits.dtype == torch.float32 and logits.shape == (4, 307)
    close(logits, xn.double().cpu() @ table.double().cpu().T, dtype)


def test_unknown_kind_is_reported_with_the_known_ones():
    from rustyllm_b200.config.spec import PartSpec
    from rustyllm_b200.parts import build_part
    with pytest.raises(KeyError, match="gated_mlp"):
        build_part("feed_forward", PartSpec("experts", {}), _runtime(torch.float32))
