"""Two more toy parts, registered from this test with no change to the framework's files:
a feed-forward that routes every token to one of several experts, and a position encoding
of its own (rotation with position-interpolated, learned-looking frequencies).  A toy
architecture puts them beside the framework's attention; the engine's logits are compared
with a float64 restatement written here, whole and token by token."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F64 = torch.float64


def _register():
    from rustyllm_b200.config.registry import register_architecture
    from rustyllm_b200.config.spec import LayerSpec, ModelSpec, ParamSource, ParamSpec, PartSpec
    from rustyllm_b200.parts import FeedForward, PositionEncoding, register_feed_forward, register_position
    from rustyllm_b200.parts.linear import OUT_ADD_F32, OUT_F32, linear

    @register_feed_forward("toy_top1_experts")
    class ToyTop1Experts(FeedForward):
        """x += p_e * W_out[e] relu(W_in[e] xn), e = the expert with the highest router logit,
        p_e its softmax probability over all experts.  Router logits and probabilities are
        32-bit; the experts' weights are two 3-D tensors."""
        graph_capturable = False          # tokens are grouped by expert on the host

        def __init__(self, runtime, hidden_size, intermediate_size, num_experts, name):
            self.runtime = runtime
            self.d, self.I, self.E, self.name = hidden_size, intermediate_size, num_experts, name

        def param_specs(self):
            n = self.name
            return {"router": ParamSpec((ParamSource(n + ".router", (self.E, self.d)),)),
                    "w_in": ParamSpec((ParamSource(n + ".w_in", (self.E, self.I, self.d)),)),
                    "w_out": ParamSpec((ParamSource(n + ".w_out", (self.E, self.d, self.I)),))}

        def forward(self, xn, residual, step):
            M = xn.shape[0]
            logits = torch.empty((M, self.E), dtype=torch.float32, device=xn.device)
            linear(xn, self.router, logits, OUT_F32)                   # the framework's own product
            prob = torch.softmax(logits, dim=-1)
            top = logits.argmax(dim=-1)
            for e in sorted(set(top.tolist())):
                rows = (top == e).nonzero().flatten()
                h = torch.empty((rows.numel(), self.I), dtype=torch.float32, device=xn.device)
                linear(xn[rows].contiguous(), self.w_in[e], h, OUT_F32)
                h = torch.relu(h).to(xn.dtype)
                part = torch.zeros((rows.numel(), self.d), dtype=torch.float32, device=xn.device)
                linear(h, self.w_out[e], part, OUT_ADD_F32)
                residual.index_add_(0, rows, part * prob[rows, e].unsqueeze(1))

    @register_position("toy_interpolated")
    class ToyInterpolatedRotation(PositionEncoding):
        """Rotation whose frequencies are not a geometric series: 1 / (1 + i)^2, divided by
        an interpolation factor.  The mixer only asks for inv_freq, rotary_dim, interleaved."""

        def __init__(self, runtime, head_dim, factor):
            self.head_dim = head_dim
            self.rotary_dim = head_dim
            self.interleaved = False
            self.inv_freq = torch.tensor([1.0 / ((1 + i) ** 2 * factor) for i in range(head_dim // 2)],
                                         dtype=torch.float32, device=runtime.device)

    def spec(cfg):
        d, hd, H, G = cfg["hidden_size"], cfg["head_dim"], cfg["heads"], cfg["kv"]
        def norm(n): return PartSpec("rms_norm", {"size": d, "eps": cfg["eps"], "name": n})
        layers = []
        for i in range(cfg["layers"]):
            p = f"l{i}."
            attn = PartSpec("gqa_attention", {
                "hidden_size": d, "num_heads": H, "num_kv_heads": G, "head_dim": hd,
                "position": PartSpec("toy_interpolated", {"head_dim": hd, "factor": cfg["factor"]}),
                "names": {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}})
            # even layers: routed experts; odd layers: the framework's dense feed-forward
            ff = PartSpec("toy_top1_experts", {"hidden_size": d, "intermediate_size": cfg["inter"],
                                               "num_experts": cfg["experts"], "name": p + "moe"}) if i % 2 == 0 else \
                PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": cfg["inter"],
                                       "names": {"gate": p + "g", "up": p + "u", "down": p + "d"}})
            layers.append(LayerSpec(PartSpec("pre_norm"), attn, norm(p + "n1"), ff, norm(p + "n2")))
        return ModelSpec("ToyRoutedForCausalLM", cfg["vocab_size"], d, 256,
                         PartSpec("token_embedding", {"vocab_size": cfg["vocab_size"], "hidden_size": d, "name": "emb"}),
                         tuple(layers), tuple(range(cfg["layers"])), norm("nf"),
                         PartSpec("lm_head", {"vocab_size": cfg["vocab_size"], "hidden_size": d, "name": "head"}))

    register_architecture(("ToyRoutedForCausalLM",), dict, spec)


TOY = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 61, "hidden_size": 40, "inter": 56, "heads": 4, "kv": 2,
       "head_dim": 16, "eps": 1e-5, "layers": 3, "experts": 5, "factor": 2.5}


def _restated(model, tokens):
    """The toy model in float64 from the engine's bound parameters (whole sequence, no cache)."""
    c = TOY
    d, hd, H, G = c["hidden_size"], c["head_dim"], c["heads"], c["kv"]
    f = lambda t: t.detach().to(F64).cpu()
    x = f(model.embedding.weight)[torch.tensor(tokens)]
    T = len(tokens)
    inv = torch.tensor([1.0 / ((1 + i) ** 2 * c["factor"]) for i in range(hd // 2)], dtype=torch.float32)
    sin, cos = P.rope_angles(torch.arange(T), inv)
    used = set()
    for blk in model.blocks:
        xn = P.rms_norm(x, f(blk.mixer_norm.weight), c["eps"])
        qkv = xn @ f(blk.mixer.wqkv).T
        q, k, v = qkv[:, :H * hd], qkv[:, H * hd:(H + G) * hd], qkv[:, (H + G) * hd:]
        q = P.apply_rope_half(q.view(T, H, hd), sin, cos)
        k = P.apply_rope_half(k.view(T, G, hd), sin, cos)
        a = P.causal_attention(q, k, v.reshape(T, G, hd)).reshape(T, H * hd)
        x = x + a @ f(blk.mixer.wo).T
        xn = P.rms_norm(x, f(blk.feed_forward_norm.weight), c["eps"])
        ff = blk.feed_forward
        if hasattr(ff, "router"):
            logits = xn @ f(ff.router).T
            prob = torch.softmax(logits, dim=-1)
            top = logits.argmax(dim=-1)
            for t in range(T):
                e = int(top[t]); used.add(e)
                x[t] = x[t] + prob[t, e] * (f(ff.w_out)[e] @ torch.relu(f(ff.w_in)[e] @ xn[t]))
        else:
            gu = xn @ f(ff.wgu).T
            I = c["inter"]
            x = x + P.swiglu(gu[:, :I], gu[:, I:]) @ f(ff.wdown).T
    xn = P.rms_norm(x, f(model.final_norm.weight), c["eps"])
    return xn @ f(model.head.weight).T, used


def test_routed_feed_forward_and_own_position_encoding_register_build_and_step():
    _register()
    from rustyllm_b200 import Runner
    r = Runner.from_config(TOY, seed=11, dtype="float32", max_cache_tokens=64 * 4, max_batch=3, std=0.35)
    m = r.model
    assert type(m.blocks[0].feed_forward).__name__ == "ToyTop1Experts" and m.blocks[0].feed_forward.w_in.shape == (5, 56, 40)
    assert type(m.blocks[1].feed_forward).__name__ == "GatedMLP"
    assert type(m.blocks[0].mixer.position).__name__ == "ToyInterpolatedRotation"
    assert not m.graph_capturable
    eng = r.engine
    seqs = [[3, 9, 27, 31, 4, 4, 18, 60, 2, 2, 45, 7, 13], [7, 1, 44, 0]]
    slots = [eng.alloc_slot() for _ in seqs]
    whole = eng.step(slots, seqs, "all")
    for s in slots:
        eng.free_slot(s)
    want = []
    experts_used = set()
    for s in seqs:
        w, used = _restated(m, s)
        want.append(w); experts_used |= used
    assert len(experts_used) >= 3                                  # the router really routes
    torch.testing.assert_close(whole.double().cpu(), torch.cat(want), rtol=2e-4, atol=2e-4)
    # a prompt step and then single tokens, unequal lengths, in reused slots
    slots = [eng.alloc_slot() for _ in seqs]
    a = eng.step(slots, [seqs[0][:5], seqs[1][:1]], "all")
    rows = {0: [a[:5]], 1: [a[5:6]]}
    fed = [5, 1]
    while any(fed[i] < len(seqs[i]) for i in range(2)):
        live = [i for i in range(2) if fed[i] < len(seqs[i])]
        out = eng.step([slots[i] for i in live], [[seqs[i][fed[i]]] for i in live], "last")
        for row, i in enumerate(live):
            rows[i].append(out[row:row + 1]); fed[i] += 1
    stepped = torch.cat(rows[0] + rows[1])
    torch.testing.assert_close(stepped, whole, rtol=1e-5, atol=1e-5)
    for sl in slots:
        eng.free_slot(sl)
    r.cache.check()
    assert math.isfinite(float(whole.abs().max())) and whole.std() > 1e-3


# ----------------------------------------------------------------------------- a learned position table, narrow value heads
def _register_absolute():
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.config.registry import register_architecture
    from rustyllm_b200.config.spec import LayerSpec, ModelSpec, ParamSource, ParamSpec, PartSpec
    from rustyllm_b200.parts import Part, register

    @register("embedding", "toy_token_plus_position")
    class ToyTokenPlusPosition(Part):
        """x = E[token] + P[position]: a learned absolute position table.  The embedding part is
        handed the step, so it finds the positions beside the tokens; both look-ups are the
        framework's own gather kernel."""

        def __init__(self, runtime, vocab_size, max_positions, hidden_size, name):
            self.V, self.maxpos, self.d, self.name = vocab_size, max_positions, hidden_size, name
            self.bad_token = torch.zeros(1, dtype=torch.int32, device=runtime.device)

        def param_specs(self):
            return {"weight": ParamSpec((ParamSource(self.name + ".tokens", (self.V, self.d)),), role="table"),
                    "positions": ParamSpec((ParamSource(self.name + ".positions", (self.maxpos, self.d)),), role="table")}

        def forward(self, step):
            M = step.tokens.numel()
            x = torch.empty((M, self.d), dtype=torch.float32, device=step.tokens.device)
            p = torch.empty_like(x)
            K.embedding(self.weight, step.tokens, x, self.bad_token)
            K.embedding(self.positions, step.positions, p, self.bad_token)
            return x.add_(p)

    def spec(cfg):
        d = cfg["hidden_size"]
        def norm(n): return PartSpec("rms_norm", {"size": d, "eps": cfg["eps"], "name": n})
        layers = []
        for i in range(cfg["layers"]):
            p = f"l{i}."
            attn = PartSpec("gqa_attention", {
                "hidden_size": d, "num_heads": cfg["heads"], "num_kv_heads": cfg["kv"], "head_dim": cfg["head_dim"],
                "value_dim": cfg["value_dim"], "position": PartSpec("none", {"head_dim": cfg["head_dim"]}),
                "names": {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}})
            ff = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": cfg["inter"],
                                        "names": {"gate": p + "g", "up": p + "u", "down": p + "d"}})
            layers.append(LayerSpec(PartSpec("pre_norm"), attn, norm(p + "n1"), ff, norm(p + "n2")))
        return ModelSpec("ToyAbsoluteForCausalLM", cfg["vocab_size"], d, cfg["max_positions"],
                         PartSpec("toy_token_plus_position", {"vocab_size": cfg["vocab_size"], "max_positions": cfg["max_positions"],
                                                              "hidden_size": d, "name": "emb"}),
                         tuple(layers), tuple(range(cfg["layers"])), norm("nf"),
                         PartSpec("lm_head", {"vocab_size": cfg["vocab_size"], "hidden_size": d, "name": "head"}))

    register_architecture(("ToyAbsoluteForCausalLM",), dict, spec)


ABS = {"architectures": ["ToyAbsoluteForCausalLM"], "vocab_size": 53, "max_positions": 200, "hidden_size": 48, "inter": 72,
       "heads": 6, "kv": 2, "head_dim": 16, "value_dim": 10, "eps": 1e-5, "layers": 2}


def _restated_absolute(model, tokens):
    c = ABS
    hd, vd, H, G = c["head_dim"], c["value_dim"], c["heads"], c["kv"]
    f = lambda t: t.detach().to(F64).cpu()
    T = len(tokens)
    x = f(model.embedding.weight)[torch.tensor(tokens)] + f(model.embedding.positions)[:T]
    scale = 1.0 / math.sqrt(hd)
    for blk in model.blocks:
        xn = P.rms_norm(x, f(blk.mixer_norm.weight), c["eps"])
        qkv = xn @ f(blk.mixer.wqkv).T
        q = qkv[:, :H * hd].view(T, H, hd)
        k = qkv[:, H * hd:(H + G) * hd].view(T, G, hd)
        v = qkv[:, (H + G) * hd:].view(T, G, vd)
        a = torch.empty(T, H, vd, dtype=F64)
        mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
        for h in range(H):
            g = h // (H // G)
            s = (q[:, h] @ k[:, g].T * scale).masked_fill(~mask, float("-inf"))
            a[:, h] = torch.softmax(s, -1) @ v[:, g]
        x = x + a.reshape(T, H * vd) @ f(blk.mixer.wo).T
        xn = P.rms_norm(x, f(blk.feed_forward_norm.weight), c["eps"])
        gu = xn @ f(blk.feed_forward.wgu).T
        # a bfloat16 run keeps gate and up rows in turn, a 32-bit run one block after the other
        gate, up = (gu[:, 0::2], gu[:, 1::2]) if blk.feed_forward.interleaved else (gu[:, :c["inter"]], gu[:, c["inter"]:])
        x = x + P.swiglu(gate, up) @ f(blk.feed_forward.wdown).T
    return P.rms_norm(x, f(model.final_norm.weight), c["eps"]) @ f(model.head.weight).T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_learned_positions_and_narrow_value_heads_register_build_and_step(dtype):
    """An architecture registered from here whose embedding adds a learned absolute position
    table (no rotation at all) and whose value heads (10) are narrower than its key heads (16):
    value storage of its own width in the cache, the any-shape attention kernel, whole prompts
    and token by token, against the float64 restatement above."""
    _register_absolute()
    from rustyllm_b200 import Runner
    r = Runner.from_config(ABS, seed=13, dtype=dtype, storage_dtype="bfloat16", max_cache_tokens=64 * 8, max_batch=3, std=0.05)
    m = r.model
    assert type(m.embedding).__name__ == "ToyTokenPlusPosition" and m.embedding.positions.shape == (200, 48)
    assert m.blocks[0].mixer.wqkv.shape == (6 * 16 + 2 * 16 + 2 * 10, 48) and m.blocks[0].mixer.wo.shape == (48, 60)
    g = r.cache.groups[0]
    assert g.keys.shape[-1] == 16 and g.values.shape[-1] == 10
    eng = r.engine
    gen = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 53, (n,), generator=gen).tolist() for n in (150, 9, 70)]
    want = torch.cat([_restated_absolute(m, s) for s in seqs])
    from gpu_helpers import assert_close_logits         # the engine tests' bounds, relative to a row's scale
    slots = [eng.alloc_slot() for _ in seqs]
    whole = eng.step(slots, seqs, "all")
    for s in slots:
        eng.free_slot(s)
    assert_close_logits(whole, want, dtype, "toy absolute, whole")
    slots = [eng.alloc_slot() for _ in seqs]
    cut = [120, 3, 66]
    a = eng.step(slots, [s[:n] for s, n in zip(seqs, cut)], "all")
    rows, o = {}, 0
    for i, n in enumerate(cut):
        rows[i] = [a[o:o + n]]; o += n
    fed = list(cut)
    while any(fed[i] < len(seqs[i]) for i in range(3)):
        live = [i for i in range(3) if fed[i] < len(seqs[i])]
        out = eng.step([slots[i] for i in live], [[seqs[i][fed[i]]] for i in live], "last")
        for row, i in enumerate(live):
            rows[i].append(out[row:row + 1]); fed[i] += 1
    stepped = torch.cat(rows[0] + rows[1] + rows[2])
    assert_close_logits(stepped, want, dtype, "toy absolute, prompt step then single tokens")
    for sl in slots:
        eng.free_slot(sl)
    r.cache.check()
    assert int(m.embedding.bad_token.item()) == 0
