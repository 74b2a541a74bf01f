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
