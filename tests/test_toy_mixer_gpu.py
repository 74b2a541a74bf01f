"""A toy mixer with state of its own, a toy architecture that uses it beside attention,
a layer that runs twice and a layer that reads another layer's cache: all registered
from this test, with no change to the framework's files."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _register():
    from rustyllm_b200.cache.sequence_cache import StateNeed
    from rustyllm_b200.config.registry import register_architecture
    from rustyllm_b200.config.spec import LayerSpec, ModelSpec, ParamSource, ParamSpec, PartSpec
    from rustyllm_b200.parts import Mixer, register_mixer

    @register_mixer("toy_decay")
    class ToyDecayMixer(Mixer):
        """state <- decay * state + xn (per sequence, token after token); out = W state.
        The state lives in the cache's per-sequence state area as ``d`` floats."""
        graph_capturable = False      # the loop below reads sequence boundaries on the host

        def __init__(self, runtime, hidden_size, decay, name):
            self.d, self.decay, self.name = hidden_size, decay, name

        def param_specs(self):
            return {"w": ParamSpec((ParamSource(self.name, (self.d, self.d)),))}

        def state_need(self):
            return StateNeed(self.d * 4)

        def forward(self, xn, residual, step, cache):
            state = cache.state.view(torch.float32)            # [max_slots, d]
            w = self.w.float()
            cu = step.cu_seqlens.tolist()
            for b, slot in enumerate(step.seq_slots.tolist()):
                s = state[slot]
                for m in range(cu[b], cu[b + 1]):
                    s.mul_(self.decay).add_(xn[m].float())
                    residual[m] += w @ s

    def toy_spec(cfg):
        d, hd = cfg["hidden_size"], cfg["head_dim"]
        def norm(n): return PartSpec("rms_norm", {"size": d, "eps": cfg["eps"], "name": n})
        def ff(p): return PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": cfg["inter"],
                                                 "names": {"gate": p + "g", "up": p + "u", "down": p + "d"}})
        def attn(p): return PartSpec("gqa_attention", {
            "hidden_size": d, "num_heads": cfg["heads"], "num_kv_heads": cfg["kv"], "head_dim": hd,
            "position": PartSpec("rope", {"head_dim": hd, "rotary_dim": hd // 2, "theta": 100.0, "pairing": "interleaved"}),
            "names": {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}})
        layers = []
        for i, kind in enumerate(cfg["mixers"]):
            p = f"l{i}."
            mixer = attn(p) if kind == "attention" else PartSpec("toy_decay", {"hidden_size": d, "decay": 0.5, "name": p + "mix"})
            layers.append(LayerSpec(PartSpec("pre_norm"), mixer, norm(p + "n1"), ff(p), norm(p + "n2"),
                                    cache_from=cfg["cache_from"].get(i)))
        return ModelSpec("ToyForCausalLM", cfg["vocab_size"], d, 256,
                         PartSpec("token_embedding", {"vocab_size": cfg["vocab_size"], "hidden_size": d, "name": "emb"}),
                         tuple(layers), tuple(cfg["schedule"]), norm("nf"),
                         PartSpec("lm_head", {"vocab_size": cfg["vocab_size"], "hidden_size": d, "name": "head", "tied_to": "embedding.weight"}))

    register_architecture(("ToyForCausalLM",), dict, toy_spec)


TOY = {"architectures": ["ToyForCausalLM"], "vocab_size": 50, "hidden_size": 24, "inter": 40, "heads": 2, "kv": 1,
       "head_dim": 16, "eps": 1e-5,
       # layer 0: state mixer; layer 1: attention; layer 2: attention reading layer 1's cache
       "mixers": ["toy", "attention", "attention"], "cache_from": {2: 1},
       # layer 0 runs twice (two states), the schedule is data
       "schedule": [0, 1, 2, 0]}


def test_toy_mixer_with_state_registers_builds_and_steps():
    _register()
    from rustyllm_b200 import Runner
    r = Runner.from_config(TOY, seed=4, dtype="float32", max_cache_tokens=64 * 4, max_batch=3, std=0.3)
    m = r.model
    assert [e for e, _ in m.run_entry] == [0, 1, 1, 2] and [w for _, w in m.run_entry] == [True, True, False, True]
    assert r.cache.state_bytes == 2 * 256 and len(r.cache.groups) == 1 and r.cache.groups[0].layers == 1
    eng = r.engine
    seqs = [[3, 9, 27, 31, 4, 4, 18], [7, 1, 44]]
    # whole
    slots = [eng.alloc_slot() for _ in seqs]
    whole = eng.step(slots, seqs, "all")
    for s in slots:
        eng.free_slot(s)
    # a prompt step and then single tokens, in a reused slot (state must restart from zero)
    slots = [eng.alloc_slot() for _ in seqs]
    a = eng.step(slots, [seqs[0][:4], seqs[1][:1]], "all")
    rows = {0: [a[:4]], 1: [a[4:5]]}
    fed = [4, 1]
    while any(fed[i] < len(seqs[i]) for i in range(2)):
        live = [i for i in range(2) if fed[i] < len(seqs[i])]
        out = eng.step([slots[i] for i in live], [[seqs[i][fed[i]]] for i in live], "last")
        for row, i in enumerate(live):
            rows[i].append(out[row:row + 1]); fed[i] += 1
    stepped = torch.cat(rows[0] + rows[1])
    torch.testing.assert_close(stepped, whole, rtol=1e-5, atol=1e-5)
    assert whole.std() > 1e-3

    # the state mixer really carries state: its float64 restatement for sequence 1, layer run 0
    w = m.blocks[0].mixer.w.double().cpu()
    emb = m.embedding.weight.double().cpu()
    x = emb[torch.tensor(seqs[1])]
    n1 = m.blocks[0].mixer_norm.weight.double().cpu()
    xn = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * n1
    s = torch.zeros(24, dtype=torch.float64); want = []
    for t in range(3):
        s = 0.5 * s + xn[t]; want.append(x[t] + w @ s)
    st = r.cache.state_entry(0)
    assert st is not None and st.shape[1] == 96
    # after the run above the slot of sequence 1 holds exactly that state
    got_state = st.view(torch.float32)[slots[1]].double().cpu()
    torch.testing.assert_close(got_state, s, rtol=1e-5, atol=1e-6)
    for sl in slots:
        eng.free_slot(sl)
    r.cache.check()
