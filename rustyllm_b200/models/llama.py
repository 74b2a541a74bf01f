"""The Llama dense decoder as a ``ModelSpec``: which parts, with which constants and
which checkpoint tensor names.

Layer order and tensors follow the reference's standard path
(``forward_into``, src/model.rs:7177-7358; ``load_model``, src/model.rs:3573-4048),
with the tensor names of the architecture's own safetensors checkpoints in place
of the GGUF names:

  token_embd.weight        -> model.embed_tokens.weight              [V x d]
  blk.N.attn_norm.weight   -> model.layers.N.input_layernorm.weight  [d]
  blk.N.attn_{q,k,v}.weight-> model.layers.N.self_attn.{q,k,v}_proj.weight
  blk.N.attn_output.weight -> model.layers.N.self_attn.o_proj.weight [d x H*hd]
  blk.N.ffn_norm.weight    -> model.layers.N.post_attention_layernorm.weight
  blk.N.ffn_{gate,up,down} -> model.layers.N.mlp.{gate,up,down}_proj.weight
  output_norm.weight       -> model.norm.weight
  output.weight            -> lm_head.weight (absent = tied, src/model.rs:3654-3667)

Rotary pairing: checkpoints in this layout pair element i with i + head_dim/2
(the reference's ``apply_rope_qk_neox``, src/model.rs:5606-5647, and its comment
at 5520-5523 on why GGUF files use interleaved pairs instead).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    d, hd = cfg.hidden_size, cfg.head_dim
    rope = PartSpec("rope", {
        "head_dim": hd,
        "rotary_dim": hd,
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
        "pairing": "half",
    })
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            block=PartSpec("pre_norm"),
            mixer=PartSpec("gqa_attention", {
                "hidden_size": d,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": hd,
                "bias": cfg.attention_bias,
                "window": None,
                "position": rope,
                "names": {"q": p + "self_attn.q_proj", "k": p + "self_attn.k_proj",
                          "v": p + "self_attn.v_proj", "o": p + "self_attn.o_proj"},
            }),
            mixer_norm=PartSpec("rms_norm", {
                "size": d, "eps": cfg.rms_norm_eps, "name": p + "input_layernorm.weight"}),
            feed_forward=PartSpec("gated_mlp", {
                "hidden_size": d,
                "intermediate_size": cfg.intermediate_size,
                "activation": cfg.hidden_act,
                "bias": cfg.mlp_bias,
                "names": {"gate": p + "mlp.gate_proj", "up": p + "mlp.up_proj",
                          "down": p + "mlp.down_proj"},
            }),
            feed_forward_norm=PartSpec("rms_norm", {
                "size": d, "eps": cfg.rms_norm_eps,
                "name": p + "post_attention_layernorm.weight"}),
        ))
    spec = ModelSpec(
        architecture="LlamaForCausalLM",
        vocab_size=cfg.vocab_size,
        hidden_size=d,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {
            "vocab_size": cfg.vocab_size, "hidden_size": d,
            "name": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        schedule=tuple(range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", {
            "size": d, "eps": cfg.rms_norm_eps, "name": "model.norm.weight"}),
        head=PartSpec("lm_head", {
            "vocab_size": cfg.vocab_size, "hidden_size": d, "name": "lm_head.weight",
            "tied_to": "embedding.weight" if cfg.tie_word_embeddings else None}),
        eos_token_id=cfg.eos_token_id,
        bos_token_id=cfg.bos_token_id,
        # A tied checkpoint may still carry a copy of the head; rotary tables some
        # exporters write are recomputed from the configuration.
        ignored_tensors=(("lm_head.weight",) if cfg.tie_word_embeddings else ())
        + tuple(f"model.layers.{i}.self_attn.rotary_emb.inv_freq"
                for i in range(cfg.num_hidden_layers)),
    )
    spec.validate()
    return spec


LLAMA = register_architecture(("LlamaForCausalLM", "llama"), LlamaConfig.from_dict, llama_spec)
