"""Tiny configurations of the architecture for tests.  They differ from one another
in every size and option: heads and groups (GQA / MQA / MHA), head size, sizes that
are no power of two, number of layers, vocabulary, eps, rope base and scaling,
tied or untied head, biases."""
import os

from rustyllm_b200 import write_random_model

TINY = {
    # 2 layers, GQA 4/2, head 16, untied, plain rope, norm weights 1 + N(0, .02)
    "A": dict(seed=0, norm_noise=True, dtype="float32", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 256, "hidden_size": 64, "intermediate_size": 172, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
        "max_position_embeddings": 128, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "rope_scaling": None, "tie_word_embeddings": False, "eos_token_id": 255}),
    # 3 layers, MQA 3/1, head 32, tied, llama3 rope scaling, bf16 file
    "B": dict(seed=1, norm_noise=False, dtype="bfloat16", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 384, "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
        "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
        "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
        "tie_word_embeddings": True, "eos_token_id": [382, 383]}),
    # 2 layers, MHA 5/5, head 48 (heads * head size != hidden), odd vocabulary, biases, long context
    "C": dict(seed=2, norm_noise=True, dtype="bfloat16", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 307, "hidden_size": 80, "intermediate_size": 136, "num_hidden_layers": 2,
        "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
        "max_position_embeddings": 640, "rms_norm_eps": 3e-6, "rope_theta": 25000.0,
        "tie_word_embeddings": False, "attention_bias": True, "mlp_bias": True}),
    # 2 layers, GQA 4/2, head 64: the shape class the tensor-core attention kernels take
    "D": dict(seed=3, norm_noise=True, dtype="bfloat16", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 320, "hidden_size": 128, "intermediate_size": 192, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
        "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 256},
        "tie_word_embeddings": True}),
    # 2 layers, GQA 4/2, head 128, hidden 512: decode-sized steps split the QKV product over K, so
    # rotation and cache write ride in its epilogue; prefill attention takes the tcgen05 kernel
    "E": dict(seed=4, norm_noise=True, dtype="bfloat16", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 272, "hidden_size": 512, "intermediate_size": 640, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
        "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "tie_word_embeddings": False, "attention_bias": True}),
    # E's widths with a long context and the rope constants of the real 8B model: positions in the
    # thousands, where float rounding of pos * inv_freq and the length of a slot's page table show
    "F": dict(seed=5, norm_noise=True, dtype="bfloat16", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 272, "hidden_size": 512, "intermediate_size": 640, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
        "max_position_embeddings": 8768, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "tie_word_embeddings": False}),
    # D's widths (head 64) with a long context and the rope constants of the real 1B model
    "G": dict(seed=6, norm_noise=True, dtype="bfloat16", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 320, "hidden_size": 128, "intermediate_size": 192, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
        "max_position_embeddings": 8768, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "tie_word_embeddings": True}),
    # 32 query heads on one KV head: more than the tensor-core decode attention groups (16), so
    # single-token steps fall to the any-shape kernel while prompts take the tensor cores
    "H": dict(seed=7, norm_noise=True, dtype="bfloat16", config={
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": 300, "hidden_size": 256, "intermediate_size": 320, "num_hidden_layers": 2,
        "num_attention_heads": 32, "num_key_value_heads": 1, "head_dim": 64,
        "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "tie_word_embeddings": False}),
}


def write_tiny(name: str, path: str) -> str:
    t = TINY[name]
    os.makedirs(path, exist_ok=True)
    return write_random_model(path, t["config"], seed=t["seed"], dtype=t["dtype"], norm_noise=t["norm_noise"])
