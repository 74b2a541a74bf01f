"""Weights: the safetensors container, the loader's one error, dtype policy, random folders (no GPU)."""
import json
import os

import pytest
import torch

from rustyllm_b200 import WeightsError, write_random_model
from rustyllm_b200.config.registry import resolve_architecture
from rustyllm_b200.models.decoder import DecoderModel
from rustyllm_b200.parts import Runtime
from rustyllm_b200.weights.loader import check_checkpoint, load_parameters, runtime_dtype
from rustyllm_b200.weights.safetensors_io import Checkpoint, SafetensorsError, write_safetensors
from tiny_configs import TINY

CPU = torch.device("cpu")


def _model(cfg_dict, dtype=torch.float32):
    arch = resolve_architecture(cfg_dict)
    spec = arch.build_spec(arch.parse_config(cfg_dict))
    return DecoderModel(spec, Runtime(CPU, dtype)), spec


def test_container_round_trip_and_agrees_with_the_safetensors_package(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, t)
    ck = Checkpoint(str(tmp_path))
    for k, v in t.items():
        assert torch.equal(ck.tensor(k), v)
    safetensors_torch = pytest.importorskip("safetensors.torch")
    other = safetensors_torch.load_file(p)
    for k, v in t.items():
        assert torch.equal(other[k], v)
    # and the other way round
    p2 = tmp_path / "other"
    p2.mkdir()
    safetensors_torch.save_file(t, str(p2 / "model.safetensors"))
    ck2 = Checkpoint(str(p2))
    for k, v in t.items():
        assert torch.equal(ck2.tensor(k), v)


def test_truncated_file_is_refused(tmp_path):
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, {"a": torch.randn(64, 64)})
    data = open(p, "rb").read()
    open(p, "wb").write(data[:-100])
    with pytest.raises(SafetensorsError, match="beyond the file size"):
        Checkpoint(str(tmp_path))


def test_sharded_folder_and_duplicates(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(2)})
    json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}},
              open(tmp_path / "model.safetensors.index.json", "w"))
    ck = Checkpoint(str(tmp_path))
    assert sorted(ck.names()) == ["a", "b"]
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(2), "a": torch.ones(2)})
    with pytest.raises(SafetensorsError, match="both"):
        Checkpoint(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = TINY["A"]["config"]
    d = write_random_model(str(tmp_path / "m"), cfg, seed=3, dtype="float32")
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    ck.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)   # should be [32, 64]
    tensors["model.layers.0.extra.weight"] = torch.zeros(4)
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    model, spec = _model(cfg)
    with pytest.raises(WeightsError) as ei:
        load_parameters(model.param_specs(), Checkpoint(d), torch.float32, CPU, spec.ignored_tensors)
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.extra.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    assert e.wrong_dtype[0][0] == "model.layers.1.input_layernorm.weight"
    msg = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[16, 64]", "[32, 64]"):
        assert needle in msg


def test_dtype_policy():
    bf, f32 = torch.bfloat16, torch.float32
    assert runtime_dtype("matrix", bf, bf) == bf
    assert runtime_dtype("matrix", f32, bf) == f32      # stored in 32-bit stays 32-bit
    assert runtime_dtype("matrix", bf, f32) == f32      # a 32-bit run widens everything
    assert runtime_dtype("vector", bf, bf) == f32       # norm weights and biases: 32-bit math
    assert runtime_dtype("int_table", torch.int64, bf) == torch.int32


def test_load_concatenates_ties_and_keeps_values(tmp_path):
    cfg = TINY["B"]["config"]
    d = write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype="bfloat16")
    model, spec = _model(cfg, torch.bfloat16)
    ck = Checkpoint(d)
    assert "lm_head.weight" not in ck.entries       # tied: stored once
    p = load_parameters(model.param_specs(), ck, torch.bfloat16, CPU, spec.ignored_tensors)
    assert p["head.weight"].data_ptr() == p["embedding.weight"].data_ptr()
    wqkv = p["layers.2.mixer.wqkv"]
    assert wqkv.shape == ((3 + 2 * 1) * 32, 96) and wqkv.dtype == torch.bfloat16
    assert torch.equal(wqkv[:96], ck.tensor("model.layers.2.self_attn.q_proj.weight"))
    assert torch.equal(wqkv[96:128], ck.tensor("model.layers.2.self_attn.k_proj.weight"))
    assert torch.equal(wqkv[128:], ck.tensor("model.layers.2.self_attn.v_proj.weight"))
    wgu = p["layers.0.feed_forward.wgu"]          # bf16 run: gate and up rows interleaved
    assert torch.equal(wgu[1::2], ck.tensor("model.layers.0.mlp.up_proj.weight"))
    assert torch.equal(wgu[0::2], ck.tensor("model.layers.0.mlp.gate_proj.weight"))
    model32, _ = _model(cfg, torch.float32)       # 32-bit run: gate rows, then up rows
    p32 = load_parameters(model32.param_specs(), ck, torch.float32, CPU, spec.ignored_tensors)
    assert torch.equal(p32["layers.0.feed_forward.wgu"][256:], ck.tensor("model.layers.0.mlp.up_proj.weight").float())
    assert p["layers.0.mixer_norm.weight"].dtype == torch.float32
    model.bind(p)
    # a tied checkpoint that still carries a head copy is tolerated
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    check_checkpoint(model.param_specs(), Checkpoint(d).entries, spec.ignored_tensors)


def test_float32_file_in_a_bf16_run_stays_32_bit(tmp_path):
    cfg = TINY["A"]["config"]
    d = write_random_model(str(tmp_path / "m"), cfg, seed=0, dtype="float32")
    model, spec = _model(cfg, torch.bfloat16)
    p = load_parameters(model.param_specs(), Checkpoint(d), torch.bfloat16, CPU, spec.ignored_tensors)
    assert p["layers.0.mixer.wqkv"].dtype == torch.float32
    assert p["embedding.weight"].dtype == torch.float32
    # rounded to the compute dtype only when asked (nearest even, as a bfloat16 file would hold them)
    r = load_parameters(model.param_specs(), Checkpoint(d), torch.bfloat16, CPU, spec.ignored_tensors, keep_fp32=False)
    assert r["layers.0.mixer.wqkv"].dtype == torch.bfloat16 and r["embedding.weight"].dtype == torch.bfloat16
    assert torch.equal(r["embedding.weight"], p["embedding.weight"].to(torch.bfloat16))
    assert r["layers.0.mixer_norm.weight"].dtype == torch.float32       # vectors stay 32-bit either way


def test_random_folder_is_reproducible_and_seeded(tmp_path):
    cfg = TINY["C"]["config"]
    a = write_random_model(str(tmp_path / "a"), cfg, seed=5)
    b = write_random_model(str(tmp_path / "b"), cfg, seed=5)
    c = write_random_model(str(tmp_path / "c"), cfg, seed=6)
    ca, cb, cc = Checkpoint(a), Checkpoint(b), Checkpoint(c)
    assert sorted(ca.names()) == sorted(cb.names())
    assert "model.layers.0.self_attn.q_proj.bias" in ca.entries and "model.layers.1.mlp.down_proj.bias" in ca.entries
    for n in ca.names():
        assert torch.equal(ca.tensor(n), cb.tensor(n))
    assert not torch.equal(ca.tensor("model.embed_tokens.weight"), cc.tensor("model.embed_tokens.weight"))
    w = ca.tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and w.dtype == torch.float32
    cfg_on_disk = json.load(open(os.path.join(a, "config.json")))
    assert cfg_on_disk["hidden_size"] == 80 and cfg_on_disk["torch_dtype"] == "bfloat16"
    n = write_random_model(str(tmp_path / "n"), cfg, seed=5, norm_noise=True)
    nw = Checkpoint(n).tensor("model.norm.weight").float()
    assert 0.9 < nw.mean().item() < 1.1 and nw.std().item() > 0.005
    assert torch.all(ca.tensor("model.norm.weight").float() == 1.0)


def test_random_numbers_are_a_function_of_seed_and_index_alone():
    """The generator behind random weights: integer arithmetic and two float operations, so the
    host code here and the device kernel give the same bits (the device half is a GPU test)."""
    import numpy as np
    from rustyllm_b200.weights.random_init import _tensor_seed, normal_values
    v = normal_values(12345, 1 << 16, 0.0, 0.02)
    assert v.dtype == np.float32 and abs(float(v.mean())) < 3e-4 and abs(float(v.std()) - 0.02) < 3e-4
    assert float(np.abs(v).max()) <= 6 * 0.02
    # literal values: element 0 of seed 12345 is the sum of the twelve 16-bit fields of three splitmix64 outputs
    def sm(x):
        m = (1 << 64) - 1
        z = (x + 0x9E3779B97F4A7C15) & m
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        return z ^ (z >> 31)
    for i in (0, 1, 77):
        total = 0
        for r in range(3):
            h = sm(12345 + 3 * i + r)
            total += (h & 0xffff) + ((h >> 16) & 0xffff) + ((h >> 32) & 0xffff) + (h >> 48)
        assert v[i] == np.float32(total - 393210) * (np.float32(0.02) * np.float32(1 / 65536))
    # part of a tensor is the beginning of the whole; another seed, other numbers; mean 1 for norm weights
    assert np.array_equal(normal_values(12345, 100, 0.0, 0.02), v[:100])
    assert not np.array_equal(normal_values(12346, 100, 0.0, 0.02), v[:100])
    w = normal_values(7, 1000, 1.0, 0.02)
    assert abs(float(w.mean()) - 1.0) < 3e-3
    assert _tensor_seed(1, "a") != _tensor_seed(1, "b") != _tensor_seed(2, "b")
