"""Shared helpers of the GPU tests: tolerances, plain logits, driving the engine."""
import functools

import numpy as np
import torch

import plain_llama as P

# ---- tolerances, fixed in advance from the arithmetic (never widened to pass) ----
# 32-bit path against float64: products of up to ~300 terms accumulated in float32,
# through at most three layers, leave errors of a few 1e-7 of a row's scale; 3e-5 is
# two orders above that and two orders below the smallest real fault (a wrong key
# among hundreds moves a logit by ~1e-3 of the scale).
F32_REL = 3e-5
# bf16 path against float64: every stored activation is rounded to 8 bits of
# mantissa (rms relative error 2^-9/sqrt(3) = 1.1e-3); about six such roundings per
# layer and one before the head add up, for three layers, to ~0.5 % rms of the scale
# of a logit row; the maximum over a few thousand logits sits near four sigma.
BF16_REL_MAX = 3e-2
BF16_REL_MEAN = 6e-3


def assert_close_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = ""):
    got = got.detach().to("cpu", torch.float64)
    ref = ref.detach().to("cpu", torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = ref.pow(2).mean(dim=-1, keepdim=True).sqrt().clamp_min(1e-30)   # rms of each row
    err = (got - ref).abs() / scale
    worst = err.max().item()
    if dtype == "float32":
        assert worst <= F32_REL, f"{what}: max |diff| / rms(row) = {worst:.3e} > {F32_REL} (row {err.max(dim=-1).values.argmax().item()})"
    else:
        mean = err.mean().item()
        assert worst <= BF16_REL_MAX, f"{what}: max |diff| / rms(row) = {worst:.3e} > {BF16_REL_MAX} (row {err.max(dim=-1).values.argmax().item()})"
        assert mean <= BF16_REL_MEAN, f"{what}: mean |diff| / rms(row) = {mean:.3e} > {BF16_REL_MEAN}"
    return worst


@functools.lru_cache(maxsize=None)
def _plain_model(model_dir: str):
    return P.load_model_dir(model_dir)


_LOGITS_CACHE = {}


def plain_logits(model_dir: str, tokens) -> torch.Tensor:
    """float64 logits [T, V] of the plain implementation (cached per sequence)."""
    key = (model_dir, tuple(tokens))
    if key not in _LOGITS_CACHE:
        cfg, w = _plain_model(model_dir)
        _LOGITS_CACHE[key] = P.forward(cfg, w, list(tokens))
    return _LOGITS_CACHE[key]


def random_tokens(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def load_runner(model_dir: str, dtype: str, max_cache_tokens: int = 64 * 48, max_batch: int = 16):
    from rustyllm_b200 import Runner
    runner, _ = Runner.from_path(model_dir, dtype=dtype, max_cache_tokens=max_cache_tokens, max_batch=max_batch)
    return runner
