"""The Python entry point, in the shape of the reference's ``Runner``
(SimonWaldherr/RustyLLM src/runtime.rs:783-810; ``from_path`` 1944-2049 returns the runner with a
``LoadInfo``; ``generate`` / ``generate_stream`` 3034-3064; ``architecture`` 2052,
``model_name`` 2057, ``config`` 2072).  Prompts are token ids: this library has no
tokenizer.

    runner, info = Runner.from_path("model_dir", dtype="bfloat16")
    result = runner.generate([1, 15043], GenerationOptions(max_tokens=16))
    results = runner.generate([[1, 2, 3], [4, 5]], options)     # a batch
"""
from __future__ import annotations

import os
import sys
import threading
import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Union

import torch

from ..cache.sequence_cache import SequenceCache
from ..config.files import read_config_json, read_generation_stop_ids
from ..config.registry import resolve_architecture
from .. import kernels
from ..kernels import PAGE_SIZE
from ..models.decoder import DecoderModel
from ..parts import Runtime
from ..sampling.sampler import Sampler
from ..weights.loader import load_parameters
from ..weights.random_init import random_parameters
from ..weights.safetensors_io import Checkpoint
from .generate import GenerationOptions, GenerationResult, generate_batch, plan_batches
from .step import Engine

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported; use bfloat16 or float32")
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r} is not supported; use 'bfloat16' or 'float32'")
    return _DTYPES[dtype]


@dataclass
class LoadInfo:
    """Stage timings of a load, in seconds (SimonWaldherr/RustyLLM src/runtime.rs:437-446)."""
    file_size_bytes: int = 0
    load_time: float = 0.0
    parse_time: float = 0.0          # config.json and the safetensors headers
    compatibility_time: float = 0.0  # names, shapes and dtypes against the model
    weights_time: float = 0.0        # copies to the device
    runner_time: float = 0.0         # cache and buffers
    fp32_matrices: int = 0           # matrices kept in 32-bit in a bfloat16 run (slow products)


def _require_cuda(device: torch.device) -> None:
    if device.type != "cuda":
        raise RuntimeError(f"device {device} is not a CUDA device; this library has no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; this library has no CPU path")


class Runner:
    def __init__(self, config: Any, config_dict: Mapping[str, Any], model: DecoderModel,
                 max_cache_tokens: int, max_batch: int, name: Optional[str] = None,
                 kv_cache_dtype: Optional[torch.dtype] = None, extra_stop_ids: Sequence[int] = ()):
        self._config = config
        self._extra_stop_ids = tuple(extra_stop_ids)
        self.config_dict = dict(config_dict)
        self.model = model
        self.runtime = model.runtime
        self._name = name
        self.max_batch = max_batch
        max_seq = model.spec.max_position_embeddings
        self.cache: SequenceCache = model.new_cache(
            max_cache_tokens, max_slots=max(max_batch, 1), max_seq_len=max_seq, dtype=kv_cache_dtype)
        self.engine = Engine(model, self.cache)
        self.sampler = Sampler(self.runtime.device)
        self._generation_lock = threading.Lock()   # one generation at a time, src/runtime.rs:790-793

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_path(cls, path: str, dtype: Union[str, torch.dtype] = "bfloat16", device: str = "cuda:0",
                  max_cache_tokens: Optional[int] = None, max_batch: int = 64,
                  max_context: Optional[int] = None, keep_fp32_weights: bool = True):
        """Load a model folder (config.json + model.safetensors; generation_config.json,
        where there is one, adds its end-of-sequence ids to config.json's).  Returns
        ``(runner, load_info)``.

        ``keep_fp32_weights`` matters in a bfloat16 run only.  ``True`` (default): a matrix
        the file stores in 32-bit stays 32-bit, and its products run in 32-bit on the CUDA
        cores - many times slower than the tensor cores, so ``LoadInfo.fp32_matrices`` counts
        them and a line on stderr says so.  ``False``: they are rounded to bfloat16 (nearest
        even) like a bfloat16 file's would have been."""
        t0 = time.perf_counter()
        dev = torch.device(device)
        _require_cuda(dev)
        compute = parse_dtype(dtype)
        cfg_dict = read_config_json(path)
        arch = resolve_architecture(cfg_dict)
        config = arch.parse_config(cfg_dict)
        spec = arch.build_spec(config)
        ckpt = Checkpoint(path)
        t_parse = time.perf_counter()
        model = DecoderModel(spec, Runtime(dev, compute))
        from ..weights.loader import check_checkpoint
        check_checkpoint(model.param_specs(), ckpt.entries, spec.ignored_tensors, path)
        t_compat = time.perf_counter()
        tensors = load_parameters(model.param_specs(), ckpt, compute, dev, spec.ignored_tensors,
                                  keep_fp32=keep_fp32_weights)
        model.bind(tensors)
        torch.cuda.synchronize(dev)
        t_weights = time.perf_counter()
        size = ckpt.total_bytes
        ckpt.close()
        runner = cls(config, cfg_dict, model, cls._default_cache_tokens(spec, max_cache_tokens, max_batch, max_context),
                     max_batch, name=os.path.basename(os.path.normpath(path)),
                     extra_stop_ids=read_generation_stop_ids(path, spec.vocab_size))
        t1 = time.perf_counter()
        kept = 0
        if compute != torch.float32:
            kept = sum(1 for p, ps in model.param_specs().items()
                       if ps.role in ("matrix", "table") and p in tensors and tensors[p].dtype == torch.float32)
            if kept:
                print(f"rustyllm_b200: {kept} matrices of {path!r} are stored in 32-bit and stay 32-bit in this "
                      f"{dtype} run; their products run on the CUDA cores (keep_fp32_weights=False rounds them)",
                      file=sys.stderr)
        info = LoadInfo(file_size_bytes=size, load_time=t1 - t0, parse_time=t_parse - t0,
                        compatibility_time=t_compat - t_parse, weights_time=t_weights - t_compat,
                        runner_time=t1 - t_weights, fp32_matrices=kept)
        return runner, info

    @classmethod
    def from_config(cls, config: Union[Mapping[str, Any], Any], seed: int = 0,
                    dtype: Union[str, torch.dtype] = "bfloat16", device: str = "cuda:0",
                    max_cache_tokens: Optional[int] = None, max_batch: int = 64,
                    max_context: Optional[int] = None, std: float = 0.02, norm_noise: bool = False,
                    num_layers: Optional[int] = None,
                    storage_dtype: Union[str, torch.dtype, None] = None) -> "Runner":
        """Random weights drawn on the device from a configuration and a seed; no
        files.  ``num_layers`` overrides the number of layers (for measurements that
        must fit in less memory or time; layer sizes stay as configured).
        ``storage_dtype``: the dtype a checkpoint file would hold the values in (they are
        rounded to it once); default bfloat16 for a bfloat16 run, float32 for a float32 run.
        A float32 run with bfloat16 storage computes in 32-bit on exactly the weights of
        the bfloat16 run of the same seed."""
        dev = torch.device(device)
        _require_cuda(dev)
        compute = parse_dtype(dtype)
        cfg_dict = dict(config.to_dict() if hasattr(config, "to_dict") else config)
        if num_layers is not None:
            cfg_dict["num_hidden_layers"] = num_layers
        arch = resolve_architecture(cfg_dict)
        typed = arch.parse_config(cfg_dict)
        spec = arch.build_spec(typed)
        model = DecoderModel(spec, Runtime(dev, compute))
        storage = parse_dtype(storage_dtype) if storage_dtype is not None else \
            (torch.bfloat16 if compute == torch.bfloat16 else torch.float32)
        model.bind(random_parameters(model.param_specs(), seed, compute, dev, storage_dtype=storage,
                                     std=std, norm_noise=norm_noise))
        return cls(typed, cfg_dict, model,
                   cls._default_cache_tokens(spec, max_cache_tokens, max_batch, max_context), max_batch,
                   name=f"random-{seed}")

    @staticmethod
    def _default_cache_tokens(spec, max_cache_tokens, max_batch, max_context) -> int:
        if max_cache_tokens is not None:
            return max_cache_tokens
        ctx = min(spec.max_position_embeddings, max_context or 4096)
        return max_batch * (-(-ctx // PAGE_SIZE) * PAGE_SIZE)

    # ------------------------------------------------------------------ facts
    @property
    def config(self):
        return self._config

    def architecture(self) -> str:
        return self.model.spec.architecture

    def model_name(self) -> Optional[str]:
        return self._name

    @property
    def max_context(self) -> int:
        return self.cache.max_seq_len

    def stop_token_ids(self) -> Sequence[int]:
        """End-of-sequence ids of the model (the reference's ``is_stop_token``,
        src/runtime.rs:3869-3892, asks its tokenizer; here config.json gives them, together
        with the folder's generation_config.json where it has one)."""
        ids = list(self.model.spec.eos_token_id)
        ids.extend(t for t in self._extra_stop_ids if t not in ids)
        return tuple(ids)

    # ------------------------------------------------------------------ lower level
    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None) -> SequenceCache:
        """Replace the runner's cache by one that holds ``max_tokens`` tokens."""
        self.cache = self.model.new_cache(max_tokens, max_slots=max_slots,
                                          max_seq_len=self.model.spec.max_position_embeddings)
        self.engine = Engine(self.model, self.cache)
        return self.cache

    def step(self, slots, tokens, want="last"):
        return self.engine.step(slots, tokens, want)

    def warm_up(self, batch_sizes: Sequence[int]) -> None:
        """Capture the decode step for these batch sizes ahead of the first request."""
        with self._generation_lock:
            self.engine.warm_up(batch_sizes)
            torch.cuda.synchronize(self.runtime.device)

    # ------------------------------------------------------------------ generation
    def generate(self, prompt: Union[Sequence[int], Sequence[Sequence[int]]],
                 options: Optional[GenerationOptions] = None,
                 seeds: Optional[Sequence[int]] = None,
                 on_token: Optional[Callable[[int, int], None]] = None):
        """Generate for one prompt (a list of token ids; returns one
        ``GenerationResult``) or for several (a list of lists; returns a list).

        Several prompts run as batches of at most ``max_batch`` sequences that fit the
        cache, one batch after another.  Sequence i draws from its own generator,
        seeded ``seeds[i]`` or ``options.seed + i`` (the reference's benchmark seeds
        its runs the same way, src/main.rs:1507-1510); a seed of 0 is taken from the
        clock as in the reference.  ``on_token(i, token)`` is called as tokens come.
        """
        options = options or GenerationOptions()
        options.validate()
        single = len(prompt) > 0 and not isinstance(prompt[0], (list, tuple))
        prompts: List[List[int]] = [list(prompt)] if single else [list(p) for p in prompt]
        if not prompts:
            raise ValueError("No prompt provided.")
        if seeds is None:
            base = options.seed if options.seed != 0 else (time.time_ns() & ((1 << 63) - 1))
            seeds = [(base + i) & ((1 << 64) - 1) for i in range(len(prompts))]
        elif len(seeds) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(seeds)} seeds")
        max_seq = self.cache.max_seq_len
        if options.max_context is not None:
            max_seq = min(max_seq, options.max_context)
        with self._generation_lock:
            batches = plan_batches([len(p) for p in prompts], options.max_tokens, self.max_batch,
                                   self.cache.free_pages, max_seq)
            results: List[Optional[GenerationResult]] = [None] * len(prompts)
            dev = self.runtime.device
            for batch in batches:
                cb = None
                if on_token is not None:
                    cb = (lambda j, tok, _b=batch: on_token(_b[j], tok))
                rs = generate_batch(self.engine, self.sampler, [prompts[i] for i in batch], options,
                                    [seeds[i] for i in batch], self.stop_token_ids(), max_seq,
                                    on_token=cb, sync=lambda: torch.cuda.synchronize(dev))
                for i, r in zip(batch, rs):
                    results[i] = r
            kernels.check_device_errors()      # a kernel that gave up waiting must not pass silently
            bad = getattr(self.model.embedding, "bad_token", None)
            if bad is not None and int(bad.item()) != 0:
                bad.zero_()
                raise RuntimeError("a token id outside the vocabulary reached the device")
        return results[0] if single else results

    def generate_stream(self, prompt: Sequence[int], options: Optional[GenerationOptions],
                        on_token: Callable[[int], None]) -> GenerationResult:
        """One prompt, tokens handed to ``on_token`` as they are produced
        (the reference's ``generate_stream``, src/runtime.rs:3053-3064)."""
        return self.generate(list(prompt), options, on_token=lambda _i, tok: on_token(tok))
