"""rustyllm_b200: a small model library with generation for NVIDIA B200 (sm_100a),
after SimonWaldherr/RustyLLM's Llama dense decoder.

    from rustyllm_b200 import Runner, GenerationOptions, SamplerConfig
    runner, info = Runner.from_path("model_dir", dtype="bfloat16")
    result = runner.generate([1, 2, 3], GenerationOptions(max_tokens=8, sampler=SamplerConfig.greedy()))
"""
from .config.files import ConfigError  # noqa: F401
from .config.llama import LlamaConfig, RopeScaling  # noqa: F401
from .config.registry import (UnknownArchitecture, known_architectures, register_architecture,  # noqa: F401
                              resolve_architecture)
from .config.spec import LayerSpec, ModelSpec, ParamSource, ParamSpec, PartSpec  # noqa: F401
from .engine.generate import GenerationOptions, GenerationResult, GenerationStats  # noqa: F401
from .engine.runner import LoadInfo, Runner  # noqa: F401
from .engine.step import Engine  # noqa: F401
from .models import llama as _llama  # noqa: F401  (registers the architecture)
from .sampling.config import Rng, SamplerConfig  # noqa: F401
from .weights.loader import WeightsError  # noqa: F401
from .weights.random_init import write_random_model  # noqa: F401

__version__ = "0.1.0"
