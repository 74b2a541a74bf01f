"""Typed configuration of the Llama dense decoder, read from config.json keys.

Counterpart of the reference's ``Config`` (src/model.rs:19-39) and
``Config::from_gguf`` (src/model.rs:43-120).  The reference fills the same
fields from GGUF metadata; here they come from the architecture's own
config.json keys.  Defaults follow the reference where it has one:
``num_key_value_heads`` = heads, ``head_dim`` = hidden/heads (src/model.rs:69-74),
context 2048 (src/model.rs:105), ``rope_theta`` 10000 and ``rms_norm_eps`` 1e-5.
Every size the model uses lives here; nothing downstream hard-codes one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .files import ConfigError, token_ids as _token_ids


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of rotary embeddings (``rope_type`` "llama3")."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> dict:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


def _require_int(d: Mapping[str, Any], key: str) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks required key '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config key '{key}' must be an integer, got {v!r}")
    if v <= 0:
        raise ConfigError(f"config key '{key}' must be > 0, got {v}")
    return v


def _opt_int(d: Mapping[str, Any], key: str, default: Optional[int]) -> Optional[int]:
    v = d.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config key '{key}' must be an integer, got {v!r}")
    if v <= 0:
        raise ConfigError(f"config key '{key}' must be > 0, got {v}")
    return v


def _opt_float(d: Mapping[str, Any], key: str, default: float) -> float:
    v = d.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config key '{key}' must be a number, got {v!r}")
    return float(v)


def parse_rope_scaling(raw: Any) -> Optional[RopeScaling]:
    """``rope_scaling`` (or the scaling fields of ``rope_parameters``) -> RopeScaling.

    ``None``, a missing ``rope_type`` or ``"default"`` mean no scaling.  Only
    "llama3" is known; anything else is refused instead of being ignored,
    because ignoring it would silently change every rotation angle.
    """
    if raw is None:
        return None
    if not isinstance(raw, Mapping):
        raise ConfigError(f"rope_scaling must be an object or null, got {raw!r}")
    rope_type = raw.get("rope_type", raw.get("type"))
    if rope_type is None or rope_type == "default":
        return None
    if rope_type != "llama3":
        raise ConfigError(f"unknown rope_type {rope_type!r}; known: 'default', 'llama3'")
    missing = [k for k in ("factor", "low_freq_factor", "high_freq_factor",
                           "original_max_position_embeddings") if raw.get(k) is None]
    if missing:
        raise ConfigError(f"rope_scaling of type 'llama3' lacks {missing}")
    sc = RopeScaling(
        rope_type="llama3",
        factor=float(raw["factor"]),
        low_freq_factor=float(raw["low_freq_factor"]),
        high_freq_factor=float(raw["high_freq_factor"]),
        original_max_position_embeddings=int(raw["original_max_position_embeddings"]),
    )
    if sc.factor <= 0 or sc.original_max_position_embeddings <= 0:
        raise ConfigError("rope_scaling factor and original_max_position_embeddings must be > 0")
    if sc.high_freq_factor <= sc.low_freq_factor:
        raise ConfigError("rope_scaling needs high_freq_factor > low_freq_factor")
    return sc


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    bos_token_id: Tuple[int, ...] = ()
    eos_token_id: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    architectures: Tuple[str, ...] = ("LlamaForCausalLM",)
    model_type: str = "llama"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ---- derived sizes (src/model.rs:69-74, 3718-3719) ----
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotary pairs")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"rope_theta must be > 0, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported; known: 'silu'")
        for name, ids in (("bos_token_id", self.bos_token_id), ("eos_token_id", self.eos_token_id)):
            for t in ids:
                if t < 0 or t >= self.vocab_size:
                    raise ConfigError(f"{name} {t} lies outside the vocabulary [0, {self.vocab_size})")

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        hidden = _require_int(d, "hidden_size")
        heads = _require_int(d, "num_attention_heads")
        kv_heads = _opt_int(d, "num_key_value_heads", heads)
        head_dim = _opt_int(d, "head_dim", None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"hidden_size ({hidden}) is no multiple of num_attention_heads ({heads}) "
                    "and config.json gives no head_dim")
            head_dim = hidden // heads
        # transformers >= 5 writes rope_theta and the scaling fields into one
        # "rope_parameters" object; older files have rope_theta + rope_scaling.
        rope_params = d.get("rope_parameters")
        rope_theta = _opt_float(d, "rope_theta", 10000.0)
        scaling_raw = d.get("rope_scaling")
        if isinstance(rope_params, Mapping):
            if rope_params.get("rope_theta") is not None:
                rope_theta = float(rope_params["rope_theta"])
            if scaling_raw is None:
                scaling_raw = rope_params
        # keys of other architectures that would change the arithmetic if they meant anything here:
        # refused rather than ignored
        if d.get("partial_rotary_factor") not in (None, 1, 1.0):
            raise ConfigError(f"partial_rotary_factor = {d['partial_rotary_factor']!r}: this architecture rotates the whole head")
        if d.get("sliding_window") is not None:
            raise ConfigError(f"sliding_window = {d['sliding_window']!r}: this architecture attends to the whole context")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            raise ConfigError(f"torch_dtype {dtype!r} is not one of bfloat16, float32, float16")
        archs = d.get("architectures") or ("LlamaForCausalLM",)
        known = {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                 "num_attention_heads", "num_key_value_heads", "head_dim",
                 "max_position_embeddings", "rms_norm_eps", "rope_theta", "rope_scaling",
                 "rope_parameters", "tie_word_embeddings", "attention_bias", "mlp_bias",
                 "hidden_act", "bos_token_id", "eos_token_id", "torch_dtype", "dtype",
                 "architectures", "model_type"}
        cfg = cls(
            vocab_size=_require_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_require_int(d, "intermediate_size"),
            num_hidden_layers=_require_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_opt_int(d, "max_position_embeddings", 2048),
            rms_norm_eps=_opt_float(d, "rms_norm_eps", 1e-5),
            rope_theta=rope_theta,
            rope_scaling=parse_rope_scaling(scaling_raw),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
            hidden_act=d.get("hidden_act", "silu"),
            bos_token_id=_token_ids(d, "bos_token_id"),
            eos_token_id=_token_ids(d, "eos_token_id"),
            torch_dtype=dtype,
            architectures=tuple(archs),
            model_type=d.get("model_type", "llama"),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.bos_token_id:
            d["bos_token_id"] = self.bos_token_id[0] if len(self.bos_token_id) == 1 else list(self.bos_token_id)
        if self.eos_token_id:
            d["eos_token_id"] = self.eos_token_id[0] if len(self.eos_token_id) == 1 else list(self.eos_token_id)
        return d
