"""Reading the JSON files of a model folder; nothing here belongs to one architecture.

``config.json`` describes the model (the registry picks the architecture by its
``architectures`` / ``model_type`` keys).  ``generation_config.json``, where a folder
has one, lists the ids that end a generation: instruction-tuned checkpoints name
their end-of-turn ids there and not in config.json.  The reference asks its tokenizer
for these ids (``is_stop_token``, SimonWaldherr/RustyLLM src/runtime.rs:3869-3892); this library
has no tokenizer, so the two files are the source.
"""
from __future__ import annotations

import json
import os
from typing import Any, Mapping, Tuple


class ConfigError(ValueError):
    """A model folder's JSON that cannot describe a model."""


def _read_object(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    return _read_object(path)


def token_ids(d: Mapping[str, Any], key: str) -> Tuple[int, ...]:
    """An id or a list of ids under ``key`` (absent or null: none)."""
    v = d.get(key)
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, (list, tuple)) and all(isinstance(t, int) and not isinstance(t, bool) for t in v):
        return tuple(v)
    raise ConfigError(f"config key '{key}' must be an integer or a list of integers, got {v!r}")


def read_generation_stop_ids(model_dir: str, vocab_size: int) -> Tuple[int, ...]:
    """``eos_token_id`` (an id or a list) of the folder's generation_config.json; ``()``
    if there is no such file.  An id outside the vocabulary is an error."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return ()
    ids = token_ids(_read_object(path), "eos_token_id")
    for t in ids:
        if t < 0 or t >= vocab_size:
            raise ConfigError(f"{path}: eos_token_id {t} lies outside the vocabulary [0, {vocab_size})")
    return ids
