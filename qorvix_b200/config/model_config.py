"""Typed model configuration read from an architecture's own config.json keys.

The reference fills its ModelConfig from GGUF metadata
(runtime/include/qorvix/runtime/model_config.hpp:25-57, runtime/src/model_config.cpp:59-130);
here the source is config.json.  Every size and constant the model code uses comes
from one of these fields; nothing is fixed in code.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


def _require(d: dict, key: str, kind=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    try:
        return kind(d[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: key '{key}' = {d[key]!r} is not a {kind.__name__}") from None


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of config.json.  rope_type 'llama3' is the only scaled kind."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Optional[dict]) -> Optional["RopeScaling"]:
        if not d:
            return None
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"config.json: rope_scaling.rope_type '{kind}' is not supported (known: llama3, default)")
        return RopeScaling(
            rope_type="llama3",
            factor=_require(d, "factor", float),
            low_freq_factor=_require(d, "low_freq_factor", float),
            high_freq_factor=_require(d, "high_freq_factor", float),
            original_max_position_embeddings=_require(d, "original_max_position_embeddings", int),
        )

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration has in common: its name, and what the entry points
    (command line, LLM) read of any model: the vocabulary's size and the ids that end a generation."""
    architecture: str
    vocab_size: int = 0
    eos_token_id: Optional[Any] = None

    @property
    def eos_token_ids(self) -> tuple:
        e = self.eos_token_id
        if e is None:
            return ()
        return tuple(int(x) for x in e) if isinstance(e, (list, tuple)) else (int(e),)


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """Llama dense decoder.  Field names are the config.json keys."""
    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    max_position_embeddings: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Any] = None
    torch_dtype: str = "bfloat16"

    @staticmethod
    def from_dict(d: dict) -> "LlamaConfig":
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        heads = _require(d, "num_attention_heads")
        hidden = _require(d, "hidden_size")
        kv_heads = d.get("num_key_value_heads")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if heads <= 0 or hidden % heads:
                raise ConfigError(f"config.json: hidden_size {hidden} is not divisible by num_attention_heads {heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ConfigError("config.json: attention_bias / mlp_bias are not supported by the Llama dense decoder here")
        cfg = LlamaConfig(
            architecture=str(archs[0]),
            vocab_size=_require(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_require(d, "intermediate_size"),
            num_hidden_layers=_require(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(kv_heads) if kv_heads is not None else heads,
            head_dim=int(head_dim),
            max_position_embeddings=int(d.get("max_position_embeddings") or 0),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id"),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        """Same rules as the reference's valid() (model_config.hpp:52-56) plus the ones the
        rotary encoding and the activation add."""
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (known: silu)")
        if self.rms_norm_eps < 0:
            raise ConfigError("config.json: rms_norm_eps must not be negative")

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["rope_scaling"] = self.rope_scaling.to_dict() if self.rope_scaling else None
        d["model_type"] = "llama"
        return d


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
