"""Typed model configuration for the Qwen3 dense decoder, read from a Hugging Face ``config.json``.

Key names, defaults and fall-backs follow the reference's ``ModelConfig::from_hf_json``
(config.h:34-59): ``hidden_size``, ``num_hidden_layers``, ``num_attention_heads``, ``vocab_size`` and
``intermediate_size`` are required; ``num_key_value_heads`` defaults to the number of query heads,
``head_dim`` to ``hidden_size / num_attention_heads`` (so ``heads * head_dim`` may differ from the
hidden size), ``rms_norm_eps`` to 1e-6, ``max_position_embeddings`` to 40960, ``tie_word_embeddings``
to false.  Two deliberate differences: ``rope_theta`` is honoured as a top-level key as well as under
``rope_parameters`` (the reference reads only the latter, config.h:50-52), and ``eos_token_id`` may be
a scalar as well as a list (the reference ignores a scalar, config.h:54-56).

No size of the model is written anywhere else in the package: every part receives its sizes from an
instance of this class through the architecture's builder.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that cannot describe a model: a missing key, a bad value or an unknown architecture."""


def _require(d: Mapping[str, Any], key: str, typ=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    try:
        return typ(d[key])
    except (TypeError, ValueError) as e:
        raise ConfigError(f"config.json: key '{key}' has a bad value {d[key]!r}") from e


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    eos_token_ids: tuple = (151645,)
    bos_token_id: int = 151643
    architecture: str = "Qwen3ForCausalLM"

    # ---- derived -------------------------------------------------------------------------------------
    @property
    def gqa_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ---- construction --------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        hidden = _require(d, "hidden_size")
        layers = _require(d, "num_hidden_layers")
        heads = _require(d, "num_attention_heads")
        vocab = _require(d, "vocab_size")
        inter = _require(d, "intermediate_size")
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive")
        kv_heads = int(d["num_key_value_heads"]) if d.get("num_key_value_heads") is not None else heads
        if d.get("head_dim") is not None:
            head_dim = int(d["head_dim"])
        else:
            if hidden % heads:
                raise ConfigError("config.json: hidden_size is not divisible by num_attention_heads "
                                  "and no head_dim is given")
            head_dim = hidden // heads

        theta = 1000000.0
        rp = d.get("rope_parameters")
        if isinstance(rp, Mapping) and rp.get("rope_theta") is not None:
            theta = float(rp["rope_theta"])
        if d.get("rope_theta") is not None:
            theta = float(d["rope_theta"])

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids = (151645,)
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(t) for t in eos)
        else:
            eos_ids = (int(eos),)

        arch = "Qwen3ForCausalLM"
        if isinstance(d.get("architectures"), (list, tuple)) and d["architectures"]:
            arch = str(d["architectures"][0])

        cfg = cls(
            hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter, vocab_size=vocab,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6) if d.get("rms_norm_eps") is not None else 1e-6),
            rope_theta=theta,
            max_position_embeddings=int(d.get("max_position_embeddings") or 40960),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
            bos_token_id=int(d["bos_token_id"]) if d.get("bos_token_id") is not None else 151643,
            architecture=arch,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        pos = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
               "intermediate_size", "vocab_size", "max_position_embeddings")
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"config.json: {k} must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary embedding")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if not (self.rope_theta > 0):
            raise ConfigError("config.json: rope_theta must be positive")

    def to_dict(self) -> dict:
        """The config.json form of this configuration (the keys the parser reads)."""
        return {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "eos_token_id": list(self.eos_token_ids),
            "bos_token_id": self.bos_token_id,
            "hidden_act": "silu",
            "torch_dtype": "bfloat16",
        }


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: the top level must be a JSON object")
    return d
