"""Typed configuration of the dense Llama decoder, read from ``config.json``.

The reference engine has no configuration file: it derives every size from
weight shapes (``src/cli.cpp:57-143``) and fixes rope theta, the RMSNorm
epsilon, the end-of-sequence id and the cache geometry in code
(``src/layers/attention.cpp:68``, ``include/stratakv/layers/rmsnorm.h:13-16``,
``src/cli.cpp:276-279``).  Here every one of those numbers comes from the
model folder's ``config.json``; the validation rules are those of
``src/generation/generator.cpp:156-189`` (non-zero sizes, query heads a
multiple of KV heads) plus refusals for options this decoder does not
implement.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any, Mapping, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that is malformed or asks for something unsupported."""


def _need(raw: Mapping[str, Any], key: str, kind):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return _typed(raw, key, kind)


def _typed(raw: Mapping[str, Any], key: str, kind):
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {value!r}")
        value = float(value)
        if not math.isfinite(value):
            raise ConfigError(f"config.json: '{key}' must be finite, got {value!r}")
        return value
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {value!r}")
        return value
    raise TypeError(kind)


def _optional(raw, key, kind, default):
    if key not in raw or raw[key] is None:
        return default
    return _typed(raw, key, kind)


# What the published Llama configuration schema says a checkpoint means when
# its config.json leaves a key out.  They are the schema's defaults, not sizes
# of any model: a key that config.json gives always wins.
SCHEMA_DEFAULTS = {"rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 2048}


@dataclass(frozen=True)
class LlamaConfig:
    """Sizes and constants of one Llama checkpoint (keys of its ``config.json``)."""

    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    bos_token_id: int | None = None
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str | None = None
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)

    # ---- derived sizes -------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        """Query heads that share one KV head (``src/layers/attention.cpp:50-53``)."""
        return self.num_attention_heads // self.num_key_value_heads

    def parameter_count(self) -> int:
        per_layer = (2 * self.hidden_size
                     + self.hidden_size * (self.q_dim + 2 * self.kv_dim)
                     + self.q_dim * self.hidden_size
                     + 3 * self.hidden_size * self.intermediate_size)
        head = 0 if self.tie_word_embeddings else self.vocab_size * self.hidden_size
        return (self.num_hidden_layers * per_layer + self.vocab_size * self.hidden_size
                + self.hidden_size + head)

    # ---- parsing -------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        if not isinstance(raw, Mapping):
            raise ConfigError("config.json: top level must be an object")
        archs = raw.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
        hidden = _need(raw, "hidden_size", int)
        heads = _need(raw, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        kv_heads = _optional(raw, "num_key_value_heads", int, heads)
        head_dim = _optional(raw, "head_dim", int, None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("config.json: 'eos_token_id' must be an integer or a list of integers")
        known = {
            "architectures", "hidden_size", "intermediate_size", "num_hidden_layers",
            "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
            "rms_norm_eps", "rope_theta", "max_position_embeddings", "tie_word_embeddings",
            "hidden_act", "bos_token_id", "eos_token_id", "torch_dtype", "dtype",
            "attention_bias", "mlp_bias", "rope_scaling", "rope_parameters",
        }
        rope_theta = _optional(raw, "rope_theta", float, None)
        rope_parameters = raw.get("rope_parameters")
        if rope_parameters is not None:
            if not isinstance(rope_parameters, Mapping):
                raise ConfigError("config.json: 'rope_parameters' must be an object")
            if rope_parameters.get("rope_type", "default") != "default":
                raise ConfigError("config.json: rope_parameters.rope_type "
                                  f"'{rope_parameters.get('rope_type')}' is not supported (default only)")
            if rope_theta is None and rope_parameters.get("rope_theta") is not None:
                rope_theta = _typed(rope_parameters, "rope_theta", float)
        if rope_theta is None:
            rope_theta = SCHEMA_DEFAULTS["rope_theta"]
        config = cls(
            architecture=archs[0],
            hidden_size=hidden,
            intermediate_size=_need(raw, "intermediate_size", int),
            num_hidden_layers=_need(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_need(raw, "vocab_size", int),
            rms_norm_eps=_optional(raw, "rms_norm_eps", float, SCHEMA_DEFAULTS["rms_norm_eps"]),
            rope_theta=rope_theta,
            max_position_embeddings=_optional(raw, "max_position_embeddings", int,
                                              SCHEMA_DEFAULTS["max_position_embeddings"]),
            tie_word_embeddings=_optional(raw, "tie_word_embeddings", bool, False),
            hidden_act=_optional(raw, "hidden_act", str, "silu"),
            bos_token_id=_optional(raw, "bos_token_id", int, None),
            eos_token_ids=eos_ids,
            torch_dtype=_optional(raw, "torch_dtype", str, _optional(raw, "dtype", str, None)),
            extra={k: v for k, v in raw.items() if k not in known},
        )
        for flag in ("attention_bias", "mlp_bias"):
            if _optional(raw, flag, bool, False):
                raise ConfigError(f"config.json: '{flag}': true is not supported "
                                  "(this decoder's projections have no bias)")
        if raw.get("rope_scaling") is not None:
            raise ConfigError("config.json: 'rope_scaling' is not supported; it must be null or absent")
        config.validate()
        return config

    @classmethod
    def from_file(cls, path) -> "LlamaConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        try:
            raw = json.loads(path.read_text())
        except FileNotFoundError:
            raise ConfigError(f"no config.json at {path}") from None
        except json.JSONDecodeError as error:
            raise ConfigError(f"{path}: not valid JSON ({error})") from None
        return cls.from_dict(raw)

    def validate(self) -> None:
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: '{name}' must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a "
                f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act not in ("silu", "swish"):
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if self.vocab_size > 2**31 - 1:
            raise ConfigError("config.json: vocab_size exceeds the 32-bit token id range")
        for eos in self.eos_token_ids:
            if not (0 <= eos < self.vocab_size):
                raise ConfigError(f"config.json: eos_token_id {eos} is outside the vocabulary")
        if self.bos_token_id is not None and not (0 <= self.bos_token_id < self.vocab_size):
            raise ConfigError(f"config.json: bos_token_id {self.bos_token_id} is outside the vocabulary")

    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
        }
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.torch_dtype is not None:
            out["torch_dtype"] = self.torch_dtype
        return out

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2) + "\n"
