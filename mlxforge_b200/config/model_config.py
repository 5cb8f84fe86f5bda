"""Typed model configuration read from an architecture's own ``config.json`` keys.

The dense-decoder subset of the reference's ``ModelConfig``
(src/core/config.h:72-204, parsed in src/core/config.cpp:134-228).  Error texts
for a missing or mistyped required field follow src/core/config.cpp:16-28, the
rope-scaling object follows src/core/config.cpp:53-78 and its validation
src/core/config.cpp:246-280.

Nothing in the engine hard-codes a size: every part receives its sizes and
constants from an instance of this class (through the architecture's builder).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


_MISSING = object()


def _require(j: Dict[str, Any], key: str, kind: type):
    """Fetch a required key with the reference's error wording (src/core/config.cpp:16-28)."""
    v = j.get(key, _MISSING)
    if v is _MISSING:
        raise ConfigError(f"config.json: missing required field '{key}'")
    return _typed(key, v, kind)


def _typed(key: str, v: Any, kind: type):
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                return int(v)
            raise ConfigError(
                f"config.json: field '{key}' has wrong type: expected integer, got {type(v).__name__}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(
                f"config.json: field '{key}' has wrong type: expected number, got {type(v).__name__}")
        return float(v)
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(
                f"config.json: field '{key}' has wrong type: expected boolean, got {type(v).__name__}")
        return v
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(
                f"config.json: field '{key}' has wrong type: expected string, got {type(v).__name__}")
        return v
    raise TypeError(kind)


def _optional(j: Dict[str, Any], key: str, kind: type, default):
    """Absent or explicit null gives the default (src/core/config.cpp:33-38)."""
    v = j.get(key, None)
    if v is None:
        return default
    return _typed(key, v, kind)


@dataclass(frozen=True)
class RopeScaling:
    """The ``rope_scaling`` object (src/core/config.h:26-37)."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_position_embeddings: int = 0

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "RopeScaling":
        # type from "rope_type", else legacy "type", else "default" (src/core/config.cpp:53-57)
        t = o.get("rope_type", o.get("type", "")) or "default"
        if not isinstance(t, str):
            raise ConfigError("config.json: field 'rope_scaling.rope_type' has wrong type: expected string")
        return RopeScaling(
            rope_type=t,
            factor=_optional(o, "factor", float, 1.0),
            low_freq_factor=_optional(o, "low_freq_factor", float, 1.0),
            high_freq_factor=_optional(o, "high_freq_factor", float, 1.0),
            original_max_position_embeddings=_optional(o, "original_max_position_embeddings", int, 0),
        )

    def to_json(self) -> Dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


SUPPORTED_ROPE_TYPES = ("default", "llama3", "linear")


def validate_rope_scaling(rs: Optional[RopeScaling]) -> None:
    """Reject what the position encoding cannot compute; never fall through silently.

    The reference accepts default/llama3 always and yarn/linear conditionally
    (src/core/config.cpp:246-280).  This engine computes default, llama3 and
    linear; for llama3 it also checks the constants the formula divides by.
    """
    if rs is None:
        return
    t = rs.rope_type
    if t not in SUPPORTED_ROPE_TYPES:
        raise ConfigError(
            f"unsupported rope_scaling rope_type '{t}' (supported: {', '.join(SUPPORTED_ROPE_TYPES)})")
    if t in ("llama3", "linear") and not (rs.factor > 0.0 and math.isfinite(rs.factor)):
        raise ConfigError(f"rope_scaling '{t}' requires factor > 0")
    if t == "llama3":
        if rs.original_max_position_embeddings <= 0:
            raise ConfigError("rope_scaling 'llama3' requires original_max_position_embeddings > 0")
        if rs.low_freq_factor <= 0.0 or rs.high_freq_factor <= 0.0:
            raise ConfigError("rope_scaling 'llama3' requires low_freq_factor > 0 and high_freq_factor > 0")
        if rs.high_freq_factor == rs.low_freq_factor:
            raise ConfigError("rope_scaling 'llama3' requires high_freq_factor != low_freq_factor")


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's typed configuration: the name the registry
    dispatches on and the raw json it was parsed from."""

    architecture: str
    raw: Dict[str, Any] = field(compare=False, repr=False, default_factory=dict)

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "ModelConfig":  # pragma: no cover - overridden
        raise NotImplementedError


def architecture_name(j: Dict[str, Any]) -> str:
    archs = j.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: missing required field 'architectures' (a list naming the model class)")
    return archs[0]


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """Hyper-parameters of the dense GQA decoder (``LlamaForCausalLM``).

    Keys, defaults and requiredness follow src/core/config.cpp:146-168.
    ``attention_bias`` / ``mlp_bias`` / ``hidden_act`` are not read by the
    reference (it never loads a bias and hard-codes SiLU,
    src/model/decoder_model.cpp:277-282); a config that sets them to something
    this decoder does not compute is refused here rather than run wrongly.
    """

    num_hidden_layers: int = 0
    hidden_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    vocab_size: int = 0
    intermediate_size: int = 0
    rope_theta: float = 0.0
    rms_norm_eps: float = 0.0
    head_dim: int = 0
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = True
    bos_token_id: int = -1
    eos_token_ids: tuple = ()
    rope_scaling: Optional[RopeScaling] = None
    model_type: str = ""

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "LlamaConfig":
        if not isinstance(j, dict):
            raise ConfigError("config.json: top level must be an object")
        arch = architecture_name(j)
        n_layers = _require(j, "num_hidden_layers", int)
        hidden = _require(j, "hidden_size", int)
        n_heads = _require(j, "num_attention_heads", int)
        n_kv = _require(j, "num_key_value_heads", int)
        vocab = _require(j, "vocab_size", int)
        inter = _require(j, "intermediate_size", int)
        # rope_theta: nested rope_parameters.rope_theta wins (src/core/config.cpp:83-88)
        rp = j.get("rope_parameters")
        if isinstance(rp, dict) and "rope_theta" in rp:
            theta = _typed("rope_parameters.rope_theta", rp["rope_theta"], float)
        else:
            theta = _require(j, "rope_theta", float)
        eps = _require(j, "rms_norm_eps", float)
        for name, v in (("num_hidden_layers", n_layers), ("hidden_size", hidden),
                        ("num_attention_heads", n_heads), ("num_key_value_heads", n_kv),
                        ("vocab_size", vocab), ("intermediate_size", inter)):
            if v <= 0:
                raise ConfigError(f"config.json: field '{name}' must be positive, got {v}")
        head_dim = _optional(j, "head_dim", int, hidden // n_heads)
        if head_dim <= 0:
            raise ConfigError(f"config.json: field 'head_dim' must be positive, got {head_dim}")
        if n_heads % n_kv != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({n_heads}) must be a multiple of "
                f"num_key_value_heads ({n_kv})")
        if not (theta > 0.0 and math.isfinite(theta)):
            raise ConfigError(f"config.json: field 'rope_theta' must be positive, got {theta}")
        if not (eps >= 0.0 and math.isfinite(eps)):
            raise ConfigError(f"config.json: field 'rms_norm_eps' must be non-negative, got {eps}")

        eos = j.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, list):
            eos_ids = tuple(_typed("eos_token_id", e, int) for e in eos)
        else:
            eos_ids = (_typed("eos_token_id", eos, int),)

        rs = None
        for key in ("rope_scaling", "rope_parameters"):
            o = j.get(key)
            if isinstance(o, dict):
                rs = RopeScaling.from_json(o)
                break
        validate_rope_scaling(rs)

        if _optional(j, "attention_bias", bool, False):
            raise ConfigError("config.json: attention_bias=true is not supported by this decoder (no bias terms)")
        if _optional(j, "mlp_bias", bool, False):
            raise ConfigError("config.json: mlp_bias=true is not supported by this decoder (no bias terms)")
        act = _optional(j, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (the feed-forward is SiLU-gated)")

        return cls(
            architecture=arch, raw=dict(j),
            num_hidden_layers=n_layers, hidden_size=hidden, num_attention_heads=n_heads,
            num_key_value_heads=n_kv, vocab_size=vocab, intermediate_size=inter,
            rope_theta=theta, rms_norm_eps=eps, head_dim=head_dim,
            max_position_embeddings=_optional(j, "max_position_embeddings", int, 0),
            tie_word_embeddings=_optional(j, "tie_word_embeddings", bool, True),
            bos_token_id=_optional(j, "bos_token_id", int, -1),
            eos_token_ids=eos_ids, rope_scaling=rs,
            model_type=_optional(j, "model_type", str, ""),
        )

    def to_json(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        j: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type or "llama",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "intermediate_size": self.intermediate_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.bos_token_id >= 0:
            j["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            j["eos_token_id"] = list(self.eos_token_ids)
        if self.rope_scaling is not None:
            j["rope_scaling"] = self.rope_scaling.to_json()
        return j


def apply_rope_scaling_override(j: Dict[str, Any], text: str) -> Dict[str, Any]:
    """``j`` with its ``rope_scaling`` replaced wholesale by the JSON object in ``text`` (a full
    replacement, not a merge; src/core/config.cpp:282-300).  The type is validated when the
    result is parsed."""
    try:
        o = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"invalid rope_scaling override JSON: {e}")
    if not isinstance(o, dict):
        raise ConfigError('rope_scaling override must be a JSON object, e.g. {"rope_type":"linear","factor":4.0}')
    j = dict(j)
    j["rope_scaling"] = o
    return j


def read_config_json(path: str) -> Dict[str, Any]:
    """Read ``config.json`` (a file, or the folder holding it) with the
    reference's file errors (src/core/config.cpp:232-244)."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
    except OSError:
        raise ConfigError(f"config.json: cannot open file '{path}'")
    try:
        j = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"config.json: parse error in '{path}': {e}")
    if not isinstance(j, dict):
        raise ConfigError(f"config.json: parse error in '{path}': top level must be an object")
    return j
