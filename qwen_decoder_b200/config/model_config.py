"""Typed model configuration, read from a model folder's ``config.json``.

The reference keeps eight numbers in ``struct Config`` (common.h:15-24) and fills
them from GGUF metadata (common.cpp:38-91); several constants of the model are
literals in its kernels (RMSNorm eps, gpu_kernels.cu:63; head size = dim / heads,
gpu_decoder.cu:265).  Here every such number is a configuration key: nothing that
``config.json`` gives stands in code.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a typed configuration."""


_MISSING = object()


def _get(d: Mapping[str, Any], key: str, kind, default=_MISSING):
    """Fetch ``key`` with a type check; the error names the key."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
        return v
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {v!r}")
        return v
    raise AssertionError(kind)


@dataclass(frozen=True)
class Qwen2Config:
    """Configuration of the Qwen2.5 dense decoder (``Qwen2ForCausalLM``).

    Key names are those of the architecture's own ``config.json``.  The
    correspondence with the reference's GGUF metadata is (common.cpp:65-79):
    hidden_size = qwen2.embedding_length, intermediate_size =
    qwen2.feed_forward_length, num_hidden_layers = qwen2.block_count,
    num_attention_heads = qwen2.attention.head_count, num_key_value_heads =
    qwen2.attention.head_count_kv, max_position_embeddings = qwen2.context_length,
    rope_theta = qwen2.rope.freq_base, vocab_size = rows of token_embd.weight.
    """

    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    # Which elements of a head rotate together.  "half" pairs (p, p + d/2): what checkpoints of this
    # architecture in safetensors form are trained with, hence the default.  "adjacent" pairs (2p, 2p+1),
    # as the reference rotates the tensors of its own file format (gpu_kernels.cu:94-100,
    # cpu_decoder.cpp:135-146); the optional key ``rope_pairing`` selects it.
    rope_pairing: str = "half"
    attention_bias: bool = True  # q, k, v carry a bias (gpu_decoder.cu:347-349)
    eos_token_ids: tuple = ()
    torch_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    # ---- derived sizes -------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ---- construction --------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        archs = d.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of strings")
        hidden = _get(d, "hidden_size", int)
        heads = _get(d, "num_attention_heads", int)
        kv_heads = _get(d, "num_key_value_heads", int, heads)
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads != 0:
            raise ConfigError(
                f"config.json: 'num_key_value_heads' ({kv_heads}) must divide "
                f"'num_attention_heads' ({heads})")
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _get(d, "head_dim", int)
        else:
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: 'hidden_size' ({hidden}) is not a multiple of "
                    f"'num_attention_heads' ({heads}) and no 'head_dim' is given")
            head_dim = hidden // heads
        if head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' ({head_dim}) must be a positive even number")
        if _get(d, "use_sliding_window", bool, False):
            raise ConfigError(
                "config.json: 'use_sliding_window' = true is not supported for "
                "Qwen2ForCausalLM (the reference decoder has no windowed layers)")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: 'rope_scaling' is not supported for Qwen2ForCausalLM")
        act = _get(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu', got {act!r}")
        pairing = _get(d, "rope_pairing", str, "half")
        if pairing not in ("adjacent", "half"):
            raise ConfigError(f"config.json: 'rope_pairing' must be 'adjacent' or 'half', got {pairing!r}")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("config.json: 'eos_token_id' must be an integer or a list of integers")
        cfg = cls(
            architecture=archs[0],
            hidden_size=hidden,
            intermediate_size=_get(d, "intermediate_size", int),
            num_hidden_layers=_get(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_get(d, "vocab_size", int),
            max_position_embeddings=_get(d, "max_position_embeddings", int),
            rope_theta=_get(d, "rope_theta", float),
            rms_norm_eps=_get(d, "rms_norm_eps", float),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            hidden_act=act,
            rope_pairing=pairing,
            attention_bias=_get(d, "attention_bias", bool, True),
            eos_token_ids=eos_ids,
            torch_dtype=_get(d, "torch_dtype", str, "bfloat16"),
        )
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size",
                     "max_position_embeddings"):
            if getattr(cfg, name) <= 0:
                raise ConfigError(f"config.json: '{name}' must be positive, got {getattr(cfg, name)}")
        if cfg.rope_theta <= 0:
            raise ConfigError("config.json: 'rope_theta' must be positive")
        if cfg.rms_norm_eps <= 0:
            raise ConfigError("config.json: 'rms_norm_eps' must be positive")
        return cfg

    def to_dict(self) -> dict:
        """The ``config.json`` form of this configuration."""
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "rope_pairing": self.rope_pairing,
            "attention_bias": self.attention_bias,
            "use_sliding_window": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def read_config_json(model_dir: str) -> dict:
    """Parse ``<model_dir>/config.json`` into a plain dict."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder {model_dir!r}")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def write_config_json(config, model_dir: str) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
        f.write("\n")


__all__ = ["ConfigError", "Qwen2Config", "read_config_json", "write_config_json", "asdict"]
