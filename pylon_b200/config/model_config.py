"""Typed model configurations read from a checkpoint's ``config.json``.

Every size and constant of a model comes from here; no part of the engine carries a
size of its own.  A configuration class knows two things: how to read its architecture's
``config.json`` keys (and which options it refuses), and how to describe the model as an
architecture-neutral :class:`~pylon_b200.parts.spec.ModelSpec` that the part builders use.

Reference parity: the field list follows ``src/pylon/model/config.py:20-32`` and the
refusals follow ``src/pylon/model/config.py:35-62``; unlike the reference, no shape is
pinned to the Qwen3-4B checkpoint.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, ClassVar, Mapping


class ConfigError(ValueError):
    """A config.json that is malformed or asks for something the engine does not build."""


def _require(data: Mapping[str, Any], key: str, kind: type | tuple[type, ...]) -> Any:
    if key not in data:
        raise ConfigError(f"config.json has no '{key}'")
    value = data[key]
    if isinstance(value, bool) and kind is not bool:
        raise ConfigError(f"config.json '{key}' must be {kind}, got a bool")
    if not isinstance(value, kind):
        raise ConfigError(f"config.json '{key}' must be {kind}, got {type(value).__name__}")
    return value


def _positive_int(data: Mapping[str, Any], key: str) -> int:
    value = _require(data, key, int)
    if value < 1:
        raise ConfigError(f"config.json '{key}' must be positive, got {value}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    """Qwen3 dense decoder (``Qwen3ForCausalLM``).

    Field names are the checkpoint's own config.json keys.
    """

    architecture: ClassVar[str] = "Qwen3ForCausalLM"
    model_type: ClassVar[str] = "qwen3"

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)
    torch_dtype: str = "bfloat16"

    def __post_init__(self) -> None:
        for name in (
            "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "intermediate_size", "max_position_embeddings",
        ):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value < 1:
                raise ConfigError(f"{name} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")

    # -- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen3Config":
        if data.get("model_type", cls.model_type) != cls.model_type:
            raise ConfigError(f"model_type must be '{cls.model_type}', got {data.get('model_type')!r}")
        # Options of the checkpoint format that this architecture's engine does not build.
        if data.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {data.get('hidden_act')!r} is not supported (silu only)")
        if data.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported")
        if data.get("rope_scaling") is not None:
            raise ConfigError("rope_scaling is not supported")
        if data.get("use_sliding_window", False):
            raise ConfigError("use_sliding_window=true is not supported")
        if data.get("sliding_window") is not None:   # refused as raun6k/Pylon refuses it (src/pylon/model/config.py:48), whatever use_sliding_window says
            raise ConfigError(f"sliding_window={data.get('sliding_window')!r} is not supported (Qwen3 dense attends to every earlier token)")
        heads = _positive_int(data, "num_attention_heads")
        hidden = _positive_int(data, "hidden_size")
        if "head_dim" in data and data["head_dim"] is not None:
            head_dim = _positive_int(data, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            head_dim = hidden // heads
        kv_heads = data.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else _positive_int(data, "num_key_value_heads")
        eos = data.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(x) for x in eos)
        return cls(
            vocab_size=_positive_int(data, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=_positive_int(data, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_positive_int(data, "intermediate_size"),
            max_position_embeddings=_positive_int(data, "max_position_embeddings"),
            rope_theta=float(_require(data, "rope_theta", (int, float))),
            rms_norm_eps=float(_require(data, "rms_norm_eps", (int, float))),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
            torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen3Config":
        return cls.from_dict(json.loads(Path(path).read_text()))

    # -- writing -----------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        data = asdict(self)
        eos = data.pop("eos_token_ids")
        data["architectures"] = [self.architecture]
        data["model_type"] = self.model_type
        data["hidden_act"] = "silu"
        data["attention_bias"] = False
        data["rope_scaling"] = None
        data["use_sliding_window"] = False
        data["sliding_window"] = None
        if eos:
            data["eos_token_id"] = eos[0] if len(eos) == 1 else list(eos)
        return data

    # -- derived sizes -----------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim
