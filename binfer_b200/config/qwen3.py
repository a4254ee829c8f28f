"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

Keys and defaults follow the reference's parser (src/model/config.ts:73-192):
``hidden_size``, ``num_attention_heads``, ``intermediate_size``,
``num_hidden_layers`` and ``vocab_size`` are required; ``num_key_value_heads``
defaults to the head count (:108-112), ``head_dim`` to ``hidden_size //
num_attention_heads`` (:115-119), ``rms_norm_eps`` to 1e-5 (:161),
``rope_theta`` to 10000 (:163), ``max_position_embeddings`` to 4096,
``tie_word_embeddings`` to false (:168).  Per-head q/k RMSNorm is on for this
family (:138-141).  Both snake_case and camelCase spellings are accepted
(:75-84).

Unlike the reference, which parses ``sliding_window`` and then never reads it
(src/model/config.ts:102), a window that the file switches on is honoured, and
anything the engine cannot do is refused here with a :class:`ConfigError`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .specs import (AttentionSpec, ConfigError, GatedMLPSpec, LayerSpec,
                    ModelSpec, NameLayout, NormSpec, RopeSpec, ScheduleEntry)

_MISSING = object()


def _camel(key: str) -> str:
    head, *rest = key.split("_")
    return head + "".join(w.capitalize() for w in rest)


def _get(raw: Dict[str, Any], key: str, default: Any = _MISSING) -> Any:
    for k in (key, _camel(key)):
        if k in raw and raw[k] is not None:
            return raw[k]
    if default is _MISSING:
        raise ConfigError(f"Missing required config key: {key}")
    return default


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_factor: float = 1.0
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    qk_norm: bool = True
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None
    eos_token_id: Tuple[int, ...] = (2,)
    bos_token_id: Optional[int] = 1
    pad_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)
    model_type: str = "qwen3"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        hidden = int(_get(raw, "hidden_size"))
        heads = int(_get(raw, "num_attention_heads"))
        kv_heads = int(_get(raw, "num_key_value_heads", heads))
        head_dim = int(_get(raw, "head_dim", hidden // heads))

        theta = float(_get(raw, "rope_theta", 10000.0))
        factor = 1.0
        scaling = raw.get("rope_scaling")
        params = raw.get("rope_parameters")
        if isinstance(params, dict):
            theta = float(params.get("rope_theta", theta))
            if scaling is None and params.get("rope_type", "default") != "default":
                scaling = params
        if scaling:
            kind = scaling.get("rope_type", scaling.get("type", "default"))
            if kind == "linear":
                factor = float(scaling["factor"])
            elif kind != "default":
                raise ConfigError(
                    f"rope_scaling type {kind!r} is not supported (supported: none, 'linear')")

        eos = _get(raw, "eos_token_id", 2)
        eos = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        layer_types = raw.get("layer_types")
        window = _get(raw, "sliding_window", None)
        mwl = _get(raw, "max_window_layers", None)
        bos = _get(raw, "bos_token_id", 1)
        pad = _get(raw, "pad_token_id", None)

        cfg = cls(
            vocab_size=int(_get(raw, "vocab_size")),
            hidden_size=hidden,
            intermediate_size=int(_get(raw, "intermediate_size")),
            num_hidden_layers=int(_get(raw, "num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(_get(raw, "rms_norm_eps", 1e-5)),
            rope_theta=theta,
            rope_factor=factor,
            max_position_embeddings=int(_get(raw, "max_position_embeddings", 4096)),
            tie_word_embeddings=bool(_get(raw, "tie_word_embeddings", False)),
            hidden_act=str(_get(raw, "hidden_act", "silu")),
            attention_bias=bool(_get(raw, "attention_bias", False)),
            qk_norm=bool(_get(raw, "qk_norm", True)),
            use_sliding_window=bool(_get(raw, "use_sliding_window", False)),
            sliding_window=None if window is None else int(window),
            max_window_layers=None if mwl is None else int(mwl),
            layer_types=None if layer_types is None else tuple(str(t) for t in layer_types),
            eos_token_id=eos,
            bos_token_id=None if bos is None else int(bos),
            pad_token_id=None if pad is None else int(pad),
            torch_dtype=str(_get(raw, "torch_dtype", _get(raw, "dtype", "bfloat16"))),
            architectures=tuple(_get(raw, "architectures", ["Qwen3ForCausalLM"])),
            model_type=str(_get(raw, "model_type", "qwen3")),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if not os.path.exists(path):
            raise ConfigError(f"config.json not found at {path}")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    # --------------------------------------------------------------- validate
    def validate(self) -> None:
        pos = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
               "num_attention_heads", "num_key_value_heads", "head_dim",
               "max_position_embeddings")
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"{k} must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for rotary encoding, got {self.head_dim}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (supported: 'silu')")
        if self.attention_bias:
            raise ConfigError("attention_bias=true is not supported")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"layer_types has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers")
            bad = sorted(set(self.layer_types) - {"full_attention", "sliding_attention"})
            if bad:
                raise ConfigError(f"unknown layer_types entries: {bad}")
        if self.use_sliding_window and not (self.sliding_window and self.sliding_window > 0):
            raise ConfigError("use_sliding_window needs a positive sliding_window")

    # ------------------------------------------------------------- derivation
    def layer_windows(self) -> List[Optional[int]]:
        """Window of each layer, ``None`` where a layer sees every earlier key.

        Without ``use_sliding_window`` no layer has a window, whatever ``layer_types``
        and ``sliding_window`` say (the architecture's own configuration drops the window
        then, so its ``sliding_attention`` layers attend to every key).  With it,
        ``layer_types`` decides when present; otherwise layers from ``max_window_layers``
        on are windowed (the first ``max_window_layers`` keep full attention).
        """
        n = self.num_hidden_layers
        if not self.use_sliding_window:
            return [None] * n
        if self.layer_types is not None:
            return [self.sliding_window if t == "sliding_attention" else None
                    for t in self.layer_types]
        if self.use_sliding_window and self.sliding_window:
            first = self.max_window_layers if self.max_window_layers is not None else 0
            return [self.sliding_window if i >= first else None for i in range(n)]
        return [None] * n

    def to_spec(self) -> ModelSpec:
        norm = NormSpec(eps=self.rms_norm_eps)
        rope = RopeSpec(theta=self.rope_theta, rotary_dim=self.head_dim, factor=self.rope_factor)
        ffn = GatedMLPSpec(intermediate_size=self.intermediate_size, activation=self.hidden_act)
        layers = []
        for w in self.layer_windows():
            mixer = AttentionSpec(
                num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim, qk_norm=self.qk_norm, qk_norm_eps=self.rms_norm_eps,
                bias=self.attention_bias, window=w, position=rope)
            layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm=norm))
        return ModelSpec(
            architecture=self.architectures[0],
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            final_norm=norm,
            tie_word_embeddings=self.tie_word_embeddings,
            max_position_embeddings=self.max_position_embeddings,
            eos_token_ids=self.eos_token_id,
            bos_token_id=self.bos_token_id,
            pad_token_id=self.pad_token_id,
            names=NameLayout(),
        )

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that :meth:`from_dict` reads back to this object."""
        d: Dict[str, Any] = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": (None if self.rope_factor == 1.0
                             else {"rope_type": "linear", "factor": self.rope_factor}),
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "eos_token_id": (self.eos_token_id[0] if len(self.eos_token_id) == 1
                             else list(self.eos_token_id)),
            "bos_token_id": self.bos_token_id,
            "pad_token_id": self.pad_token_id,
            "torch_dtype": self.torch_dtype,
        }
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        return d

    # ---------------------------------------------------------------- memory
    def num_parameters(self) -> int:
        """Parameter count (the reference's estimate: src/model/config.ts:199-255)."""
        h, q = self.hidden_size, self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        per_layer = h * (q + 2 * kv) + q * h + 3 * h * self.intermediate_size + 2 * h
        per_layer += 2 * self.head_dim if self.qk_norm else 0
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return self.vocab_size * h + self.num_hidden_layers * per_layer + h + head

    def kv_bytes_per_token(self, element_size: int = 2) -> int:
        return (2 * self.num_key_value_heads * self.head_dim * element_size
                * self.num_hidden_layers)
