"""Architecture-neutral descriptions of a decoder: what each layer is made of.

A model family (for instance ``config/qwen3.py``) turns its own ``config.json``
keys into a :class:`ModelSpec`.  Everything downstream (weights, parts, cache
manager, step function) reads only these specs, never a family's config, so a
new architecture is a new config class plus, where needed, new parts.

The reference keeps every size in one flat ``LlamaConfig`` and branches on it
inside the engine (src/model/config.ts:5-60, src/engine/batched_engine.ts:834,
1186); here each part gets exactly the sizes and constants it needs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary position encoding over the first ``rotary_dim`` of a head."""

    kind: str = "rope"
    theta: float = 10000.0
    rotary_dim: int = 0          # 0 means the whole head
    # linear position scaling (angle = position / factor * inv_freq); 1.0 = none
    factor: float = 1.0


@dataclass(frozen=True)
class NormSpec:
    kind: str = "rmsnorm"
    eps: float = 1e-6


@dataclass(frozen=True)
class ScoreSpec:
    """What is done to an attention score ``s = (q . k) * scale`` of query position p and key
    position j before the softmax.  None of it is Qwen3's; a family whose attention has it
    names it here, and the mixer takes the kernel that applies it.

    ``softcap`` c > 0: ``s <- c * tanh(s / c)``.  ``slopes`` (one number per query head):
    ``s <- s + slope_h * (j - p)``, a bias per distance.  ``sinks``: a learned logit per query
    head (tensor ``sinks [heads]`` of the mixer) that joins the softmax's denominator and
    takes no value: ``P_j = exp(s_j) / (exp(sink_h) + sum_j exp(s_j))``."""

    softcap: float = 0.0
    slopes: Optional[Tuple[float, ...]] = None
    sinks: bool = False


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal attention over a paged key/value cache."""

    kind: str = "attention"
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False        # per-head RMSNorm on q and k before the rotation
    qk_norm_eps: float = 1e-6
    bias: bool = False           # q/k/v/o projection biases
    window: Optional[int] = None  # keys j with p - window < j <= p; None = all keys
    scale: Optional[float] = None  # None = 1/sqrt(head_dim)
    position: Optional[object] = None   # RopeSpec, or any spec whose kind is registered
    score: Optional[ScoreSpec] = None   # changes to the scores before the softmax; None: none

    @property
    def group_size(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def softmax_scale(self) -> float:
        return self.scale if self.scale is not None else self.head_dim ** -0.5


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    kind: str = "gated_mlp"
    intermediate_size: int = 0
    activation: str = "silu"
    bias: bool = False


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which mixer, which feed-forward, which norm, how arranged."""

    mixer: object = None         # a mixer spec with a ``kind`` attribute
    ffn: object = None           # a feed-forward spec with a ``kind`` attribute
    norm: NormSpec = NormSpec()
    block: str = "prenorm"       # arrangement of the parts inside the layer


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes :attr:`ModelSpec.layers`.  ``cache_from`` is ``None`` when
    this execution keeps a cache of its own, else the index of the schedule
    entry whose cache it reads (it then writes none).
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 4096
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    # multiplies the embedding output / the logits; 1.0 = none
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    # tensor-name layout of the family (prefixes for embed, layers, norm, head)
    names: "NameLayout" = None


@dataclass(frozen=True)
class NameLayout:
    """Where a family keeps its tensors in a checkpoint (Hugging Face names).

    The reference builds these strings inline at each use
    (src/engine/batched_engine.ts:773,802,811-813,1717,1737,1753-1755).
    """

    embed: str = "model.embed_tokens.weight"
    layer_prefix: str = "model.layers.{i}."
    input_norm: str = "input_layernorm"
    post_mixer_norm: str = "post_attention_layernorm"
    mixer: str = "self_attn"
    ffn: str = "mlp"
    final_norm: str = "model.norm.weight"
    lm_head: str = "lm_head.weight"
    # further norms of a layer, for arrangements that have more than the two above:
    # (role, name inside the layer) pairs
    more_norms: Tuple[Tuple[str, str], ...] = ()

    def norm(self, role: str) -> str:
        """The name, inside a layer, of the norm that plays ``role``: ``input``,
        ``post_mixer`` or one of ``more_norms``."""
        table = {"input": self.input_norm, "post_mixer": self.post_mixer_norm,
                 **dict(self.more_norms)}
        if role not in table:
            raise KeyError(f"no norm with the role {role!r} in this family's names "
                           f"(known: {sorted(table)})")
        return table[role]


class ConfigError(ValueError):
    """A config.json that is missing a key or asks for something unsupported."""
