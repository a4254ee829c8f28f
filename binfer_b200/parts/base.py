"""Interfaces of the parts a layer is put together from, and their registries.

A *part* is built from its spec (sizes and constants as parameters), names the
checkpoint tensors it needs, takes them, and runs on a :class:`StepContext`.
No part knows which model it is in: it sees its spec, the hidden size, a name
prefix, and the step's batch description.

Kinds are looked up in per-role registries, so a new mixer, feed-forward, norm,
position encoding or block arrangement is one class and one ``register_*`` call;
the configuration picks parts layer by layer through each spec's ``kind``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager, KVNeed, StateNeed
from ..weights.loader import ParamSpec


@dataclass
class BuildEnv:
    """Where and in which precision a model is built."""

    dtype: torch.dtype            # activations, matrices and cache pages
    device: torch.device


@dataclass
class StepContext:
    """One step's batch, as the parts see it.

    The batch is a flat run of ``T`` tokens belonging to ``B`` requests; request
    ``b`` owns tokens ``q_start[b] .. q_start[b+1]-1``, which sit at absolute
    positions ``ctx_lens[b] - q_lens[b] ..  ctx_lens[b] - 1`` of that request.
    """

    env: BuildEnv
    cache: CacheManager
    T: int
    B: int
    token_ids: torch.Tensor            # int32 [T]
    positions: torch.Tensor            # int32 [T]
    seq_of_token: torch.Tensor         # int32 [T]
    q_start: torch.Tensor              # int32 [B + 1]
    ctx_lens: torch.Tensor             # int32 [B]
    state_slots: torch.Tensor          # int32 [B]
    slots: List[torch.Tensor]          # per cache group: int32 [T], place of each token
    block_tables: List[torch.Tensor]   # per cache group: int32 [B, P]
    logit_rows: torch.Tensor           # int32 [R]
    err: torch.Tensor                  # int32 [1], error bits set by kernels
    # host copies, for launch decisions only
    q_lens: Sequence[int] = ()
    ctx_lens_host: Sequence[int] = ()
    max_q_len: int = 1
    max_ctx_len: int = 1
    decode_only: bool = False
    # rows that bring one token, and portions that bring more (for kernels that treat
    # the two apart): decode_rows int32 [n_decode] of token rows; prefill_items int32
    # [n_prefill, 4] of (request index, first token row, rows, first position)
    decode_rows: Optional[torch.Tensor] = None
    n_decode: int = 0
    max_decode_ctx: int = 1
    prefill_items: Optional[torch.Tensor] = None
    n_prefill: int = 0
    max_prefill_rows: int = 0
    entry: int = 0                     # schedule entry being run
    scratch: Dict[str, object] = field(default_factory=dict)


class Part:
    """Base of every part: tensors it needs, and how it takes them."""

    def param_specs(self) -> List[ParamSpec]:
        return []

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        """``get(spec)`` returns the tensor on the device, in the dtype of its role."""


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here).

    ``forward(x, ctx, view)`` maps normed activations ``[T, H]`` to ``[T, H]``.
    ``view`` (:class:`EntryView`) holds this execution's cache pages and state.
    """

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, view: "EntryView") -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding:
    """How a token's absolute position enters an attention mixer's queries and keys.

    Two forms, told apart by ``inv_freq``:

    * the rotary family sets ``inv_freq`` (float32 ``[rot/2]`` on the device, ``rot`` at
      most the head size): the pair ``(i, i + rot/2)`` of each query and key head turns by
      ``position * inv_freq[i]`` inside the kernel that also norms the heads and stores the
      keys.  Any table of frequencies goes this way (scaled, stretched, partial);
    * every other encoding leaves ``inv_freq`` None and defines ``apply(q, k, positions)``,
      which changes ``q [T, heads, d]`` and ``k [T, kv_heads, d]`` in place after the head
      norms and before the keys are stored; the mixer then runs norm, ``apply`` and the
      store as separate launches.

    An encoding with tensors of its own names them in ``param_specs(prefix)`` (``prefix`` is
    the mixer's) and takes them in ``load(get)``, like a part.
    """

    inv_freq: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return []

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        pass

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    """Per-token transformation ``[T, H] -> [T, H]`` (dense here; experts elsewhere)."""

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    """Normalises the residual stream; fuses the stream's pending add."""

    def forward(self, stream: "ResidualStream", rows: Optional[torch.Tensor] = None,
                n_rows: int = 0) -> torch.Tensor:
        raise NotImplementedError


@dataclass
class EntryView:
    """What one layer execution may touch in the cache manager's storage."""

    entry: int
    group: Optional[int]               # cache group index, None if the mixer keeps no pages
    k_cache: Optional[torch.Tensor]    # [pages + 1, kv_heads, page_size, head_dim]
    v_cache: Optional[torch.Tensor]
    writes_cache: bool                 # False when the pages belong to another entry
    state: Optional[torch.Tensor]      # [slots, *shape] of the mixer's StateNeed


class DeferredLinear:
    """``x @ w^T`` not yet computed: how a part may hand its output to the block
    (``forward_deferred``), so that the product can be fused with what follows it, the add
    into the residual stream and the next norm."""
    __slots__ = ("x", "w")

    def __init__(self, x: torch.Tensor, w: torch.Tensor):
        self.x, self.w = x, w

    def compute(self) -> torch.Tensor:
        from .linear import linear
        return linear(self.x, self.w)


class ScaledRows:
    """Activations ``[T, H]`` whose rows still lack a common factor (``scale``, an
    ``ops.RowScale``): a norm's output as a fused product leaves it.  A part that sets
    ``accepts_scaled_rows`` runs its first product on ``tensor`` and hands ``scale`` to the
    kernel after that product; for any other part the block calls :meth:`dense`."""
    __slots__ = ("tensor", "scale")

    def __init__(self, tensor: torch.Tensor, scale):
        self.tensor, self.scale = tensor, scale

    def dense(self) -> torch.Tensor:
        f = self.scale.factors().unsqueeze(1)
        return (self.tensor.float() * f).to(self.tensor.dtype)


def split_scaled(x):
    """``(tensor, scale or None)`` of what a norm returned."""
    return (x.tensor, x.scale) if isinstance(x, ScaledRows) else (x, None)


class ResidualStream:
    """The float residual stream ``[T, H]`` with at most one sublayer output not yet added.

    A sublayer's output is recorded with :meth:`add`; the next norm folds it into
    the stream while it normalises (one pass over memory instead of two).  Where a
    sublayer ends in a product and the kernels can do it, :meth:`add_linear` goes further:
    the product's epilogue adds into the stream and prepares the next norm's output, which
    then waits in ``ready`` for that norm (``ready_for``).
    """

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending: Optional[torch.Tensor] = None
        self.ready: Optional[ScaledRows] = None
        self.ready_for = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
        self.pending = delta
        self.ready = self.ready_for = None

    def add_linear(self, d: DeferredLinear, norm=None, consumer=None) -> None:
        """Add ``d.x @ d.w^T``.  ``norm`` is the norm that reads the stream next and
        ``consumer`` the part that takes its output; the fused path needs a norm with a
        ``fused_scale`` (weight, eps) over whole rows and a consumer that accepts
        :class:`ScaledRows`."""
        from .linear import linear_add_norm
        fs = getattr(norm, "fused_scale", None)
        if fs is not None and getattr(consumer, "accepts_scaled_rows", False):
            self.flush()
            weight, eps = fs()
            got = linear_add_norm(d.x, d.w, self.x, weight, eps)
            if got is not None:
                self.ready, self.ready_for = ScaledRows(*got), norm
                return
        self.add(d.compute())

    def flush(self) -> None:
        if self.pending is not None:
            from ..csrc import ops
            ops.residual_add(self.x, self.pending)
            self.pending = None


# ------------------------------------------------------------------ registries
_MIXERS: Dict[str, Callable] = {}
_FFNS: Dict[str, Callable] = {}
_NORMS: Dict[str, Callable] = {}
_POSITIONS: Dict[str, Callable] = {}
_BLOCKS: Dict[str, Callable] = {}


def register_mixer(kind: str, factory: Callable) -> None:
    """``factory(spec, hidden_size, prefix, env) -> Mixer``"""
    _MIXERS[kind] = factory


def register_ffn(kind: str, factory: Callable) -> None:
    """``factory(spec, hidden_size, prefix, env) -> FeedForward``"""
    _FFNS[kind] = factory


def register_norm(kind: str, factory: Callable) -> None:
    """``factory(spec, size, name, env) -> Norm`` (``name`` is the weight tensor's name)"""
    _NORMS[kind] = factory


def register_position(kind: str, factory: Callable) -> None:
    """``factory(spec, head_dim, env) -> PositionEncoding``"""
    _POSITIONS[kind] = factory


def register_block(kind: str, factory: Callable) -> None:
    """``factory(layer_spec, hidden_size, names, layer_index, env) -> block``"""
    _BLOCKS[kind] = factory


def _build(table: Dict[str, Callable], role: str, spec, *args):
    kind = getattr(spec, "kind", None)
    if kind not in table:
        raise KeyError(f"no {role} of kind {kind!r} is registered (known: {sorted(table)})")
    return table[kind](spec, *args)


def build_mixer(spec, hidden_size: int, prefix: str, env: BuildEnv) -> Mixer:
    return _build(_MIXERS, "mixer", spec, hidden_size, prefix, env)


def build_ffn(spec, hidden_size: int, prefix: str, env: BuildEnv) -> FeedForward:
    return _build(_FFNS, "feed-forward", spec, hidden_size, prefix, env)


def build_norm(spec, size: int, name: str, env: BuildEnv) -> Norm:
    return _build(_NORMS, "norm", spec, size, name, env)


def build_position(spec, head_dim: int, env: BuildEnv):
    return _build(_POSITIONS, "position encoding", spec, head_dim, env)


def build_block(layer_spec, hidden_size: int, names, layer_index: int, env: BuildEnv):
    if layer_spec.block not in _BLOCKS:
        raise KeyError(f"no block arrangement {layer_spec.block!r} is registered "
                       f"(known: {sorted(_BLOCKS)})")
    return _BLOCKS[layer_spec.block](layer_spec, hidden_size, names, layer_index, env)
