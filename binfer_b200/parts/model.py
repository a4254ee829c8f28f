"""The decoder: embedding, a schedule of layer executions, final norm, output head.

Built from a :class:`ModelSpec` alone.  The schedule is data: a list of
(layer, cache source) pairs that may run a layer twice or let an execution read
the pages of another one.  The reference hard-codes ``for layer in 0..L-1``
(src/engine/batched_engine.ts:1729-1731).

Output head (src/engine/batched_engine.ts:1733-1770): final norm, then logits
``y W^T`` with ``W = lm_head.weight`` or, when the embeddings are tied, the
embedding table (:1753-1755).  Only the rows whose logits are wanted go through
the norm and the head; logits are float32 (the reference's are bfloat16).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheManager, KVNeed, StateNeed
from ..config.specs import ModelSpec
from ..csrc import ops
from ..weights.loader import ParamSpec, TensorSource, check_names, place
from .base import (BuildEnv, EntryView, ResidualStream, StepContext, build_block, build_norm)
from .linear import linear

# importing the modules registers the built-in parts
from . import attention as _attention  # noqa: F401
from . import block as _block          # noqa: F401
from . import mlp as _mlp              # noqa: F401
from . import norms as _norms          # noqa: F401
from . import rope as _rope            # noqa: F401


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec, self.env = spec, env
        names = spec.names
        self.blocks = [build_block(ls, spec.hidden_size, names, i, env)
                       for i, ls in enumerate(spec.layers)]
        self.final_norm = build_norm(spec.final_norm, spec.hidden_size, names.final_norm, env)
        self.embed_spec = ParamSpec(names.embed, (spec.vocab_size, spec.hidden_size))
        self.head_spec = (None if spec.tie_word_embeddings
                          else ParamSpec(names.lm_head, (spec.vocab_size, spec.hidden_size)))
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        for e, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {e} names layer {entry.layer}, "
                                 f"but there are {len(self.blocks)} layers")
            if entry.cache_from is not None:
                src = spec.schedule[entry.cache_from] if 0 <= entry.cache_from < e else None
                if src is None or src.cache_from is not None:
                    raise ValueError(f"schedule entry {e}: cache_from must name an earlier "
                                     f"entry that keeps a cache of its own")

    # ----------------------------------------------------------------- weights
    def param_specs(self) -> List[ParamSpec]:
        specs = [self.embed_spec]
        for b in self.blocks:
            specs += b.param_specs()
        specs += self.final_norm.param_specs()
        if self.head_spec is not None:
            specs.append(self.head_spec)
        return specs

    def load(self, source: TensorSource, allow_unexpected: bool = False) -> None:
        """Check every name and shape first (one error for all), then take the tensors.
        ``allow_unexpected``: tensors the model does not use are a warning, not an error."""
        optional = [self.spec.names.lm_head] if self.head_spec is None else []
        check_names(self.param_specs(), source.shapes, optional=optional, where=source.where,
                    allow_unexpected=allow_unexpected)

        def get(spec: ParamSpec) -> torch.Tensor:
            return place(source.get(spec.name), spec, self.env.dtype, self.env.device)

        self.embed = get(self.embed_spec)
        for b in self.blocks:
            b.load(get)
        self.final_norm.load(get)
        self.lm_head = self.embed if self.head_spec is None else get(self.head_spec)

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (a tied table counts once per use)."""
        seen, total = set(), 0
        for obj in [self] + self.blocks + [self.final_norm] + \
                [p for b in self.blocks for p in (b.parts() if hasattr(b, "parts") else [])]:
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    # ------------------------------------------------------------------- cache
    def kv_needs(self) -> List[Optional[KVNeed]]:
        """Per schedule entry: the pages it keeps (None if it keeps none of its own)."""
        out: List[Optional[KVNeed]] = []
        for entry in self.spec.schedule:
            need = self.blocks[entry.layer].mixer.kv_need()
            out.append(need if entry.cache_from is None else None)
        return out

    def state_needs(self) -> List[Optional[StateNeed]]:
        return [self.blocks[entry.layer].mixer.state_need() for entry in self.spec.schedule]

    def entry_views(self, cache: CacheManager) -> List[EntryView]:
        views: List[EntryView] = []
        for e, entry in enumerate(self.spec.schedule):
            src = e if entry.cache_from is None else entry.cache_from
            if cache.entry_location[src] is None:
                k = v = g = None
            else:
                k, v, g = cache.kv_view(src)
            views.append(EntryView(e, g, k, v, entry.cache_from is None, cache.state_storage[e]))
        return views

    # ----------------------------------------------------------------- forward
    def forward(self, ctx: StepContext, views: List[EntryView]) -> torch.Tensor:
        """Logits ``[R, vocab]`` (float32) at ``ctx.logit_rows``."""
        spec = self.spec
        resid = torch.empty((ctx.T, spec.hidden_size), dtype=torch.float32, device=self.env.device)
        ops.embed_gather(self.embed, ctx.token_ids, resid, spec.embedding_scale, ctx.err)
        stream = ResidualStream(resid)
        last = len(spec.schedule) - 1
        for e, entry in enumerate(spec.schedule):
            ctx.entry = e
            block = self.blocks[entry.layer]
            if getattr(block, "takes_successor", False):
                # a block may let its last product prepare the next block's first norm
                nxt = self.blocks[spec.schedule[e + 1].layer] if e < last else None
                block.forward(stream, ctx, views[e], nxt)
            else:
                block.forward(stream, ctx, views[e])
        R = ctx.logit_rows.shape[0]
        if R == 0:
            stream.flush()
            return torch.empty((0, spec.vocab_size), dtype=torch.float32, device=self.env.device)
        y = self.final_norm.forward(stream, rows=ctx.logit_rows, n_rows=R)
        logits = linear(y, self.lm_head, out_dtype=torch.float32)
        if spec.logit_scale != 1.0:
            logits.mul_(spec.logit_scale)
        return logits


def param_specs_for(spec: ModelSpec) -> List[ParamSpec]:
    """Names, shapes and roles of every tensor a checkpoint of ``spec`` must hold."""
    env = BuildEnv(torch.float32, torch.device("cpu"))
    return DecoderModel(spec, env).param_specs()


def build_model(spec: ModelSpec, env: BuildEnv, source: TensorSource,
                allow_unexpected: bool = False) -> DecoderModel:
    model = DecoderModel(spec, env)
    model.load(source, allow_unexpected=allow_unexpected)
    return model
