"""Grouped-query causal attention over the paged cache, as a mixer part.

Order of operations (src/engine/batched_engine.ts:811-1118): q/k/v projections,
optional per-head RMSNorm of q and k (:834-839), rotation of q and k (:861-876),
k and v written to their pages (:933-961), softmax(q k^T / sqrt(d)) v over the
keys at or before the query with query head h reading kv head h // group
(cuda/kernels/paged_attention.cu:408-487), output projection (:1116-1118).

Differences from the reference, on purpose: the three projections are one
product against the concatenated weight; norm, rotation and cache write are one
kernel; and every key, also those of the step's own tokens, is read from the
pages, so a prompt can be cut into portions anywhere and portions can share a
step with decoded tokens (the reference's prefill ignores the cache, :1082-1086).
An optional window restricts a query at p to keys in (p - window, p].
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..cache.manager import KVNeed
from ..config.specs import AttentionSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import (BuildEnv, DeferredLinear, EntryView, Mixer, StepContext, build_position,
                   register_mixer, split_scaled)
from .linear import linear


class GQAAttention(Mixer):
    def __init__(self, spec: AttentionSpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim % 2 or spec.head_dim > 256:
            raise ValueError(f"head_dim {spec.head_dim} is not supported (even, at most 256)")
        if spec.bias:
            raise ValueError("attention projection biases are not supported")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.position = (build_position(spec.position, spec.head_dim, env)
                         if spec.position is not None else None)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # ----------------------------------------------------------------- weights
    def param_specs(self) -> List[ParamSpec]:
        p, s = self.prefix, self.spec
        specs = [ParamSpec(p + "q_proj.weight", (self.q_size, self.hidden)),
                 ParamSpec(p + "k_proj.weight", (self.kv_size, self.hidden)),
                 ParamSpec(p + "v_proj.weight", (self.kv_size, self.hidden)),
                 ParamSpec(p + "o_proj.weight", (self.hidden, self.q_size))]
        if s.qk_norm:
            specs += [ParamSpec(p + "q_norm.weight", (s.head_dim,), init="norm", role="vector"),
                      ParamSpec(p + "k_norm.weight", (s.head_dim,), init="norm", role="vector")]
        return specs

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        sp = {s.name[len(self.prefix):]: s for s in self.param_specs()}
        # one [Q + 2 KV, H] weight: a single product yields q, k and v of a token side by side
        self.w_qkv = torch.cat([get(sp["q_proj.weight"]), get(sp["k_proj.weight"]),
                                get(sp["v_proj.weight"])], dim=0).contiguous()
        self.w_o = get(sp["o_proj.weight"])
        if self.spec.qk_norm:
            self.q_norm = get(sp["q_norm.weight"])
            self.k_norm = get(sp["k_norm.weight"])

    # ------------------------------------------------------------------- cache
    def kv_need(self) -> Optional[KVNeed]:
        s = self.spec
        return KVNeed(s.num_kv_heads, s.head_dim, s.window)

    # ----------------------------------------------------------------- forward
    accepts_scaled_rows = True

    def forward(self, x, ctx: StepContext, view: EntryView) -> torch.Tensor:
        return self.forward_deferred(x, ctx, view).compute()

    def forward_deferred(self, x, ctx: StepContext, view: EntryView) -> DeferredLinear:
        """Everything but the output projection, which is left to the caller (the block
        fuses it with the add into the stream and the next norm where it can).  ``x`` may be
        ``ScaledRows``: its factor is applied to the rows of q, k and v as they are read."""
        x, row_scale = split_scaled(x)
        s, T = self.spec, x.shape[0]
        g = view.group
        if view.writes_cache:
            qkv = linear(x, self.w_qkv)
        else:       # the pages belong to another layer execution: only q is needed
            qkv = linear(x, self.w_qkv[: self.q_size])
        q = torch.empty((T, self.q_size), dtype=x.dtype, device=x.device)
        ops.qk_norm_rope_kv_write(
            qkv, self.q_norm, self.k_norm,
            self.position.inv_freq if self.position is not None else None,
            ctx.positions, ctx.slots[g] if view.writes_cache else None, q,
            view.k_cache if view.writes_cache else None,
            view.v_cache if view.writes_cache else None,
            s.num_heads, s.num_kv_heads, s.head_dim, s.qk_norm_eps, ctx.err, row_scale=row_scale)
        out = torch.empty_like(q)
        self.attend(q, out, ctx, view)
        return DeferredLinear(out, self.w_o)

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext,
               view: EntryView) -> None:
        """Attention of every token row over its request's pages.

        float32: the generic kernel, whose sums have one fixed order per position.
        bfloat16: rows that bring a single token go to the split-KV decode kernel;
        the rest (and head sizes the tuned kernels do not take) to the generic one.
        """
        s = self.spec
        tables = ctx.block_tables[view.group]
        fast = q.dtype == torch.bfloat16 and s.head_dim in ops.DECODE_HEAD_DIMS
        if not fast:
            ops.paged_attention_generic(
                q, view.k_cache, view.v_cache, ctx.seq_of_token, ctx.positions, tables, out,
                s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.softmax_scale, ctx.err)
            return
        common = (s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.softmax_scale)
        if ctx.decode_only:
            ops.decode_attention(q, view.k_cache, view.v_cache, None, ctx.T, ctx.seq_of_token,
                                 ctx.positions, tables, out, *common, ctx.max_ctx_len, ctx.err)
            return
        if ctx.n_decode:
            ops.decode_attention(q, view.k_cache, view.v_cache, ctx.decode_rows, ctx.n_decode,
                                 ctx.seq_of_token, ctx.positions, tables, out, *common,
                                 ctx.max_decode_ctx, ctx.err)
        if ctx.n_prefill:
            ops.prefill_attention(q, view.k_cache, view.v_cache, ctx.prefill_items,
                                  ctx.n_prefill, ctx.max_prefill_rows, tables, out, *common,
                                  ctx.err)


register_mixer("attention", GQAAttention)
