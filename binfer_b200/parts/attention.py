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
An optional window restricts a query at p to keys in (p - window, p].  Changes to
the scores before the softmax (``AttentionSpec.score``: a soft cap, a bias per
distance, a sink logit per head) are not Qwen3's; a spec that names one gets the
generic attention kernel, which applies them, in both precisions.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch

from ..cache.manager import KVNeed
from ..config.specs import AttentionSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import (BuildEnv, DeferredLinear, EntryView, Mixer, StepContext, build_position,
                   register_mixer, split_scaled)
from .linear import cluster_token_limit, linear

# BINFER_B200_FUSE_QKV=1: steps of few tokens run the q/k/v projection with the head norms,
# the rotation and the store into the pages as one kernel.  Off unless asked for: its tiles
# must be whole heads, which leaves the 8B shape 96 CTAs where the plain product has 128, and
# inside a decode step that cost more (3.6 us) than the kernel it saves (8 layers, batch 8,
# context 4096: 1.204 against 1.186 ms a step).
FUSE_QKV = os.environ.get("BINFER_B200_FUSE_QKV", "0") != "0"
# ... and only where those tiles give work to this share of the SMs
FUSE_QKV_FILL = 0.6


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
        self.sinks = self.slopes = None
        if spec.score is not None and spec.score.slopes is not None:
            if len(spec.score.slopes) != spec.num_heads:
                raise ValueError("score.slopes needs one slope per query head")
            self.slopes = torch.tensor(spec.score.slopes, dtype=torch.float32, device=env.device)
        self._qkv_plans = {}

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
        if s.score is not None and s.score.sinks:
            specs.append(ParamSpec(p + "sinks", (s.num_heads,), init="norm", role="vector"))
        if self.position is not None:
            specs += self.position.param_specs(p)
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
        if self.spec.score is not None and self.spec.score.sinks:
            self.sinks = get(sp["sinks"])
        if self.position is not None:
            self.position.load(get)

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
        pos = self.position
        q = torch.empty((T, self.q_size), dtype=x.dtype, device=x.device)
        # the pages may belong to another layer execution: only q is needed then
        w = self.w_qkv if view.writes_cache else self.w_qkv[: self.q_size]
        if not self._project_fused(x, w, q, row_scale, ctx, view):
            qkv = linear(x, w)
            if pos is None or pos.inv_freq is not None:
                # head norms, rotation and the store into the pages: one kernel
                writes = view.writes_cache
                ops.qk_norm_rope_kv_write(
                    qkv, self.q_norm, self.k_norm, pos.inv_freq if pos is not None else None,
                    ctx.positions, ctx.slots[g] if writes else None, q,
                    view.k_cache if writes else None, view.v_cache if writes else None,
                    s.num_heads, s.num_kv_heads, s.head_dim, s.qk_norm_eps, ctx.err,
                    row_scale=row_scale)
            else:
                self._encode_unfused(qkv, q, row_scale, ctx, view)
        out = torch.empty_like(q)
        self.attend(q, out, ctx, view)
        return DeferredLinear(out, self.w_o)

    def _project_fused(self, x, w, q, row_scale, ctx: StepContext, view: EntryView) -> bool:
        """Few token rows in bfloat16: the projection, the head norms, the rotation and the
        store into the pages as one kernel, where the split-K cluster product has a plan with
        tiles of whole heads for this shape.  False, having done nothing, otherwise."""
        s, pos = self.spec, self.position
        if (not FUSE_QKV or x.dtype != torch.bfloat16 or x.shape[0] > cluster_token_limit()
                or (pos is not None and pos.inv_freq is None)):
            return False
        key = (w.shape[0], w.shape[1])
        if key not in self._qkv_plans:
            self._qkv_plans[key] = ops.gemm_cluster_qkv_plan(*key, s.head_dim, x.device,
                                                             max(FUSE_QKV_FILL, 0.6))
        plan = self._qkv_plans[key]
        if plan is None or plan[2] < FUSE_QKV_FILL * ops.num_sms(x.device):
            return False
        writes = view.writes_cache
        return ops.gemm_bf16_cluster_qkv(
            x, w, self.q_norm, self.k_norm, pos.inv_freq if pos is not None else None,
            ctx.positions, ctx.slots[view.group] if writes else None, q,
            view.k_cache if writes else None, view.v_cache if writes else None, s.num_heads,
            s.num_kv_heads, s.head_dim, s.qk_norm_eps, ctx.err, *plan[:2], row_scale=row_scale)

    def _encode_unfused(self, qkv, q, row_scale, ctx: StepContext, view: EntryView) -> None:
        """A position encoding that is no rotation: the head norms write q, and k and v
        into token-major scratch (a cache of one-token pages, token t in page t); the
        encoding changes q and k there; a second pass stores k and v into the pages."""
        s, T = self.spec, qkv.shape[0]
        if not view.writes_cache:
            qkv = torch.cat([qkv, qkv.new_zeros((T, 2 * self.kv_size))], dim=1)
        k_rows = torch.empty((T, s.num_kv_heads, 1, s.head_dim), dtype=q.dtype, device=q.device)
        v_rows = torch.empty_like(k_rows)
        each = torch.arange(T, dtype=torch.int32, device=q.device)
        ops.qk_norm_rope_kv_write(qkv, self.q_norm, self.k_norm, None, ctx.positions, each, q,
                                  k_rows, v_rows, s.num_heads, s.num_kv_heads, s.head_dim,
                                  s.qk_norm_eps, ctx.err, row_scale=row_scale)
        self.position.apply(q.view(T, s.num_heads, s.head_dim),
                            k_rows.view(T, s.num_kv_heads, s.head_dim), ctx.positions)
        if view.writes_cache:
            encoded = torch.cat([q, k_rows.view(T, self.kv_size), v_rows.view(T, self.kv_size)],
                                dim=1)
            ops.qk_norm_rope_kv_write(encoded, None, None, None, ctx.positions,
                                      ctx.slots[view.group], q, view.k_cache, view.v_cache,
                                      s.num_heads, s.num_kv_heads, s.head_dim, s.qk_norm_eps,
                                      ctx.err)

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext,
               view: EntryView) -> None:
        """Attention of every token row over its request's pages.

        float32: the generic kernel, whose sums have one fixed order per position.
        bfloat16: rows that bring a single token go to the split-KV decode kernel;
        the rest (and head sizes the tuned kernels do not take) to the generic one.
        """
        s = self.spec
        tables = ctx.block_tables[view.group]
        fast = (q.dtype == torch.bfloat16 and s.head_dim in ops.DECODE_HEAD_DIMS
                and s.score is None)
        if not fast:
            ops.paged_attention_generic(
                q, view.k_cache, view.v_cache, ctx.seq_of_token, ctx.positions, tables, out,
                s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.softmax_scale, ctx.err,
                softcap=s.score.softcap if s.score is not None else 0.0,
                slopes=self.slopes, sinks=self.sinks)
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
                                  ctx.err, max_ctx=ctx.max_ctx_len)


register_mixer("attention", GQAAttention)
