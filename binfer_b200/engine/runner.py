"""The step function: one forward over a batch of (request, its next tokens).

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.
The step reserves pages for exactly the tokens it writes, describes the batch to
the device in one copy, runs only the tokens it was given (every key comes from
the cache that earlier steps left) and returns float32 logits at the wanted
places only.

The reference has two disjoint calls instead: ``prefillBatch`` for whole prompts
from position 0 (src/engine/batched_engine.ts:1676-1780) and ``decodeBatch`` for
one token per sequence (:1785-2463), each rebuilding and uploading five host
arrays per call (:2237-2269).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..parts.base import BuildEnv, StepContext
from ..parts.model import DecoderModel


@dataclass
class StepItem:
    """A request's next tokens and the places among them whose logits are wanted."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(RuntimeError):
    """A kernel flagged bad input (token id, cache slot or page id out of range)."""


class _Staging:
    """A small ring of pinned host buffers, so that filling the next step's batch
    description cannot overtake the copy of the previous one."""

    def __init__(self, depth: int = 4):
        self.bufs: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.i = 0

    def take(self, n: int) -> Tuple[torch.Tensor, int]:
        self.i = (self.i + 1) % len(self.bufs)
        ev = self.events[self.i]
        if ev is not None:
            ev.synchronize()
        buf = self.bufs[self.i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1024), dtype=torch.int32, pin_memory=True)
            self.bufs[self.i] = buf
        return buf, self.i

    def sent(self, i: int) -> None:
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class ModelRunner:
    """Owns the model, the cache manager's storage and the step function."""

    def __init__(self, model: DecoderModel, cache: CacheManager, env: BuildEnv):
        if env.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only (there is no CPU path)")
        self.model, self.cache, self.env = model, cache, env
        if any(g.storage is None for g in cache.groups):
            cache.allocate_storage(env.dtype, env.device)
        self.views = model.entry_views(cache)
        self.err = torch.zeros(1, dtype=torch.int32, device=env.device)
        self._staging = _Staging()
        self.steps = 0
        self.h2d_bytes = 0

    # --------------------------------------------------------------- requests
    def add_request(self, rid: Hashable) -> None:
        self.cache.add_request(rid)

    def free_request(self, rid: Hashable) -> None:
        self.cache.free_request(rid)

    # -------------------------------------------------------------- the batch
    def _layout(self, T: int, B: int, R: int, widths: Sequence[int]):
        """Offsets (in int32 elements) of each field inside the batch description."""
        off, fields = 0, {}
        for name, n in (("token_ids", T), ("positions", T), ("seq_of_token", T),
                        ("q_start", B + 1), ("ctx_lens", B), ("state_slots", B),
                        ("logit_rows", R)):
            fields[name] = (off, n)
            off += n
        for g, w in enumerate(widths):
            fields[f"slots{g}"] = (off, T)
            off += T
            fields[f"tables{g}"] = (off, B * w)
            off += B * w
        return fields, off

    def build_context(self, items: Sequence[StepItem]) -> StepContext:
        """Describe ``items`` to the device.  Pages must already be reserved."""
        cache = self.cache
        B = len(items)
        q_lens = [len(it.tokens) for it in items]
        T = sum(q_lens)
        rcs = [cache.get(it.rid) for it in items]
        starts = [rc.length for rc in rcs]
        ctx_lens = [s + n for s, n in zip(starts, q_lens)]
        R = sum(len(it.want) for it in items)
        widths = [max(1, max(len(rc.tables[g.index]) for rc in rcs)) for g in cache.groups]
        fields, total = self._layout(T, B, R, widths)
        host, ring = self._staging.take(total)
        h = host.numpy()

        def view(name):
            a, n = fields[name]
            return h[a:a + n]

        tok, pos, sot = view("token_ids"), view("positions"), view("seq_of_token")
        qs, rows = view("q_start"), view("logit_rows")
        t = r = 0
        for b, it in enumerate(items):
            n = q_lens[b]
            tok[t:t + n] = np.asarray(it.tokens, dtype=np.int32)
            pos[t:t + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
            sot[t:t + n] = b
            qs[b] = t
            for w in it.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {it.rid!r}: wanted place {w} is outside its "
                                     f"{n} tokens of this step")
                rows[r] = t + w
                r += 1
            t += n
        qs[B] = T
        view("ctx_lens")[:] = ctx_lens
        view("state_slots")[:] = [rc.slot for rc in rcs]
        for g in cache.groups:
            w, ps = widths[g.index], g.page_size
            sl = view(f"slots{g.index}")
            tb = view(f"tables{g.index}").reshape(B, w)
            tb[:] = 0
            t = 0
            for b, rc in enumerate(rcs):
                table = np.asarray(rc.tables[g.index], dtype=np.int32)
                tb[b, :len(table)] = table
                p = np.arange(starts[b], ctx_lens[b])
                sl[t:t + q_lens[b]] = table[p // ps] * ps + p % ps
                t += q_lens[b]

        dev = torch.empty(total, dtype=torch.int32, device=self.env.device)
        dev.copy_(host[:total], non_blocking=True)
        self._staging.sent(ring)
        self.h2d_bytes += total * 4

        def dview(name):
            a, n = fields[name]
            return dev[a:a + n]

        return StepContext(
            env=self.env, cache=cache, T=T, B=B,
            token_ids=dview("token_ids"), positions=dview("positions"),
            seq_of_token=dview("seq_of_token"), q_start=dview("q_start"),
            ctx_lens=dview("ctx_lens"), state_slots=dview("state_slots"),
            slots=[dview(f"slots{g.index}") for g in cache.groups],
            block_tables=[dview(f"tables{g.index}").view(B, widths[g.index])
                          for g in cache.groups],
            logit_rows=dview("logit_rows"), err=self.err,
            q_lens=q_lens, ctx_lens_host=ctx_lens, max_q_len=max(q_lens),
            max_ctx_len=max(ctx_lens), decode_only=all(n == 1 for n in q_lens))

    # ---------------------------------------------------------------- the step
    def reserve(self, items: Sequence[StepItem]) -> None:
        """Pages for every item, or :class:`OutOfPages` with nothing changed."""
        wants = [(it.rid, self.cache.get(it.rid).length + len(it.tokens)) for it in items]
        if not self.cache.can_reserve(wants):
            raise OutOfPages(
                f"not enough free pages for this step (free per group: "
                f"{self.cache.num_free_pages()})")
        for rid, new_len in wants:
            self.cache.reserve(rid, new_len)

    def step(self, items: Sequence[StepItem]) -> torch.Tensor:
        """Run the items as one batch; logits ``[R, vocab]`` float32 on the device, in
        the order of the items and of each item's ``want``."""
        if not items:
            raise ValueError("a step needs at least one item")
        seen = set()
        for it in items:
            if len(it.tokens) == 0:
                raise ValueError(f"request {it.rid!r} brings no tokens to this step")
            if it.rid in seen:
                raise ValueError(f"request {it.rid!r} appears twice in one step")
            seen.add(it.rid)
        self.reserve(items)
        for it in items:
            self.cache.zero_fresh_state(self.cache.get(it.rid))
        ctx = self.build_context(items)
        logits = self.model.forward(ctx, self.views)
        for it, new_len in zip(items, ctx.ctx_lens_host):
            self.cache.commit(it.rid, new_len)
        self.steps += 1
        return logits

    def check_errors(self) -> None:
        """Raise if a kernel flagged bad input since the last check (synchronises)."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            what = [name for bit, name in ((1, "token id outside the vocabulary"),
                                           (2, "cache slot outside the pool"),
                                           (4, "page id outside the pool or already released"),
                                           (8, "a bounded wait gave up")) if code & bit]
            raise StepError("kernel error: " + "; ".join(what))
