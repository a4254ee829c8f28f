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
    # the (single) token is not known on the host yet: it is row `src_row` of the ids that
    # the previous step sampled, which are still on the device
    src_row: Optional[int] = None


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
        from ..csrc import ops
        self.err = ops.error_word(env.device)
        self._staging = _Staging()
        self.steps = 0
        self.h2d_bytes = 0

    # --------------------------------------------------------------- requests
    def add_request(self, rid: Hashable) -> None:
        self.cache.add_request(rid)

    def free_request(self, rid: Hashable) -> None:
        self.cache.free_request(rid)

    # -------------------------------------------------------------- the batch
    def _layout(self, T: int, B: int, R: int, widths: Sequence[int], n_dec: int = 0,
                n_pf: int = 0):
        """Offsets (in int32 elements) of each field inside the batch description."""
        off, fields = 0, {}
        for name, n in (("token_ids", T), ("positions", T), ("seq_of_token", T),
                        ("q_start", B + 1), ("ctx_lens", B), ("state_slots", B),
                        ("logit_rows", R), ("decode_rows", n_dec), ("prefill_items", 4 * n_pf),
                        ("id_pairs", 2 * B)):
            fields[name] = (off, n)
            off += n
        for g, w in enumerate(widths):
            fields[f"slots{g}"] = (off, T)
            off += T
            fields[f"tables{g}"] = (off, B * w)
            off += B * w
        return fields, off

    def build_context(self, items: Sequence[StepItem], pad_to: Optional[int] = None,
                      widths: Optional[Sequence[int]] = None,
                      dev: Optional[torch.Tensor] = None,
                      device_ids: Optional[torch.Tensor] = None) -> StepContext:
        """Describe ``items`` to the device.  Pages must already be reserved.

        ``pad_to`` (single-token items only) pads the batch with rows that belong to
        no request: token 0 at position 0, writing to and reading from the scratch
        page.  ``widths`` fixes the block tables' widths and ``dev`` the device buffer,
        so that a captured graph finds every field at the same address each time.
        """
        cache = self.cache
        n_real = len(items)
        B = pad_to or n_real
        q_lens = [len(it.tokens) for it in items] + [1] * (B - n_real)
        T = sum(q_lens)
        rcs = [cache.get(it.rid) for it in items]
        starts = [rc.length for rc in rcs] + [0] * (B - n_real)
        ctx_lens = [s + n for s, n in zip(starts, q_lens)]
        if pad_to:
            R = B                               # every row's logits; the caller picks
        else:
            R = sum(len(it.want) for it in items)
        if widths is None:
            widths = [max(1, max(len(rc.tables[g.index]) for rc in rcs)) for g in cache.groups]
        mixed = not pad_to and any(n > 1 for n in q_lens)
        dec = [b for b, n in enumerate(q_lens) if n == 1] if mixed else []
        pf = [b for b, n in enumerate(q_lens) if n > 1] if mixed else []
        fields, total = self._layout(T, B, R, widths, len(dec), len(pf))
        host, ring = self._staging.take(total)
        h = host.numpy()
        h[:total] = 0

        def view(name):
            a, n = fields[name]
            return h[a:a + n]

        tok, pos, sot = view("token_ids"), view("positions"), view("seq_of_token")
        qs, rows = view("q_start"), view("logit_rows")
        pairs: List[Tuple[int, int]] = []
        t = r = 0
        for b, it in enumerate(items):
            n = q_lens[b]
            if n == 1:
                if it.src_row is not None:
                    pairs.append((t, it.src_row))
                    tok[t] = 0
                else:
                    tok[t] = it.tokens[0]
                pos[t] = starts[b]
                sot[t] = b
            else:
                tok[t:t + n] = it.tokens
                pos[t:t + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
                sot[t:t + n] = b
            qs[b] = t
            if not pad_to:
                for w in it.want:
                    if not 0 <= w < n:
                        raise ValueError(f"request {it.rid!r}: wanted place {w} is outside "
                                         f"its {n} tokens of this step")
                    rows[r] = t + w
                    r += 1
            t += n
        if mixed:
            view("decode_rows")[:] = [int(qs[b]) for b in dec]
            items4 = view("prefill_items").reshape(len(pf), 4)
            for i, b in enumerate(pf):
                items4[i] = (b, int(qs[b]), q_lens[b], starts[b])
        for b in range(n_real, B):              # padding rows
            sot[b] = b
            qs[b] = b
        qs[B] = T
        if pad_to:
            rows[:] = np.arange(B, dtype=np.int32)
        view("ctx_lens")[:] = ctx_lens
        view("state_slots")[:n_real] = [rc.slot for rc in rcs]
        for g in cache.groups:
            gi, w, ps = g.index, widths[g.index], g.page_size
            sl = view(f"slots{gi}")
            tb = view(f"tables{gi}").reshape(B, w)
            t = 0
            for b, rc in enumerate(rcs):
                table = rc.table_array(gi)
                if len(table) > w:
                    raise ValueError(f"request {rc.rid!r} holds {len(table)} pages, the "
                                     f"block table has room for {w}")
                tb[b, :len(table)] = table
                n, start = q_lens[b], starts[b]
                if n == 1:
                    sl[t] = int(table[start // ps]) * ps + start % ps
                else:
                    p = np.arange(start, start + n)
                    sl[t:t + n] = table[p // ps] * ps + p % ps
                t += n

        if pairs:
            view("id_pairs")[:2 * len(pairs)] = np.asarray(pairs, dtype=np.int32).reshape(-1)
        if dev is None:
            dev = torch.empty(total, dtype=torch.int32, device=self.env.device)
        dev[:total].copy_(host[:total], non_blocking=True)
        self._staging.sent(ring)
        self.h2d_bytes += total * 4

        def dview(name):
            a, n = fields[name]
            return dev[a:a + n]

        if pairs:
            if device_ids is None:
                raise ValueError("an item takes its token from the device, but no ids were given")
            from ..csrc import ops
            ops.copy_ids(dview("token_ids"), device_ids, dview("id_pairs"), len(pairs))

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
            max_ctx_len=max(ctx_lens), decode_only=all(n == 1 for n in q_lens),
            decode_rows=dview("decode_rows") if dec else None, n_decode=len(dec),
            max_decode_ctx=max([ctx_lens[b] for b in dec], default=1),
            prefill_items=dview("prefill_items").view(len(pf), 4) if pf else None,
            n_prefill=len(pf), max_prefill_rows=max([q_lens[b] for b in pf], default=0))

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

    def step(self, items: Sequence[StepItem], device_ids: Optional[torch.Tensor] = None,
             bucket: Optional[int] = None) -> torch.Tensor:
        """Run the items as one batch; logits ``[R, vocab]`` float32 on the device, in
        the order of the items and of each item's ``want``.  ``device_ids``: int32 ids on
        the device from which items with ``src_row`` take their token.  ``bucket``: run a
        step of single tokens from the graph of this batch bucket (a larger one than the
        items need: how the graphs are captured ahead of the first request)."""
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
        new_lens = [self.cache.get(it.rid).length + len(it.tokens) for it in items]
        if self._can_replay(items, new_lens):
            logits = self._graph_step(items, device_ids, bucket)
        else:
            ctx = self.build_context(items, device_ids=device_ids)
            logits = self.model.forward(ctx, self.views)
        for it, new_len in zip(items, new_lens):
            self.cache.commit(it.rid, new_len)
        self.steps += 1
        return logits

    # ------------------------------------------------------- captured decoding
    def enable_decode_graphs(self, max_batch: int = 64, max_seq_len: int = 4096) -> None:
        """Replay steps that hold only single tokens from CUDA graphs, one graph per
        batch-size bucket (1, 2, 4, ... up to ``max_batch``), captured at first use.

        The reference captures decode only for batches up to 8 and relies on its
        allocator handing back the same addresses (src/engine/batched_engine.ts:1790,
        2152-2164); its padded rows write into block 0 of a live request (:2060-2078).
        Here every input sits in a fixed buffer per bucket, and padded rows use the
        scratch page.  The returned logits are a view of the graph's output buffer:
        they are valid until the next step of the same bucket.
        """
        buckets = [b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b < max_batch]
        self._buckets = sorted(set(buckets + [int(max_batch)]))
        self._graph_seq_len = int(max_seq_len)
        self._graphs = {}

    def _can_replay(self, items: Sequence[StepItem], new_lens: Sequence[int]) -> bool:
        return (getattr(self, "_buckets", None) is not None
                and len(items) <= self._buckets[-1]
                and all(len(it.tokens) == 1 for it in items)
                and max(new_lens) <= self._graph_seq_len)

    def _graph_step(self, items: Sequence[StepItem], device_ids: Optional[torch.Tensor] = None,
                    bucket: Optional[int] = None) -> torch.Tensor:
        B = len(items)
        if bucket is None:
            bucket = next(b for b in self._buckets if b >= B)
        elif bucket not in self._buckets or bucket < B:
            raise ValueError(f"no graph bucket {bucket} for {B} items")
        widths = [-(-self._graph_seq_len // g.page_size) for g in self.cache.groups]
        st = self._graphs.get(bucket)
        if st is None:
            _, total = self._layout(bucket, bucket, bucket, widths)
            st = {"dev": torch.zeros(total, dtype=torch.int32, device=self.env.device),
                  "graph": None, "logits": None}
            self._graphs[bucket] = st
        ctx = self.build_context(items, pad_to=bucket, widths=widths, dev=st["dev"],
                                 device_ids=device_ids)
        ctx.max_ctx_len = self._graph_seq_len     # launch shapes must not follow the batch
        if st["graph"] is None:
            logits = self.model.forward(ctx, self.views)      # this step's result, eagerly
            torch.cuda.synchronize()
            from ..csrc import ops
            graph = torch.cuda.CUDAGraph()
            before = ops.launches()
            with torch.cuda.graph(graph):
                st["logits"] = self.model.forward(ctx, self.views)
            st["graph"] = graph
            st["own_kernels"] = ops.launches() - before     # this library's kernels per replay
            self.graph_captures = getattr(self, "graph_captures", 0) + 1
        else:
            st["graph"].replay()
            logits = st["logits"]
            self.graph_kernel_launches = (getattr(self, "graph_kernel_launches", 0)
                                          + st["own_kernels"])
            self.graph_replays = getattr(self, "graph_replays", 0) + 1
        rows = [b for b, it in enumerate(items) if len(it.want) > 0]
        if len(rows) == B:
            return logits[:B]
        return logits[torch.tensor(rows, dtype=torch.long, device=self.env.device)] \
            if rows else logits[:0]

    def check_errors(self) -> None:
        """Raise if a kernel flagged bad input since the last check (synchronises)."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            what = [name for bit, name in ((1, "token id outside the vocabulary"),
                                           (2, "cache slot outside the pool"),
                                           (4, "page id outside the pool or already released"),
                                           (8, "a bounded wait gave up"),
                                           (16, "a row's context needs more key splits than "
                                                "the attention scratch holds")) if code & bit]
            raise StepError("kernel error: " + "; ".join(what))
