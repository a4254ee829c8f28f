"""Sampling on the device from the step's float32 logits.

The reference copies the whole vocabulary of logits to the host for every token
and samples there (src/engine/sampler.ts:57-157; the copy:
src/engine/batched_engine.ts:2282-2283).  Here the penalty, the filters and the
draw run in one kernel per row, and only the chosen ids come back.
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams, uniform


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device
        self.d2h_bytes = 0
        self.h2d_bytes = 0
        self._host = None          # the last uploaded per-row options, and their device copy
        self._dev = None
        self._ring = [None] * 4    # pinned staging buffers and the events of their copies
        self._events = [None] * 4
        self._turn = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draw_index: Sequence[int], generated: Sequence[Sequence[int]]) -> List[int]:
        """One token per row of ``logits [R, V]``.  ``draw_index[r]`` is how many tokens
        request r has drawn so far; ``generated[r]`` feeds the repetition penalty."""
        return self.finish(self.start(logits, params, draw_index, generated))

    def start(self, logits: torch.Tensor, params: Sequence[SamplingParams],
              draw_index: Sequence[int], generated: Sequence[Sequence[int]],
              extra: Optional[torch.Tensor] = None):
        """Launch the sampling and the copy of the ids to pinned host memory; returns a
        handle ``(device ids, host ids, event)`` for :meth:`finish`.  ``extra``: one int32
        word on the device (the kernels' error word) that rides back with the ids."""
        R = logits.shape[0]
        assert R == len(params) == len(draw_index) == len(generated)
        out = self.sample_async(logits, params, draw_index, generated)
        self._id_turn = (getattr(self, "_id_turn", 0) + 1) % 4
        bufs = self.__dict__.setdefault("_id_bufs", [None] * 4)
        host = bufs[self._id_turn]
        if host is None or host.numel() < R + 1:
            host = bufs[self._id_turn] = torch.empty(max(R, 64) + 1, dtype=torch.int32,
                                                     pin_memory=True)
        host[:R].copy_(out, non_blocking=True)
        if extra is not None:
            host[R:R + 1].copy_(extra, non_blocking=True)
        else:
            host[R] = 0
        ev = torch.cuda.Event()
        ev.record()
        self.d2h_bytes += R * 4 + (4 if extra is not None else 0)
        return out, host[:R + 1], ev

    def finish(self, handle) -> List[int]:
        """Wait for a started sampling and return its ids."""
        return self.finish_with_extra(handle)[0]

    def finish_with_extra(self, handle):
        """(ids, the extra word) of a started sampling."""
        _, host, ev = handle
        ev.synchronize()
        vals = host.tolist()
        return vals[:-1], vals[-1]

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     draw_index: Sequence[int], generated: Sequence[Sequence[int]]) -> torch.Tensor:
        R = logits.shape[0]
        host = np.empty((5, R), dtype=np.float32)
        host[0] = [p.temperature for p in params]
        host[1] = [p.top_p for p in params]
        host[2] = [uniform(p.seed, n) if not p.greedy else 0.0
                   for p, n in zip(params, draw_index)]
        host[3] = [p.repetition_penalty for p in params]
        host[4].view(np.int32)[:] = [p.top_k for p in params]
        if self._host is not None and self._host.shape == host.shape and \
                np.array_equal(self._host, host):
            dev = self._dev            # same rows, same options (every greedy decode step)
        else:
            self._turn = (self._turn + 1) % len(self._ring)
            if self._events[self._turn] is not None:
                self._events[self._turn].synchronize()
            pinned = self._ring[self._turn]
            if pinned is None or pinned.shape[1] < R:
                pinned = torch.empty((5, max(R, 64)), dtype=torch.float32, pin_memory=True)
                self._ring[self._turn] = pinned
            pinned[:, :R].copy_(torch.from_numpy(host))
            dev = torch.empty((5, R), dtype=torch.float32, device=self.device)
            dev.copy_(pinned[:, :R], non_blocking=True)
            ev = self._events[self._turn] or torch.cuda.Event()
            ev.record()
            self._events[self._turn] = ev
            self._host, self._dev = host, dev
            self.h2d_bytes += host.nbytes
        if any(p.repetition_penalty != 1.0 for p in params):
            items = [(r, tok, cnt) for r, (p, g) in enumerate(zip(params, generated))
                     if p.repetition_penalty != 1.0 for tok, cnt in Counter(g).items()]
            if items:
                it = torch.tensor(items, dtype=torch.int32).to(self.device)
                ops.repetition_penalty(logits, it, dev[3])
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        ops.sample(logits, dev[0], dev[4].view(torch.int32), dev[1], dev[2], out)
        return out
