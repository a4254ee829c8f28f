"""The Python entry point: ``Engine(model).generate(prompt_ids, ...)``.

Option names follow the reference's engine options and generate call
(src/engine/batched_engine.ts:3224-3240: ``maxKvMemoryGB``, ``maxSeqLen`` 4096,
``maxBatchSize`` 64, ``cudaGraphs``; the cache's default size is the server's, a share of
the memory that is free once the weights are loaded, src/serve.ts:987-1002; :3133-3203: ``generate(ids, maxNewTokens,
onToken, sampling)`` returns the generated ids, the stop token included, and stops
early when the callback returns false).  Unlike the reference's ``generate``, which
serves one request and reserves pages for prompt + max tokens at once (:3144), any
number of prompts run together under the continuous-batching scheduler.
"""
from __future__ import annotations

import itertools
import time
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager, plan_pages
from ..config.registry import load_config
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import make_env, model_from_dir, model_from_seed
from .runner import ModelRunner, StepError, StepItem
from .scheduler import FINISHED, PENDING, Request, Scheduled, Scheduler


class Engine:
    def __init__(self, model: Union[str, object], dtype: str = "bfloat16", *,
                 random_seed: Optional[int] = None, random_std: float = 0.02,
                 max_kv_memory_gb: Optional[float] = None, num_pages: Optional[int] = None,
                 gpu_memory_utilization: float = 0.9,
                 page_size: int = 16, max_seq_len: int = 4096, max_batch_size: int = 64,
                 max_tokens_per_step: int = 2048, cuda_graphs: bool = True,
                 look_ahead: bool = True, device: str = "cuda:0",
                 allow_unexpected_tensors: bool = False):
        """``model``: a folder with config.json and safetensors, or (with
        ``random_seed``) a typed configuration whose weights are drawn on the device.

        The cache's size: ``num_pages`` pages per cache group, else ``max_kv_memory_gb``,
        else ``gpu_memory_utilization`` of the device memory that is free once the weights
        are loaded (less 2 GB for activations, logits and graphs), and never more than
        ``max_batch_size`` requests of ``max_seq_len`` tokens can use."""
        self.env = make_env(dtype, device)
        if isinstance(model, str):
            self.config = load_config(model)
            self.model = model_from_dir(model, self.env,
                                        allow_unexpected=allow_unexpected_tensors)
        else:
            if random_seed is None:
                raise ValueError("a configuration without a folder needs random_seed")
            self.config = model
            self.model = model_from_seed(model, self.env, random_seed, std=random_std)
        self.spec = self.model.spec
        self.max_seq_len = int(max_seq_len)
        kv_needs = self.model.kv_needs()
        if num_pages is None:
            esize = 2 if self.env.dtype == torch.bfloat16 else 4
            if max_kv_memory_gb is not None:
                budget = int(max_kv_memory_gb * (1 << 30))
            else:
                free, _ = torch.cuda.mem_get_info(self.env.device)
                budget = max(0, int(free * gpu_memory_utilization) - (2 << 30))
            # per group: a windowed group gets the pages its window needs, not the full pool's
            num_pages = plan_pages(kv_needs, page_size, budget, esize, max_batch_size,
                                   self.max_seq_len, max_tokens_per_step)
        cache = CacheManager(kv_needs, self.model.state_needs(), page_size=page_size,
                             num_pages=num_pages, max_requests=max_batch_size)
        self.runner = ModelRunner(self.model, cache, self.env)
        self.scheduler = Scheduler(cache, max_running=max_batch_size,
                                   max_tokens_per_step=max_tokens_per_step,
                                   max_model_len=max_seq_len)
        self.sampler = Sampler(self.env.device)
        self.cuda_graphs = bool(cuda_graphs)
        if self.cuda_graphs:
            self.runner.enable_decode_graphs(max_batch=max_batch_size, max_seq_len=max_seq_len)
        self.look_ahead = bool(look_ahead)
        self._pending = None        # (plan, sampling handle, sampled items) of the step in flight
        self._ids = itertools.count()
        self.requests: Dict[Hashable, Request] = {}
        self.tokens_prefilled = 0
        self.tokens_decoded = 0
        self.step_ms: List[float] = []
        # with time_gpu set, every step is bracketed by CUDA events: (start, end, tokens)
        self.time_gpu = False
        self.gpu_spans: List[tuple] = []

    # ---------------------------------------------------------------- requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    rid: Optional[Hashable] = None, eos_ids: Optional[Sequence[int]] = None
                    ) -> Hashable:
        rid = next(self._ids) if rid is None else rid
        eos = tuple(self.spec.eos_token_ids) if eos_ids is None else tuple(eos_ids)
        bad = [t for t in prompt if not 0 <= int(t) < self.spec.vocab_size]
        if bad:
            raise ValueError(f"prompt token ids outside the vocabulary "
                             f"(0..{self.spec.vocab_size - 1}): {bad[:8]}")
        req = Request(rid, [int(t) for t in prompt], params or SamplingParams(), eos_ids=eos)
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def warm_up(self) -> None:
        """Capture the decode step's CUDA graph for every batch bucket now, so that no
        request pays for a capture.  (The reference captures after five warm-up calls of a
        batch size, inside generation: src/engine/batched_engine.ts:1813-1830.)  Runs one
        padded single-token step per bucket on a scratch request and frees it again."""
        if not self.cuda_graphs or self.has_work():
            return
        rid = ("warm-up", next(self._ids))
        self.runner.add_request(rid)
        try:
            for _ in range(2 * len(self.runner._buckets)):
                missing = [b for b in self.runner._buckets if b not in self.runner._graphs
                           or self.runner._graphs[b]["graph"] is None]
                if not missing:
                    break
                self.runner.step([StepItem(rid, [0], [0])], bucket=missing[0])
        finally:
            self.runner.free_request(rid)
        torch.cuda.synchronize()

    def abort(self, rid: Hashable) -> None:
        self.scheduler.abort(self.requests[rid])

    # -------------------------------------------------------------------- step
    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._pending is not None

    def _can_look_ahead(self) -> bool:
        """Whether the next step may be launched before the last one's ids are read: its
        decode tokens then come from the device.  Not when a token's value is needed on the
        host first (repetition penalty) or when pages are so short that a request may have
        to be preempted and recomputed from its tokens."""
        running = self.scheduler.running
        if not self.look_ahead or not running:
            return False
        if any(r.params.repetition_penalty != 1.0 for r in running):
            return False
        return self.runner.cache.can_reserve([(r.rid, r.computed + 1) for r in running
                                              if r.remaining == 1])

    def _resolve(self, pending) -> List[Request]:
        """Read back the ids (and the kernels' error word) of a launched step."""
        plan, handle, sampling = pending
        ids, err = self.sampler.finish_with_extra(handle) if handle is not None else ([], 0)
        if err:
            self.runner.err.zero_()
            raise StepError(f"a kernel flagged bad input or a timed-out wait (error bits {err})")
        self.scheduler.resolve(plan, ids)
        return [s.request for s in sampling]

    def _resolve_pending(self) -> List[Request]:
        pending, self._pending = self._pending, None
        return self._resolve(pending)

    def step(self) -> List[Request]:
        """One scheduler iteration: plan, run one mixed batch, sample, record.

        The ids sampled by a step are read back one call later, after the next step has
        been launched, so that planning and describing a step overlap the previous step's
        run on the GPU; tokens that a decoding request needs as input travel from the
        sampler to the next step on the device.  Returns the requests whose token of the
        previous step has now arrived (with their ``output`` updated)."""
        t0 = time.perf_counter()
        arrived: List[Request] = []
        look = self._pending is not None and self._can_look_ahead()
        if self._pending is not None and not look:
            arrived = self._resolve_pending()
        if not self.scheduler.has_work():
            return arrived
        plan, dropped = self.scheduler.schedule()
        if not plan:
            if self._pending is not None:
                arrived += self._resolve_pending()
            return arrived
        prev_rows, prev_ids = {}, None
        if self._pending is not None and self._pending[1] is not None:
            prev_ids = self._pending[1][0]
            prev_rows = {id(s.request): i for i, s in enumerate(self._pending[2])}
        items = []
        for s in plan:
            src = None
            if len(s.tokens) == 1 and s.tokens[0] == PENDING:
                src = prev_rows[id(s.request)]
            items.append(StepItem(s.request.rid, s.tokens, [len(s.tokens) - 1] if s.sample else [],
                                  src_row=src))
        if self.time_gpu:
            ev0 = torch.cuda.Event(enable_timing=True)
            ev0.record()
        logits = self.runner.step(items, device_ids=prev_ids)
        sampling = [s for s in plan if s.sample]
        handle = None
        if sampling:
            handle = self.sampler.start(
                logits, [s.request.params for s in sampling],
                [len(s.request.output) for s in sampling],
                [s.request.output for s in sampling], extra=self.runner.err)
        if self.time_gpu:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self.gpu_spans.append((ev0, ev1, sum(len(s.tokens) for s in plan)))
        for s in plan:
            if len(s.tokens) > 1 or not s.request.output:
                self.tokens_prefilled += len(s.tokens)
            else:
                self.tokens_decoded += 1
        self.scheduler.advance(plan)
        previous, self._pending = self._pending, (plan, handle, sampling)
        if previous is not None:        # looked ahead: now read the step before this one
            arrived += self._resolve(previous)
        self.step_ms.append((time.perf_counter() - t0) * 1e3)
        return arrived

    def flush(self) -> List[Request]:
        """Read back whatever the last step sampled (nothing else is launched)."""
        return self._resolve_pending() if self._pending is not None else []

    # ---------------------------------------------------------------- generate
    def generate(self, prompts, max_tokens: int = 100, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, repetition_penalty: float = 1.0,
                 seed: Optional[int] = None, eos_ids: Optional[Sequence[int]] = None,
                 ignore_eos: bool = False,
                 on_token: Optional[Callable[[int, int], Optional[bool]]] = None):
        """Generate for one prompt (a list of token ids -> a list of ids) or several
        (a list of lists -> a list of lists).  The stop token is kept in the output.
        ``on_token(index_of_prompt, token)`` may return ``False`` to stop that request."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        batch = [prompts] if single else list(prompts)
        rids = []
        try:
            for i, p in enumerate(batch):
                params = SamplingParams(
                    temperature=temperature, top_k=top_k, top_p=top_p,
                    repetition_penalty=repetition_penalty,
                    seed=None if seed is None else seed + i, max_tokens=max_tokens,
                    ignore_eos=ignore_eos)
                rids.append(self.add_request(p, params, eos_ids=eos_ids))
        except Exception:
            # a refused prompt takes the call's earlier prompts with it: nothing of this
            # call may stay queued and run beside a later one
            for rid in rids:
                self.abort(rid)
                self.requests.pop(rid, None)
            raise
        index = {rid: i for i, rid in enumerate(rids)}
        told = {rid: 0 for rid in rids}          # tokens of each request already reported

        def unfinished(r):
            req = self.requests[r]
            return req.state != FINISHED or req.unresolved > 0

        while any(unfinished(r) for r in rids):
            for req in self.step():
                if on_token is None or req.rid not in index:
                    continue
                known = [t for t in req.output if t != PENDING]
                while told[req.rid] < len(known) and req.finish_reason != "abort":
                    tok = known[told[req.rid]]
                    told[req.rid] += 1
                    if on_token(index[req.rid], tok) is False:
                        self.abort(req.rid)
                        del req.output[told[req.rid]:]
        outs = [self.requests.pop(r).output for r in rids]
        return outs[0] if single else outs

    # ------------------------------------------------------------------- stats
    def stats(self) -> dict:
        """Pages, queues and token counts (the reference: src/engine/batched_engine.ts:2993)."""
        cache = self.runner.cache
        return {
            "pages_total": [g.pool.num_pages for g in cache.groups],
            "pages_free": cache.num_free_pages(),
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
            "tokens_prefilled": self.tokens_prefilled,
            "tokens_decoded": self.tokens_decoded,
            "preemptions": self.scheduler.num_preemptions,
            "steps": self.runner.steps,
            "kernel_launches": __import__("binfer_b200.csrc.ops", fromlist=["x"]).launches(),
        }
