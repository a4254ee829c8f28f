"""Continuous batching: admit, cut prompts into portions under a token budget, decode,
finish and free; preempt by recomputation when pages run out.

Policy, step by step:

1. Every running request whose prompt is complete gets one token (decoded tokens
   come first, so the time between a request's tokens stays bounded).
2. What is left of the step's token budget goes to prompt portions of running
   requests, in order of admission; a portion is as long as the budget allows.
3. Waiting requests are admitted first-come-first-served (never out of order)
   while there are fewer than ``max_running`` running, budget is left and the
   page pool can hold the request's first portion.
4. If a running request cannot get the page it needs, the running request that
   was admitted last is preempted: its pages and slot are given back and it
   returns to the *front* of the waiting queue, to be recomputed from its prompt
   plus the tokens it has generated (its draw counter is kept, so it samples
   what it would have sampled).  If the request in need is itself the last one
   running, it is finished with reason ``"cache"``.
5. A request whose prompt plus one token can never fit the pool, or exceeds
   ``max_model_len``, is refused when it is added.

The reference's live loop (src/serve.ts:280-550) admits whenever
``canAllocate(prompt + maxTokens)`` is true, allocates only the prompt's pages
(:335-343), runs a separate prefill forward for whole prompts and a decode
forward (:356-375,422-429), and ignores a failed page allocation while decoding
(:390,476).  Its unused library scheduler marks such a request failed
(src/scheduler/scheduler.ts:290-299) and admits strictly first-come-first-served
(:96-129), which is kept here.
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1      # an output token that was sampled on the device and not yet read back


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    eos_ids: Tuple[int, ...] = ()
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    finish_reason: Optional[str] = None     # "stop" | "length" | "cache" | "abort"
    computed: int = 0                        # tokens of `all_tokens` whose keys are cached
    preemptions: int = 0
    order: int = 0                           # admission order among running requests
    unresolved: int = 0                      # PENDING tokens in `output`
    drop: int = 0                            # sampled tokens still to come that must be discarded

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def remaining(self) -> int:
        """Tokens that must still run before the next token can be sampled."""
        return len(self.prompt) + len(self.output) - self.computed


@dataclass
class Scheduled:
    request: Request
    tokens: List[int]
    sample: bool             # the last of `tokens` completes the sequence: sample after it


class RequestRefused(ValueError):
    pass


class Scheduler:
    def __init__(self, cache: CacheManager, max_running: int = 64,
                 max_tokens_per_step: int = 2048, max_model_len: int = 4096):
        self.cache = cache
        self.max_running = int(max_running)
        self.max_tokens_per_step = int(max_tokens_per_step)
        self.max_model_len = int(max_model_len)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._order = itertools.count()
        self.num_preemptions = 0

    # ------------------------------------------------------------------ adding
    def add(self, req: Request) -> None:
        n = len(req.prompt)
        if n == 0:
            raise RequestRefused(f"request {req.rid!r} has an empty prompt")
        if n + 1 > self.max_model_len:
            raise RequestRefused(f"request {req.rid!r}: prompt of {n} tokens exceeds "
                                 f"max_model_len {self.max_model_len}")
        if not self.cache.can_ever_hold(n + 1):
            raise RequestRefused(f"request {req.rid!r}: prompt of {n} tokens can never fit "
                                 f"the cache ({[g.pool.num_pages for g in self.cache.groups]} "
                                 f"pages of {self.cache.page_size} per group)")
        req.state = WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -------------------------------------------------------------- scheduling
    def schedule(self) -> Tuple[List[Scheduled], List[Request]]:
        """The next step's items (pages are checked here, reserved by the step) and the
        requests that had to be finished for lack of cache while planning."""
        dropped: List[Request] = []
        while True:
            plan = self._plan(dropped)
            if plan or not self.running:
                return plan, dropped
            # nobody can move: every running request is short of pages for its prompt
            victim = max(self.running, key=lambda r: r.order)
            if len(self.running) == 1:
                self._finish(victim, "cache")
                dropped.append(victim)
            else:
                self._preempt(victim, [], [], [], [])

    def _plan(self, dropped: List[Request]) -> List[Scheduled]:
        plan: List[Scheduled] = []
        wants: List[Tuple[Hashable, int]] = []
        costs: List[List[int]] = []          # pages each planned item adds, per cache group
        need = [0] * len(self.cache.groups)  # their running total
        budget = self.max_tokens_per_step
        preemptions_before = self.num_preemptions
        cache = self.cache

        def cost_of(req: Request, n: int) -> List[int]:
            return cache.pages_to_add(cache.get(req.rid), req.computed + n)

        def fits(req: Request, n: int, spare: int = 0) -> bool:
            c = cost_of(req, n)
            return all(g.pool.num_free - need[i] - c[i] >= spare
                       for i, g in enumerate(cache.groups))

        def largest_fit(req: Request, n: int, spare: int = 0) -> int:
            """The longest portion <= n that fits, backing off page by page."""
            ps = self.cache.page_size
            while n > 0 and not fits(req, n, spare):
                n = ((req.computed + n - 1) // ps) * ps - req.computed
            return max(n, 0)

        def take(req: Request, n: int) -> None:
            nonlocal budget
            total = len(req.prompt) + len(req.output)
            if n == 1 and req.computed == total - 1:
                toks = [req.output[-1] if req.output else req.prompt[-1]]
            else:
                toks = req.all_tokens[req.computed:req.computed + n]
            plan.append(Scheduled(req, toks, req.computed + n == total))
            wants.append((req.rid, req.computed + n))
            c = cost_of(req, n)
            costs.append(c)
            for i, v in enumerate(c):
                need[i] += v
            budget -= n

        # 1. one token for every request that is decoding, oldest first
        for req in sorted(self.running, key=lambda r: r.order):
            if req.state != RUNNING or req.remaining != 1 or budget <= 0:
                continue
            while req.state == RUNNING and not fits(req, 1):
                victim = max(self.running, key=lambda r: r.order)
                if victim is req and len(self.running) == 1:
                    self._finish(req, "cache")
                    dropped.append(req)
                else:
                    budget += self._preempt(victim, plan, wants, costs, need)
            if req.state == RUNNING:
                take(req, 1)

        # 2. prompt portions of running requests, in order of admission
        planned = {id(s.request) for s in plan}
        for req in sorted(self.running, key=lambda r: r.order):
            if budget <= 0:
                break
            if req.state != RUNNING or id(req) in planned or req.remaining <= 1:
                continue
            n = largest_fit(req, min(req.remaining, budget))
            if n > 0:
                take(req, n)

        # 3. admission, strictly first come first served; one page per running request
        #    is left free so that those already decoding can go on; nobody is admitted
        #    in a step that had to preempt (the preempted request would come straight back)
        while (self.waiting and len(self.running) < self.max_running and budget > 0
               and self.cache.slots.num_free > 0
               and self.num_preemptions == preemptions_before):
            req = self.waiting[0]
            self.cache.add_request(req.rid)
            n = largest_fit(req, min(req.remaining, budget), spare=len(self.running))
            if n <= 0:
                self.cache.free_request(req.rid)
                break
            self.waiting.popleft()
            req.state, req.order = RUNNING, next(self._order)
            self.running.append(req)
            take(req, n)
        return plan

    def _preempt(self, req: Request, plan: List[Scheduled], wants: List, costs: List,
                 need: List[int]) -> int:
        """Take ``req`` out of the running set and out of the plan; return the budget it frees."""
        freed = 0
        for i, s in enumerate(plan):
            if s.request is req:
                freed = len(s.tokens)
                for g, v in enumerate(costs[i]):
                    need[g] -= v
                del plan[i]
                del wants[i]
                del costs[i]
                break
        self.cache.free_request(req.rid)
        self.running.remove(req)
        req.state, req.computed = WAITING, 0
        req.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)
        return freed

    # ---------------------------------------------------------------- updating
    def update(self, plan: Sequence[Scheduled], sampled: Sequence[int]) -> List[Request]:
        """Record the step: ``sampled`` holds one token per item with ``sample`` set, in
        plan order.  Returns the requests that finished."""
        self.advance(plan)
        return self.resolve(plan, sampled)

    def advance(self, plan: Sequence[Scheduled]) -> None:
        """The step has been launched: cached lengths grow, and every item that samples
        gets a PENDING output token whose value ``resolve`` fills in later.  What does not
        depend on the token's value is decided here: the length limits."""
        for s in plan:
            req = s.request
            req.computed += len(s.tokens)
            if not s.sample:
                continue
            req.output.append(PENDING)
            req.unresolved += 1
            if (len(req.output) >= req.params.max_tokens
                    or len(req.prompt) + len(req.output) >= self.max_model_len):
                self._finish(req, "length")

    def resolve(self, plan: Sequence[Scheduled], sampled: Sequence[int]) -> List[Request]:
        """The sampled ids of an advanced step have arrived.  Returns the requests that
        are finished and have no token outstanding."""
        done: List[Request] = []
        it = iter(sampled)
        for s in plan:
            if not s.sample:
                continue
            req, tok = s.request, int(next(it))
            if req.drop:                     # sampled after the request had stopped
                req.drop -= 1
                continue
            i = req.output.index(PENDING)
            req.output[i] = tok
            req.unresolved -= 1
            stops = () if req.params.ignore_eos else req.eos_ids
            if (tok in stops or tok in req.params.stop_token_ids) and \
                    req.finish_reason in (None, "length"):
                # the stop token stays; whatever was sampled after it is discarded
                req.drop += len(req.output) - (i + 1)
                req.unresolved -= len(req.output) - (i + 1)
                del req.output[i + 1:]
                if req.state != FINISHED:
                    self._finish(req, "stop")
                req.finish_reason = "stop"
            if req.state == FINISHED and req.unresolved == 0:
                done.append(req)
        return done

    def _finish(self, req: Request, reason: str) -> None:
        if req.state == RUNNING:
            self.cache.free_request(req.rid)
            self.running.remove(req)
        elif req.state == WAITING and req in self.waiting:
            self.waiting.remove(req)
        req.state, req.finish_reason = FINISHED, reason

    def abort(self, req: Request) -> None:
        """Stop a request now; tokens it still has outstanding are discarded."""
        if req.state != FINISHED:
            self._finish(req, "abort")
        n = req.output.count(PENDING)
        if n:
            req.drop += n
            req.unresolved -= n
            req.output[:] = [t for t in req.output if t != PENDING]
