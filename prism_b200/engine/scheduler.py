"""Continuous-batching scheduler above the step function.

andre-fu/prism's hot loop (engine/scheduler.py:189-281) prefills up to eight
popped requests one after the other, each alone and whole, then decodes every
active request in one batch; it has no token budget (``max_batch_tokens`` is
never read, engine/config.py:39), checks for the end of a request one
iteration late (:245), and when pages run out fails the request - or, in a
decode batch, every request of the batch (:230-235,274-281).

Here each step is planned under a token budget: one token for every request
that is decoding, then portions of prompts in admission order, then new
admissions.  A request is "decoding" when exactly one of its tokens is not yet
in the cache, so a preempted request that is recomputed needs no special case.

When pages run out:
  * a prompt portion that does not fit is shortened to what fits, or waits;
  * if a decoding request cannot get the page its next token needs, the most
    recently admitted running request is preempted: its pages and slot are
    given back, it returns to the *front* of the waiting queue and is later
    recomputed from prompt + generated tokens (its sampling counter is the
    number of generated tokens, so its draws do not change);
  * a request that could not fit even alone is refused at ``add_request``.
A plan that had to preempt admits nobody in the same call, and a request that
has been preempted before is admitted again, while others run, only when the
free pages hold all it has to recompute plus a page of growth for everyone
running: the few pages that a preemption leaves would otherwise go back to the
victim, which would recompute a portion only to be thrown out again a step later.

A sequence ends at any of the model's end-of-sequence ids (config.json may
list several) or at the request's own ``SamplingParams.eos_token_id``.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass
from typing import Deque, FrozenSet, List, Optional, Tuple

from ..config.engine_config import SchedulerConfig
from ..sampling.rng import uniform
from ..sampling.sampler import SamplingParams
from .batch import Segment
from .request import Request, RequestState


@dataclass
class SchedulerStats:
    """Counters in the manner of engine/scheduler.py:425-433."""
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    tokens_generated: int = 0
    completed: int = 0
    preemptions: int = 0


def eos_set(eos) -> FrozenSet[int]:
    """None, one id or several ids as a set."""
    if eos is None:
        return frozenset()
    if isinstance(eos, int):
        return frozenset((eos,))
    return frozenset(int(e) for e in eos)


class Scheduler:
    """``runner`` needs ``cache`` (a CacheManager), ``begin_request``,
    ``end_request`` and ``step(segments) -> logits``; ``sampler`` needs
    ``sample(logits, temperatures, us) -> token ids``."""

    def __init__(self, runner, sampler, config: Optional[SchedulerConfig] = None,
                 eos_token_id=None, seed: int = 0):
        self.runner, self.sampler = runner, sampler
        self.cache = runner.cache
        self.config = config or SchedulerConfig()
        self.eos_token_ids = eos_set(eos_token_id)       # one id, several, or none
        self.seed = seed
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in admission order
        self.finished: List[Request] = []
        self.stats = SchedulerStats()
        self._next_id = 0

    # ---- submission ---------------------------------------------------------------
    def add_request(self, prompt_tokens, params: Optional[SamplingParams] = None) -> Request:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt_tokens]
        if not prompt:
            raise ValueError("empty prompt")
        if params.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        total = len(prompt) + params.max_new_tokens
        if total > self.cache.max_seq_len:
            raise ValueError(f"prompt ({len(prompt)}) + max_new_tokens ({params.max_new_tokens}) exceeds "
                             f"the sequence limit {self.cache.max_seq_len}")
        pages = (total + self.cache.page_size - 1) // self.cache.page_size
        for g in self.cache.groups:
            if g.kind == "paged" and g.need.window is None and pages > self.cache.allocators[g.index].num_pages:
                raise ValueError(f"request needs {pages} pages, the pool has {self.cache.allocators[g.index].num_pages}")
        req = Request(self._next_id, prompt, params, arrival_time=time.time())
        self._next_id += 1
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- planning -----------------------------------------------------------------
    def _fits(self, req_id, n: int, reserve: List[int]) -> int:
        """Largest m <= n tokens that request can append given ``reserve``."""
        while n > 0 and not self.cache.can_append(req_id, n, reserve):
            # shrink to the end of the last page that is still affordable
            length = self.cache.length(req_id)
            P = self.cache.page_size
            free = min((self.cache.allocators[g.index].num_free - reserve[g.index])
                       for g in self.cache.groups if g.kind == "paged")
            have = min(len(self.cache.requests[req_id].pages[g.index]) for g in self.cache.groups if g.kind == "paged")
            room = (have + max(free, 0)) * P - length
            n = min(n - 1, room)
        return max(n, 0)

    def _reserve(self, req_id, n: int, reserve: List[int]) -> None:
        for g, k in enumerate(self.cache.pages_needed(req_id, n)):
            reserve[g] += k

    def _room_to_recompute(self, req: Request, reserve: List[int]) -> bool:
        """Whether the free pages hold every token ``req`` has so far, one more, and a page of growth
        for each running request (groups with a window need a few pages only and are not asked)."""
        P = self.cache.page_size
        want = (len(req.prompt_tokens) + len(req.generated_tokens) + 1 + P - 1) // P + len(self.running)
        return all(self.cache.allocators[g.index].num_free - reserve[g.index] >= want
                   for g in self.cache.groups if g.kind == "paged" and g.need.window is None)

    def _preempt(self, req: Request) -> None:
        self.runner.end_request(req.id)
        self.running.remove(req)
        req.num_computed = 0
        req.state = RequestState.WAITING
        req.num_preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(req)

    def plan(self) -> List[Tuple[Request, int]]:
        """Decide this step's batch: ``[(request, number of its next tokens)]``.
        Admits and preempts as a side effect; launches nothing."""
        cfg = self.config
        has_paged = any(g.kind == "paged" for g in self.cache.groups)
        preempted = False
        while True:
            reserve = [0] * len(self.cache.groups)
            batch: List[Tuple[Request, int]] = []
            budget = cfg.max_batch_tokens
            victim = None
            # 1. one token for every decoding request
            for req in self.running:
                if req.remaining != 1 or budget <= 0:
                    continue
                if has_paged and not self.cache.can_append(req.id, 1, reserve):
                    victim = self.running[-1]
                    break
                self._reserve(req.id, 1, reserve)
                batch.append((req, 1))
                budget -= 1
            if victim is not None:
                self._preempt(victim)
                preempted = True
                continue
            # 2. portions of prompts already admitted
            for req in self.running:
                if req.remaining <= 1 or budget <= 0:
                    continue
                n = min(req.remaining, cfg.prefill_chunk, budget)
                n = self._fits(req.id, n, reserve) if has_paged else n
                if n > 0:
                    self._reserve(req.id, n, reserve)
                    batch.append((req, n))
                    budget -= n
            # 3. admissions
            while self.waiting and budget > 0 and len(self.running) < cfg.max_num_seqs \
                    and self.cache.has_free_slot() and not (preempted and self.running):
                req = self.waiting[0]
                if req.num_preemptions and self.running and has_paged and not self._room_to_recompute(req, reserve):
                    break
                self.runner.begin_request(req.id)
                n = min(req.remaining, cfg.prefill_chunk, budget)
                n = self._fits(req.id, n, reserve) if has_paged else n
                if n <= 0:
                    self.runner.end_request(req.id)
                    break
                self.waiting.popleft()
                self.running.append(req)
                req.state = RequestState.PREFILLING
                self._reserve(req.id, n, reserve)
                batch.append((req, n))
                budget -= n
            if batch or not self.running:
                return batch
            # nothing can move although requests are running: free the newest one's pages
            self._preempt(self.running[-1])
            preempted = True

    # ---- one step -----------------------------------------------------------------
    def step(self) -> List[Tuple[Request, int]]:
        """Plan, run, sample, finish.  Returns ``[(request, new token)]``."""
        batch = self.plan()
        if not batch:
            return []
        segs, sampled = [], []
        for req, n in batch:
            toks = req.next_tokens(n)
            last = req.num_computed + n == len(req.prompt_tokens) + len(req.generated_tokens)
            segs.append(Segment(req.id, toks, [n - 1] if last else []))
            if last:
                sampled.append(req)
            if n == 1 and req.num_computed >= len(req.prompt_tokens):
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += n
        logits = self.runner.step(segs)
        for req, n in batch:
            req.num_computed += n
        self.stats.steps += 1
        out = []
        if sampled:
            temps = [r.params.temperature for r in sampled]
            us = [uniform(r.params.seed if r.params.seed is not None else self.seed, r.id,
                          len(r.generated_tokens)) for r in sampled]
            tokens = self.sampler.sample(logits, temps, us)
            now = time.time()
            for req, tok in zip(sampled, tokens):
                req.generated_tokens.append(int(tok))
                req.state = RequestState.DECODING
                if len(req.generated_tokens) == 1:
                    req.first_token_time = now
                self.stats.tokens_generated += 1
                out.append((req, int(tok)))
                self._maybe_finish(req, int(tok), now)
        return out

    def _ends(self, req: Request, tok: int) -> bool:
        """Whether ``tok`` is an end-of-sequence token for this request."""
        if req.params.ignore_eos:
            return False
        eos = eos_set(req.params.eos_token_id) if req.params.eos_token_id is not None else self.eos_token_ids
        return tok in eos

    def _maybe_finish(self, req: Request, tok: int, now: float) -> None:
        reason = None
        if self._ends(req, tok):
            reason = "stop"                      # the eos token stays in the output (scheduler.py:245)
        elif len(req.generated_tokens) >= req.params.max_new_tokens:
            reason = "length"
        if reason:
            req.finish_reason, req.state, req.done_time = reason, RequestState.FINISHED, now
            self.runner.end_request(req.id)      # pages and slot are free before the next plan
            self.running.remove(req)
            self.finished.append(req)
            self.stats.completed += 1

    # ---- pipelined decoding ---------------------------------------------------------
    def _steady(self) -> bool:
        """Only decoding requests, and nobody who could be admitted (nobody waiting, or no
        place for another request until one finishes): the next steps have the same rows in the
        same order, so a step can be launched before the previous step's tokens have been read."""
        nobody_to_admit = (not self.waiting or len(self.running) >= self.config.max_num_seqs
                           or not self.cache.has_free_slot())
        return (self.config.async_decode and hasattr(self.sampler, "sample_async") and nobody_to_admit
                and bool(self.running) and len(self.running) <= self.config.max_batch_tokens
                and all(r.remaining == 1 and r.generated_tokens for r in self.running))

    def _pipelined_decode(self) -> bool:
        """Decode the running set with one step always in flight: step i+1 takes its
        token ids on the device from step i's sampler output, and the host reads
        step i's tokens while step i+1 runs.  The pipeline drains when a request
        finishes (its one extra token is dropped), when pages run out, or when a
        request will reach its length limit; the ordinary ``step`` takes over.
        Returns False if it could not launch anything."""
        reqs = list(self.running)
        seed_of = [r.params.seed if r.params.seed is not None else self.seed for r in reqs]
        temps = [r.params.temperature for r in reqs]
        n_launched = [len(r.generated_tokens) for r in reqs]       # tokens sampled or in flight, per request
        inflight = []                                                  # sample handles, oldest first
        source = None
        stop = False
        while True:
            # launch the next step unless something ends the steady state
            if not stop:
                if any(n >= r.params.max_new_tokens for n, r in zip(n_launched, reqs)):
                    stop = True
                elif not all(self.cache.can_append(r.id, 1) for r in reqs) or not self.runner.can_run(
                        [Segment(r.id, [0], [0]) for r in reqs]):
                    stop = True
            if not stop:
                segs = [Segment(r.id, [r.generated_tokens[-1] if source is None else 0], [0]) for r in reqs]
                logits = self.runner.step(segs, token_source=source)
                us = [uniform(sd, r.id, n) for sd, r, n in zip(seed_of, reqs, n_launched)]
                h = self.sampler.sample_async(logits, temps, us)
                source = h.device_tokens
                inflight.append(h)
                for i in range(len(reqs)):
                    n_launched[i] += 1
                self.stats.steps += 1
                self.stats.decode_tokens += len(reqs)
            if not inflight:
                return False
            if len(inflight) < 2 and not stop:
                continue                                               # keep one step ahead
            tokens = self.sampler.read(inflight.pop(0))
            now = time.time()
            for req, tok in zip(reqs, tokens):
                if req.state == RequestState.FINISHED:
                    continue                                           # a token computed past its end: dropped
                req.num_computed += 1
                req.generated_tokens.append(int(tok))
                self.stats.tokens_generated += 1
                if self._ends(req, int(tok)):
                    req.finish_reason = "stop"
                elif len(req.generated_tokens) >= req.params.max_new_tokens:
                    req.finish_reason = "length"
                if req.finish_reason:
                    req.state, req.done_time = RequestState.FINISHED, now
                    stop = True
            if stop and not inflight:
                break
        for req in reqs:                                               # pages are given back once nothing in flight uses them
            if req.state == RequestState.FINISHED:
                self.runner.end_request(req.id)
                self.running.remove(req)
                self.finished.append(req)
                self.stats.completed += 1
        return True

    def run_to_completion(self) -> None:
        while self.has_work():
            if not (self._steady() and self._pipelined_decode()):
                self.step()
