"""The scheduler's decisions with a stand-in for the step function (CPU):
admission, token budget, portions, decode priority, finishing, and what
happens when pages run out."""

import pytest
import torch

from prism_b200.cache.manager import CacheManager, plan_groups
from prism_b200.config.engine_config import SchedulerConfig
from prism_b200.engine.request import RequestState
from prism_b200.engine.scheduler import Scheduler
from prism_b200.parts.base import CacheNeed
from prism_b200.sampling.rng import uniform
from prism_b200.sampling.sampler import SamplingParams

V = 50


class FakeRunner:
    """Keeps the real cache manager; its "logits" are a fixed function of the
    request's whole token history, so the generated tokens do not depend on
    how the scheduler cut or re-ran the work."""

    def __init__(self, num_pages, page_size=4, max_seqs=8, max_seq_len=256):
        groups, _ = plan_groups([CacheNeed("paged", 1, 8, None)], [None])
        self.cache = CacheManager(groups, page_size, num_pages, max_seqs, max_seq_len)
        self.history, self.steps = {}, []

    def begin_request(self, rid):
        self.cache.add_request(rid)
        self.history[rid] = []

    def end_request(self, rid):
        self.cache.free_request(rid)
        self.history.pop(rid)

    def step(self, segments):
        rows = []
        self.steps.append([(s.req_id, len(s.tokens), self.cache.length(s.req_id)) for s in segments])
        for s in segments:
            self.cache.append(s.req_id, len(s.tokens))
        for s in segments:
            assert len(self.history[s.req_id]) == self.cache.length(s.req_id), "tokens fed out of order"
            self.history[s.req_id] += list(s.tokens)
            for w in s.want:
                h = self.history[s.req_id][:self.cache.length(s.req_id) + w + 1]
                row = torch.zeros(V)
                row[(sum(h) * 7 + len(h)) % V] = 1.0
                rows.append(row)
            self.cache.commit(s.req_id, len(s.tokens))
        self.cache.check_invariants()
        return torch.stack(rows) if rows else None


class FakeSampler:
    def sample(self, logits, temps, us):
        return [int(r.argmax()) for r in logits]


def expected(prompt, n):
    h, out = list(prompt), []
    for _ in range(n):
        t = (sum(h) * 7 + len(h)) % V
        out.append(t)
        h.append(t)
    return out


def make(num_pages=64, **kw):
    runner = FakeRunner(num_pages, **{k: v for k, v in kw.items() if k in ("page_size", "max_seqs", "max_seq_len")})
    cfg = SchedulerConfig(**{k: v for k, v in kw.items() if k in ("max_batch_tokens", "max_num_seqs", "prefill_chunk")})
    return Scheduler(runner, FakeSampler(), cfg, eos_token_id=kw.get("eos")), runner


def test_budget_portions_and_decode_first():
    s, runner = make(max_batch_tokens=16, prefill_chunk=10, max_num_seqs=4)
    a = s.add_request(list(range(1, 24)), SamplingParams(max_new_tokens=3))     # 23 tokens
    b = s.add_request(list(range(5, 12)), SamplingParams(max_new_tokens=3))     # 7 tokens
    s.step()
    assert runner.steps[-1] == [(a.id, 10, 0), (b.id, 6, 0)]                    # chunk cap, then the rest of the budget
    s.step()
    # b has one token left, which makes it a decoding request: it goes first and samples
    assert runner.steps[-1] == [(b.id, 1, 6), (a.id, 10, 10)]
    assert len(b.generated_tokens) == 1 and b.state == RequestState.DECODING and not a.generated_tokens
    s.step()
    assert runner.steps[-1] == [(b.id, 1, 7), (a.id, 3, 20)]                    # decode token first, then the portion
    assert len(a.generated_tokens) == 1 and len(b.generated_tokens) == 2
    s.run_to_completion()
    assert a.generated_tokens == expected(a.prompt_tokens, 3) and b.generated_tokens == expected(b.prompt_tokens, 3)
    assert a.finish_reason == b.finish_reason == "length"
    assert runner.cache.pages_in_use() == 0 and not s.has_work()
    assert s.stats.completed == 2 and s.stats.tokens_generated == 6 and s.stats.prefill_tokens == 30


def test_max_num_seqs_and_fifo_admission():
    s, runner = make(max_num_seqs=2, max_batch_tokens=64)
    reqs = [s.add_request([i + 1] * 5, SamplingParams(max_new_tokens=2)) for i in range(4)]
    s.step()
    assert [x[0] for x in runner.steps[-1]] == [reqs[0].id, reqs[1].id]
    s.step()                                                                     # both finish here (2 tokens each)
    assert reqs[0].state == reqs[1].state == RequestState.FINISHED
    s.step()
    assert [x[0] for x in runner.steps[-1]] == [reqs[2].id, reqs[3].id]           # freed slots are taken at once
    s.run_to_completion()
    assert all(r.generated_tokens == expected(r.prompt_tokens, 2) for r in reqs)


def test_eos_stops_and_is_kept_and_ignore_eos():
    p = [3, 4, 5]
    first = expected(p, 1)[0]
    s, _ = make(eos=first)
    r = s.add_request(p, SamplingParams(max_new_tokens=10))
    q = s.add_request(p, SamplingParams(max_new_tokens=4, ignore_eos=True))
    s.run_to_completion()
    assert r.generated_tokens == [first] and r.finish_reason == "stop"
    assert q.generated_tokens == expected(p, 4) and q.finish_reason == "length"


def test_any_of_several_eos_ids_stops():
    """config.json may list several end-of-sequence ids (chat variants do); each of them ends a request,
    and a request's own ``eos_token_id`` (one id or a list) replaces the model's."""
    p = [2, 3, 4]                                       # six different tokens follow
    toks = expected(p, 6)
    s, _ = make(eos=[V + 7, toks[2]])                   # the second of the two ids comes up third
    r = s.add_request(p, SamplingParams(max_new_tokens=6))
    own = s.add_request(p, SamplingParams(max_new_tokens=6, eos_token_id=[toks[4], V + 9]))
    one = s.add_request(p, SamplingParams(max_new_tokens=6, eos_token_id=toks[0]))
    s.run_to_completion()
    assert r.generated_tokens == toks[:3] and r.finish_reason == "stop"
    assert own.generated_tokens == toks[:5] and own.finish_reason == "stop"
    assert one.generated_tokens == toks[:1] and one.finish_reason == "stop"


def test_tight_pool_does_not_recompute_over_and_over():
    """Two requests that do not fit together: the newer one is preempted once and waits until the older
    one has finished, instead of being admitted again into the few pages left and thrown out a step
    later.  Bound on the work thrown away: each prompt token is prefilled at most twice."""
    s, runner = make(num_pages=12, page_size=4, max_batch_tokens=64, prefill_chunk=64, max_num_seqs=4)
    a = s.add_request([1] * 11, SamplingParams(max_new_tokens=32))
    b = s.add_request([2] * 11, SamplingParams(max_new_tokens=32))
    s.run_to_completion()
    assert a.generated_tokens == expected(a.prompt_tokens, 32) and b.generated_tokens == expected(b.prompt_tokens, 32)
    assert s.stats.preemptions <= 2
    assert s.stats.prefill_tokens <= 2 * 22 + 32          # prompts twice at most, plus one recompute of what b had generated
    assert runner.cache.pages_in_use() == 0


def test_refused_at_submission():
    s, _ = make(num_pages=4, page_size=4, max_seq_len=64)
    with pytest.raises(ValueError, match="empty"):
        s.add_request([])
    with pytest.raises(ValueError, match="sequence limit"):
        s.add_request([1] * 60, SamplingParams(max_new_tokens=10))
    with pytest.raises(ValueError, match="pages"):
        s.add_request([1] * 15, SamplingParams(max_new_tokens=5))       # 20 tokens = 5 pages > 4


def test_prompt_waits_when_pages_are_short():
    s, runner = make(num_pages=6, page_size=4, max_batch_tokens=64, prefill_chunk=64)
    a = s.add_request([1] * 14, SamplingParams(max_new_tokens=4))      # 4 pages now, 5 at the end
    b = s.add_request([2] * 9, SamplingParams(max_new_tokens=2))       # 3 pages
    s.step()
    # a takes 4 pages; b gets only what is left (2 pages = 8 tokens), not an error
    assert runner.steps[-1] == [(a.id, 14, 0), (b.id, 8, 0)]
    s.run_to_completion()
    assert a.generated_tokens == expected(a.prompt_tokens, 4) and b.generated_tokens == expected(b.prompt_tokens, 2)
    assert runner.cache.pages_in_use() == 0


def test_preemption_when_decode_runs_out_of_pages():
    """Two requests that fit at first but not to their ends: the newer one is
    preempted, goes back to the front of the queue, is recomputed from
    prompt + generated, and still yields the same tokens."""
    s, runner = make(num_pages=6, page_size=4, max_batch_tokens=64, prefill_chunk=64)
    a = s.add_request([1] * 10, SamplingParams(max_new_tokens=12))     # 22 tokens = 6 pages alone
    b = s.add_request([2] * 7, SamplingParams(max_new_tokens=6))       # 13 tokens = 4 pages
    c = s.add_request([3] * 3, SamplingParams(max_new_tokens=2))
    order = []
    while s.has_work():
        out = s.step()
        order += [r.id for r, _ in out]
        assert len(runner.cache.requests) <= 3
    assert b.num_preemptions >= 1 and a.num_preemptions == 0           # the oldest request always advances
    assert s.stats.preemptions == b.num_preemptions + c.num_preemptions
    assert a.generated_tokens == expected(a.prompt_tokens, 12)
    assert b.generated_tokens == expected(b.prompt_tokens, 6)
    assert c.generated_tokens == expected(c.prompt_tokens, 2)
    assert runner.cache.pages_in_use() == 0
    # after a preemption the request was fed again from position 0
    refeeds = [st for st in runner.steps for (rid, n, cached) in st if rid == b.id and cached == 0]
    assert len(refeeds) == 1 + b.num_preemptions


def test_sampling_counter_is_the_number_of_generated_tokens():
    assert uniform(4, 2, 3) == uniform(4, 2, 3) and uniform(4, 2, 3) != uniform(4, 2, 4) != uniform(5, 2, 4)
    assert all(0.0 <= uniform(s, r, i) < 1.0 for s in range(3) for r in range(3) for i in range(50))
    mean = sum(uniform(1, 0, i) for i in range(4000)) / 4000
    assert abs(mean - 0.5) < 0.03


# --------------------------------------------------------------------------
# pipelined decoding with stand-ins: the next step takes its tokens from the
# sampler's output of the step before, which the host has not read yet
# --------------------------------------------------------------------------

class PipelinedRunner(FakeRunner):
    def can_run(self, segments):                           # as ModelRunner.can_run: all of them together
        reserve = [0] * len(self.cache.groups)
        for s in segments:
            if not self.cache.can_append(s.req_id, len(s.tokens), reserve):
                return False
            for g, n in enumerate(self.cache.pages_needed(s.req_id, len(s.tokens))):
                reserve[g] += n
        return True

    def step(self, segments, token_source=None):
        if token_source is not None:                       # "device" tokens of the step in flight
            for s, tok in zip(segments, token_source):
                s.tokens = [int(tok)]
        return super().step(segments)


class PipelinedSampler(FakeSampler):
    class Handle:
        def __init__(self, tokens):
            self.device_tokens = tokens

    def __init__(self):
        self.async_steps = 0

    def sample_async(self, logits, temps, us):
        self.async_steps += 1
        return self.Handle([int(r.argmax()) for r in logits])

    def read(self, handle):
        return list(handle.device_tokens)


def make_pipelined(num_pages=64, **kw):
    runner = PipelinedRunner(num_pages, **{k: v for k, v in kw.items() if k in ("page_size", "max_seqs", "max_seq_len")})
    cfg = SchedulerConfig(**{k: v for k, v in kw.items() if k in ("max_batch_tokens", "max_num_seqs", "prefill_chunk")})
    sampler = PipelinedSampler()
    return Scheduler(runner, sampler, cfg, eos_token_id=kw.get("eos")), runner, sampler


def test_pipelined_decoding_gives_the_same_tokens():
    s, runner, sampler = make_pipelined(max_num_seqs=4)
    prompts = [[3, 1, 4], [1, 5, 9, 2, 6], [5, 3], [5, 8, 9, 7]]
    lens = [9, 4, 12, 7]
    reqs = [s.add_request(p, SamplingParams(max_new_tokens=n)) for p, n in zip(prompts, lens)]
    s.run_to_completion()
    assert [r.generated_tokens for r in reqs] == [expected(p, n) for p, n in zip(prompts, lens)]
    assert sampler.async_steps > 0 and runner.cache.pages_in_use() == 0
    runner.cache.check_invariants()


def test_pipelined_decoding_goes_on_while_waiting_requests_have_no_place():
    """Two places, five requests: while both places are taken nobody can be admitted, so decoding is
    pipelined although requests wait; every time a request ends the pipeline drains and the next is admitted."""
    s, runner, sampler = make_pipelined(max_num_seqs=2)
    prompts = [[i + 1, i + 2, i + 3] for i in range(5)]
    reqs = [s.add_request(p, SamplingParams(max_new_tokens=6 + i)) for i, p in enumerate(prompts)]
    s.run_to_completion()
    assert [r.generated_tokens for r in reqs] == [expected(p, 6 + i) for i, p in enumerate(prompts)]
    total = sum(6 + i for i in range(5))
    assert sampler.async_steps >= total // 2 // 2            # most decode steps went through the pipeline
    assert max(len(step) for step in runner.steps) <= 2 and runner.cache.pages_in_use() == 0


def test_pipelined_decoding_stops_at_eos_and_drops_the_token_in_flight():
    prompt = [2, 7, 1]
    eos = expected(prompt, 5)[4]
    s, runner, sampler = make_pipelined(eos=eos)
    a = s.add_request(prompt, SamplingParams(max_new_tokens=20))
    b = s.add_request([9, 9], SamplingParams(max_new_tokens=8, ignore_eos=True))
    s.run_to_completion()
    want_a = expected(prompt, 20)
    assert a.generated_tokens == want_a[:want_a.index(eos) + 1] and a.finish_reason == "stop"
    assert b.generated_tokens == expected([9, 9], 8) and b.finish_reason == "length"
    assert runner.cache.pages_in_use() == 0


# --------------------------------------------------------------------------
# random workloads
# --------------------------------------------------------------------------

class WindowedRunner(FakeRunner):
    """Two cache groups: all keys, and a window of 6 (whose pages come back as the window passes)."""

    def __init__(self, num_pages, page_size=4, max_seqs=8, max_seq_len=256):
        groups, _ = plan_groups([CacheNeed("paged", 1, 8, None), CacheNeed("paged", 1, 8, 6)], [None, None])
        self.cache = CacheManager(groups, page_size, num_pages, max_seqs, max_seq_len)
        self.history, self.steps = {}, []


@pytest.mark.parametrize("seed", range(30))
def test_random_workloads_finish_with_the_same_tokens_and_no_page_lost(seed):
    """Random prompts, lengths, arrival times, budgets and pool sizes (many of them too small for
    everybody at once): every request ends with the tokens it would get alone, whatever was cut,
    made to wait, preempted and recomputed; the pool is whole again at the end."""
    import random
    rnd = random.Random(seed)
    page_size = rnd.choice([2, 4, 8])
    n_req = rnd.randint(3, 12)
    specs = [([rnd.randrange(V) for _ in range(rnd.randint(1, 40))], rnd.randint(1, 20)) for _ in range(n_req)]
    biggest = max((len(p) + n + page_size - 1) // page_size for p, n in specs)
    num_pages = biggest + rnd.randint(0, 2 * biggest)                  # from "one request at a time" to roomy
    runner = (WindowedRunner if seed % 3 == 0 else FakeRunner)(num_pages, page_size, max_seqs=rnd.randint(1, 6))
    cfg = SchedulerConfig(max_batch_tokens=rnd.choice([4, 16, 64]), max_num_seqs=rnd.randint(1, 8),
                          prefill_chunk=rnd.choice([3, 8, 64]), async_decode=False)
    s = Scheduler(runner, FakeSampler(), cfg)
    arrivals = sorted(rnd.randint(0, 30) for _ in specs)
    reqs, steps = [], 0
    while len(reqs) < n_req or s.has_work():
        while len(reqs) < n_req and arrivals[len(reqs)] <= steps:
            p, n = specs[len(reqs)]
            reqs.append(s.add_request(p, SamplingParams(max_new_tokens=n)))
        if s.has_work():
            planned_before = s.stats.steps
            s.step()
            assert s.stats.steps == planned_before + 1, "a step with work to do ran nothing"
            assert sum(n for _, n, _ in runner.steps[-1]) <= cfg.max_batch_tokens
        steps += 1
        assert steps < 5000, "the scheduler does not come to an end"
    for (p, n), r in zip(specs, reqs):
        assert r.state == RequestState.FINISHED and r.generated_tokens == expected(p, n), (r.id, r.num_preemptions)
    assert runner.cache.pages_in_use() == 0 and not runner.cache.requests
    runner.cache.check_invariants()


@pytest.mark.parametrize("seed", range(30))
def test_random_workloads_with_pipelined_decoding_and_eos(seed):
    """The same with an end-of-sequence token and pipelined decoding (one step always in flight while
    only decoding requests run): tokens as alone, cut at the first eos; nothing lost."""
    import random
    rnd = random.Random(1000 + seed)
    page_size = rnd.choice([2, 4, 8])
    eos = rnd.randrange(V)
    specs = [([rnd.randrange(V) for _ in range(rnd.randint(1, 30))], rnd.randint(1, 25), rnd.random() < 0.3)
             for _ in range(rnd.randint(2, 10))]
    biggest = max((len(p) + n + page_size - 1) // page_size for p, n, _ in specs)
    runner = PipelinedRunner(biggest + rnd.randint(0, 2 * biggest), page_size, max_seqs=rnd.randint(1, 6))
    cfg = SchedulerConfig(max_batch_tokens=rnd.choice([8, 64]), max_num_seqs=rnd.randint(1, 8),
                          prefill_chunk=rnd.choice([5, 64]), async_decode=True)
    sampler = PipelinedSampler()
    s = Scheduler(runner, sampler, cfg, eos_token_id=eos)
    reqs = [s.add_request(p, SamplingParams(max_new_tokens=n, ignore_eos=ig)) for p, n, ig in specs]
    s.run_to_completion()
    for (p, n, ig), r in zip(specs, reqs):
        want = expected(p, n)
        if not ig and eos in want:
            want = want[:want.index(eos) + 1]
        assert r.generated_tokens == want, (r.id, r.num_preemptions, r.finish_reason)
        assert r.finish_reason == ("stop" if (not ig and want[-1] == eos) else "length")
    assert runner.cache.pages_in_use() == 0 and not runner.cache.requests
    runner.cache.check_invariants()
