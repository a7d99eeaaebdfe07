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
