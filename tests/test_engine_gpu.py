"""Generation through the entry point, decode graphs, sampling, preemption,
long decoding and the replay program, against the plain implementation (GPU)."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import (P, TINY, compare_with_plain, model_folder, plain_logits, plain_model, random_tokens,
                     trace_budget, trace_mixed)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(name, dtype, **kw):
    from prism_b200 import Engine, EngineConfig, SchedulerConfig
    sched = SchedulerConfig(**{k: kw.pop(k) for k in ("max_batch_tokens", "max_num_seqs", "prefill_chunk") if k in kw})
    ec = EngineConfig(kv_page_size=kw.pop("page_size", TINY[name][2]), num_pages=kw.pop("num_pages", 64),
                      use_cuda_graph=kw.pop("graph", False), graph_batch_sizes=(1, 2, 4), scheduler=sched, **kw)
    return Engine(model_folder(name), ec, dtype=dtype)


def near_greedy(name, prompt, tokens, slack):
    """Every generated token is the plain model's best token given the same
    history, up to a logit gap of ``slack`` (bf16 may flip a near-tie)."""
    for i, tok in enumerate(tokens):
        lg = plain_logits(name, list(prompt) + list(tokens[:i]))[-1]
        assert float(lg.max() - lg[tok]) <= slack * float(lg.abs().max()) + 1e-6, (i, tok)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_greedy_generation_matches_the_plain_model(name):
    from prism_b200 import SamplingParams
    cfg, t = plain_model(name)
    vocab = TINY[name][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 10 + n) for n in (5, 17, 33)]
    want = [P.generate(cfg, t, p, 8) for p in prompts]
    got = engine(name, "float32").generate(prompts, SamplingParams(max_new_tokens=8))
    assert [r.token_ids for r in got] == want and all(r.finish_reason == "length" for r in got)
    got16 = engine(name, "bfloat16").generate(prompts, SamplingParams(max_new_tokens=8))
    for p, r in zip(prompts, got16):
        near_greedy(name, p, r.token_ids, 0.03)


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16"), ("A", "bfloat16")])
def test_decode_graphs_give_the_eager_result(name, dtype):
    """Chunked prefill mixed with decode, then decode steps replayed from captured
    graphs (buckets 1, 2, 4 with padding rows): same tokens as without graphs."""
    from prism_b200 import SamplingParams
    vocab = TINY[name][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 70 + n) for n in (1, 9, 40)]
    sp = [SamplingParams(max_new_tokens=n) for n in (12, 7, 9)]
    a = engine(name, dtype, graph=False, prefill_chunk=16, max_batch_tokens=24).generate(prompts, sp)
    eg = engine(name, dtype, graph=True, prefill_chunk=16, max_batch_tokens=24)
    b = eg.generate(prompts, sp)
    assert [r.token_ids for r in a] == [r.token_ids for r in b]
    assert eg.runner.graph_kernel_launches > 0 and {key[0] for key in eg.runner._graphs} <= {1, 2, 4}
    b2 = eg.generate(prompts, sp)                       # the captured graphs again, other pages
    assert [r.token_ids for r in b2] == [r.token_ids for r in b]


def test_warmup_captures_the_decode_graphs_ahead_of_the_first_request():
    """``Engine.warmup()``: every bucket's graphs (with and without the merge of split contexts) exist before the
    first request, and generation then captures nothing more and gives the tokens of an engine without graphs."""
    from prism_b200 import SamplingParams
    vocab = TINY["D"][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 170 + n) for n in (3, 90, 260)]
    sp = [SamplingParams(max_new_tokens=n) for n in (9, 12, 7)]
    eg = engine("D", "bfloat16", graph=True)
    eg.warmup()
    buckets = set(eg.runner.graph_batch_sizes)
    assert {key[0] for key in eg.runner._graphs} == buckets and len(eg.runner._graphs) == 2 * len(buckets)
    before = set(eg.runner._graphs)
    got = eg.generate(prompts, sp)
    assert set(eg.runner._graphs) == before and eg.runner.graph_kernel_launches > 0
    want = engine("D", "bfloat16", graph=False).generate(prompts, sp)
    assert [r.token_ids for r in got] == [r.token_ids for r in want]


def test_temperature_sampling_matches_the_plain_sampler():
    """Config B's workload: prompts 1/9/40/71, prefill in portions of 16 mixed with
    decode, 6 tokens at temperature 0.7 from seed 4 - the same draws as the plain
    loop, whose uniform numbers are keyed by (seed, request, step)."""
    from prism_b200 import SamplingParams
    cfg, t = plain_model("B")
    prompts = [random_tokens(320, n, 3 + n) for n in (1, 9, 40, 71)]
    eng = engine("B", "float32", prefill_chunk=16, max_batch_tokens=40)
    got = eng.generate(prompts, SamplingParams(max_new_tokens=6, temperature=0.7, seed=4))
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert r.token_ids == P.generate(cfg, t, p, 6, temperature=0.7, seed=4, request_index=i)
    assert len({tuple(r.token_ids) for r in got}) > 1


def test_preemption_recomputes_and_keeps_the_tokens():
    """A pool too small for all running requests to reach their ends: requests
    are preempted and recomputed, and the tokens are those of an ample pool."""
    from prism_b200 import SamplingParams
    prompts = [random_tokens(256, n, 90 + n) for n in (20, 14, 9)]
    sp = SamplingParams(max_new_tokens=24)
    ample = engine("A", "float32", num_pages=64).generate(prompts, sp)
    tight = engine("A", "float32", num_pages=6, page_size=8)     # 48 tokens of cache for 44 + 38 + 33
    got = tight.generate(prompts, sp)
    assert tight.stats.preemptions > 0 and sum(r.num_preemptions for r in got) == tight.stats.preemptions
    assert [r.token_ids for r in got] == [r.token_ids for r in ample]
    assert tight.cache.pages_in_use() == 0
    cfg, t = plain_model("A")
    assert got[0].token_ids == P.generate(cfg, t, prompts[0], 24)


def test_preemption_under_pipelined_decoding_with_graphs_in_bfloat16():
    """Everything on at once, on the tensor-core kernels (config D: heads of 64): decode graphs, pipelined
    decoding (a step launched before the last one's tokens are read) and a pool too small for the running
    requests, so that requests are preempted while a step may be in flight and recomputed later from
    pages that others have used.  The tokens are those of an ample pool, and the plain model's."""
    from prism_b200 import SamplingParams
    vocab = TINY["D"][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 600 + n) for n in (70, 45, 100, 20)]
    sp = SamplingParams(max_new_tokens=60)
    kw = dict(graph=True, page_size=32, max_num_seqs=4, prefill_chunk=64, max_batch_tokens=128)
    ample_eng = engine("D", "bfloat16", num_pages=64, **kw)
    ample = ample_eng.generate(prompts, sp)
    assert ample_eng.stats.preemptions == 0
    tight_eng = engine("D", "bfloat16", num_pages=12, **kw)           # 384 tokens of cache for 130 + 105 + 160 + 80
    assert tight_eng.scheduler.config.async_decode
    got = tight_eng.generate(prompts, sp)
    assert tight_eng.stats.preemptions > 0 and tight_eng.runner.graph_kernel_launches > 0
    assert tight_eng.cache.pages_in_use() == 0
    for p, a, b in zip(prompts, ample, got):
        assert len(b.token_ids) == 60
        near_greedy("D", p, b.token_ids, 0.03)
        if a.token_ids != b.token_ids:
            # recomputing a request cuts its work differently, which changes bfloat16 rounding: the two runs may
            # part ways, but only where the plain model itself sees a near-tie between the two tokens
            i = next(j for j, (x, y) in enumerate(zip(a.token_ids, b.token_ids)) if x != y)
            lg = plain_logits("D", list(p) + list(b.token_ids[:i]))[-1]
            assert abs(float(lg[a.token_ids[i]] - lg[b.token_ids[i]])) <= 0.03 * float(lg.abs().max()), (i, a.token_ids[i], b.token_ids[i])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype):
    """One token a step from the first position on, for 300 steps across many
    pages (and far beyond the window of config D's upper layer)."""
    from test_replay_gpu import TOL, make_runner
    from helpers import run_trace
    seq = random_tokens(301, 300, 5)
    steps = [dict(step=i, entries=[dict(id="r", tokens=[tok], want=[0])], end=["r"] if i == 299 else [])
             for i, tok in enumerate(seq)]
    runner = make_runner("D", dtype, num_pages=10)        # 10 pages of 32
    got = run_trace(runner, steps)
    worst, where = compare_with_plain("D", {"r": seq}, got, **TOL[dtype])
    assert len(got) == 300


def test_decode_many_requests_with_graphs_and_padding_rows():
    """Up to 7 requests decoding in a bucket of 8: padded rows must not disturb
    anything (they write to the scratch page)."""
    from prism_b200 import Engine, EngineConfig, SamplingParams, SchedulerConfig
    cfg, t = plain_model("A")
    ec = EngineConfig(kv_page_size=16, num_pages=40, use_cuda_graph=True, graph_batch_sizes=(8,),
                      scheduler=SchedulerConfig(max_num_seqs=8))
    eng = Engine(model_folder("A"), ec, dtype="float32")
    prompts = [random_tokens(256, 3 + 2 * i, 200 + i) for i in range(7)]
    sp = [SamplingParams(max_new_tokens=4 + i) for i in range(7)]
    got = eng.generate(prompts, sp)
    for p, s, r in zip(prompts, sp, got):
        assert r.token_ids == P.generate(cfg, t, p, s.max_new_tokens)


@pytest.mark.parametrize("name", ["D", "B"])
def test_decoding_requests_beside_a_prompt_portion(name, monkeypatch):
    """Five requests are decoding when a long prompt arrives and is prefilled in portions beside them:
    in those steps the single tokens go through the decode attention kernel and the portion through
    the prefill kernel.  Everybody's tokens are the plain model's."""
    from prism_b200 import SamplingParams, ops
    monkeypatch.setattr(ops, "MIXED_SPLIT_MIN", 2)          # the product splits from 12 decoding requests on
    vocab = TINY[name][0]["vocab_size"]
    eng = engine(name, "bfloat16", prefill_chunk=80, max_batch_tokens=96, page_size=64, num_pages=40)
    short = [random_tokens(vocab, n, 300 + n) for n in (3, 9, 14, 6, 11)]
    reqs = [eng.scheduler.add_request(p, SamplingParams(max_new_tokens=14)) for p in short]
    for _ in range(3):
        eng.scheduler.step()
    long_prompt = random_tokens(vocab, 230, 77)
    reqs.append(eng.scheduler.add_request(long_prompt, SamplingParams(max_new_tokens=5)))
    eng.scheduler.run_to_completion()
    eng.runner.check_errors()
    for p, r in zip(short + [long_prompt], reqs):
        assert len(r.generated_tokens) == r.params.max_new_tokens
        near_greedy(name, p, r.generated_tokens, 0.03)


@pytest.mark.parametrize("graph,pipelined", [(False, False), (True, False), (False, True), (True, True)])
def test_eos_ends_requests_at_different_times(graph, pipelined):
    """An end-of-sequence token that some requests produce early, some late and some never:
    every request ends where the plain model's does (the token itself is kept), with and without
    decode graphs and pipelined decoding (where a request's next token is already in flight when
    its end is seen, and is dropped)."""
    from prism_b200 import Engine, EngineConfig, SamplingParams, SchedulerConfig
    cfg, t = plain_model("A")
    prompts = [random_tokens(256, n, 500 + n) for n in (5, 9, 14, 6, 11, 20, 3)]
    full = [P.generate(cfg, t, p, 24) for p in prompts]
    counts = {}
    for g in full:
        for tok in set(g[2:]):
            counts[tok] = counts.get(tok, 0) + 1
    eos = max(counts, key=lambda k: (counts[k], -k))          # the token most requests meet somewhere
    want = [g[:g.index(eos) + 1] if eos in g else g for g in full]
    ec = EngineConfig(kv_page_size=16, num_pages=64, use_cuda_graph=graph, graph_batch_sizes=(1, 2, 4, 8),
                      scheduler=SchedulerConfig(async_decode=pipelined))
    eng = Engine(model_folder("A"), ec, dtype="float32")
    res = eng.generate(prompts, SamplingParams(max_new_tokens=24, eos_token_id=eos))
    assert [r.token_ids for r in res] == want
    assert [r.finish_reason for r in res] == ["stop" if eos in g else "length" for g in full]
    assert eng.runner.cache.pages_in_use() == 0


def test_bad_token_id_is_reported_not_faulted():
    from prism_b200 import SamplingParams
    from prism_b200.engine.runner import DeviceError
    eng = engine("A", "float32")
    with pytest.raises(DeviceError, match="token id"):
        eng.generate([[1, 2, 999]], SamplingParams(max_new_tokens=2))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON steps on standard input, <step>.f32
    files out, `done <step>` after each step; pool sized by --max-tokens so that
    pages are used again."""
    name = "B"
    seqs = {f"q{i}": random_tokens(320, n, 300 + i) for i, n in enumerate([70, 33, 90, 12, 64])}
    steps = trace_mixed(seqs, seed=11)
    budget = trace_budget(steps, 64)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folder(name),
                           "--dtype", dtype, "--out", str(out), "--max-tokens", str(budget), "--page-size", "16"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, fed = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n_want, 320)
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[(e["id"], fed.get(e["id"], 0) + w)] = torch.from_numpy(data[r].copy())
                r += 1
            fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
    from test_replay_gpu import TOL
    compare_with_plain(name, seqs, got, **TOL[dtype])
    assert len(got) == sum(len(s) for s in seqs.values())
