"""Layers of Qwen2.5-7B size (hidden 3584, 28/4 heads of 128, intermediate
18944) and of Qwen2.5-0.5B size (hidden 896, 14/2 heads of 64, intermediate 4864,
tied head), two of each, with a reduced vocabulary so that the plain model can run
on the CPU: the production kernels (tensor-core attention, the tcgen05 GEMM
with its fused epilogues, the library GEMM for long portions) at the sizes
they were written for, in float32 and bfloat16, whole and cut (GPU)."""

import json
import os
import tempfile

import pytest
import torch

from helpers import P, random_tokens, run_trace, trace_budget, trace_mixed, trace_tail, trace_whole

pytestmark = pytest.mark.gpu

SHAPE_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=3584,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
                vocab_size=8192, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=32768, use_sliding_window=False)


SHAPE_05B = dict(SHAPE_7B, hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                 intermediate_size=4864, tie_word_embeddings=True)


# the upper layer sees a window of 100 positions (and lands in a cache group of its own)
SHAPE_7B_WINDOW = dict(SHAPE_7B, use_sliding_window=True, sliding_window=100, max_window_layers=1)


@pytest.fixture(scope="module", params=["7B", "0.5B", "7B-window"])
def folder_and_plain(request):
    from prism_b200.weights.random_init import write_model_folder
    with tempfile.TemporaryDirectory(prefix="prism_7b_shape_") as d:
        write_model_folder({"7B": SHAPE_7B, "0.5B": SHAPE_05B, "7B-window": SHAPE_7B_WINDOW}[request.param], 3, d)
        cfg, t = P.load_folder(d)
        seqs = {"a": random_tokens(8192, 150, 1), "b": random_tokens(8192, 41, 2), "c": random_tokens(8192, 77, 3)}
        ref = {k: P.forward(cfg, t, v) for k, v in seqs.items()}
        yield d, seqs, RefLogits(cfg, t, seqs, ref)


class RefLogits(dict):
    """The plain model's float32 logits per sequence, and the bound for the engine's bfloat16 path: twice what
    rounding the stored activations to bfloat16 does to the plain model's own logits of that sequence
    (``P.forward(..., store=round to bf16)``), which is the error the engine's rounding must produce as well."""

    def __init__(self, cfg, t, seqs, ref):
        super().__init__(ref)
        self.cfg, self.t, self.bound16 = cfg, t, {}
        for k, v in seqs.items():
            self.add(k, v, ref[k])

    def add(self, k, seq, ref):
        self[k] = ref
        r16 = P.forward(self.cfg, self.t, seq, store=lambda v: v.bfloat16().float()).to(ref.device)
        self.bound16[k] = BF16_SLACK * float((r16 - ref).abs().max())


BF16_SLACK = 2.0


def runner_for(folder, dtype, num_pages, page_size=64, graphs=False, max_seqs=8):
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.weights.loader import load_model_folder
    tdt = getattr(torch, dtype)
    _, model, pool = load_model_folder(folder, "cuda:0", tdt)
    r = ModelRunner(model, "cuda:0", tdt, page_size, num_pages, max_seqs, max_seq_len=512, use_cuda_graph=graphs,
                    graph_batch_sizes=(1, 4))
    r._pool = pool
    return r


@pytest.mark.parametrize("dtype,atol,rtol", [("float32", 1e-3, 1e-4), ("bfloat16", None, None)])
@pytest.mark.parametrize("mode", ["whole", "tail", "tail_graphs", "mixed", "mixed_graphs", "whole_backlog", "mixed_backlog"])
def test_7b_sized_layers(folder_and_plain, dtype, atol, rtol, mode):
    """``*_graphs``: pure-decode steps are replayed from captured CUDA graphs, where the kernels
    really overlap (programmatic dependent launch); ``*_backlog``: a few milliseconds of other work are
    queued before every step, so that the step's kernels wait in the queue and then run back to back,
    overlapping as well; the other modes launch kernel by kernel into an idle GPU."""
    folder, seqs, ref = folder_and_plain
    kind = mode.split("_")[0]
    steps = {"whole": trace_whole, "tail": lambda s: trace_tail(s, 12), "mixed": lambda s: trace_mixed(s, seed=5)}[kind](seqs)
    runner = runner_for(folder, dtype, trace_budget(steps, 64) // 64, graphs=mode.endswith("_graphs"))
    busy = None
    if mode.endswith("_backlog"):
        big = torch.randn(8192, 8192, device="cuda:0", dtype=torch.bfloat16)

        def busy():
            for _ in range(4):
                torch.mm(big, big)
    got = run_trace(runner, steps, before_step=busy)
    worst = 0.0
    for rid, seq in seqs.items():
        scale = float(ref[rid].abs().max())
        for pos in range(len(seq)):
            err = float((got[(rid, pos)] - ref[rid][pos]).abs().max())
            worst = max(worst, err)
            assert err <= (ref.bound16[rid] if atol is None else atol + rtol * scale), (rid, pos, err, scale, ref.bound16[rid])
    assert runner.cache.pages_in_use() == 0


@pytest.mark.parametrize("graphs", [False, True])
def test_7b_sized_layers_with_pages_of_256(folder_and_plain, graphs):
    """The benchmark's page size: a whole sequence, then its last tokens one by one."""
    folder, seqs, ref = folder_and_plain
    steps = trace_tail(seqs, 10)
    runner = runner_for(folder, "bfloat16", trace_budget(steps, 256) // 256, page_size=256, graphs=graphs)
    got = run_trace(runner, steps)
    for rid, seq in seqs.items():
        scale = float(ref[rid].abs().max())
        for pos in range(len(seq)):
            err = float((got[(rid, pos)] - ref[rid][pos]).abs().max())
            assert err <= ref.bound16[rid], (rid, pos, err, scale, ref.bound16[rid])
    assert runner.cache.pages_in_use() == 0


@pytest.mark.parametrize("mode", ["tail", "tail_graphs", "mixed_graphs"])
def test_7b_sized_layers_with_the_projection_finished_inside_decode_attention(folder_and_plain, mode, monkeypatch):
    """The optional decode path without a kernel between the qkv projection and attention
    (``ops.QKV_IN_ATTENTION``): the decode kernel adds the projection's partial sums, rotates, and
    stores each token's key and value itself."""
    from prism_b200 import ops
    monkeypatch.setattr(ops, "QKV_IN_ATTENTION", True)
    launches = []
    real = ops.attention_decode_qkv_bf16
    monkeypatch.setattr(ops, "attention_decode_qkv_bf16", lambda *a, **k: (launches.append(1), real(*a, **k))[1])
    folder, seqs, ref = folder_and_plain
    kind = mode.split("_")[0]
    steps = {"tail": lambda s: trace_tail(s, 12), "mixed": lambda s: trace_mixed(s, seed=5)}[kind](seqs)
    runner = runner_for(folder, "bfloat16", trace_budget(steps, 64) // 64, graphs=mode.endswith("_graphs"))
    got = run_trace(runner, steps)
    cfg = json.load(open(os.path.join(folder, "config.json")))
    qkv_rows = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    if ops.tc_ksplit(qkv_rows, cfg["hidden_size"]) > 1:          # a projection that is not K-split keeps the usual path
        assert launches, "the fused path did not run"
    for rid, seq in seqs.items():
        scale = float(ref[rid].abs().max())
        for pos in range(len(seq)):
            err = float((got[(rid, pos)] - ref[rid][pos]).abs().max())
            assert err <= ref.bound16[rid], (rid, pos, err, scale, ref.bound16[rid])
    assert runner.cache.pages_in_use() == 0


def test_thirteen_decoding_requests_beside_a_prompt_portion(folder_and_plain, monkeypatch):
    """A mixed step as the scheduler builds it under load: thirteen requests each feed one decoded token
    and a fourteenth a portion of its prompt.  From twelve single tokens at the head of the batch on
    (``ops.MIXED_SPLIT_MIN``, at its default here) those go to the decode attention kernel and only the
    portion to the prefill kernel - in one step, over one block table.  Every logit row against the plain model."""
    from prism_b200 import ops
    folder, _, _ = folder_and_plain
    assert ops.MIXED_SPLIT_MIN == 12
    calls = []
    real = ops.attention_decode_bf16
    monkeypatch.setattr(ops, "attention_decode_bf16", lambda q, *a, **k: (calls.append(q.shape[0]), real(q, *a, **k))[1])
    cfg, t = P.load_folder(folder, device="cuda:0")
    seqs = {f"d{i}": random_tokens(8192, 21 + 3 * i, 400 + i) for i in range(13)}
    seqs["long"] = random_tokens(8192, 230, 77)
    with torch.no_grad():
        ref = RefLogits(cfg, t, seqs, {k: P.forward(cfg, t, v) for k, v in seqs.items()})
        for k in seqs:
            ref[k] = ref[k].cpu()
    steps, n = [], 0
    for rid in list(seqs)[:13]:                          # the short ones whole but for their last six tokens
        head = len(seqs[rid]) - 6
        steps.append(dict(step=n, entries=[dict(id=rid, tokens=seqs[rid][:head], want=list(range(head)))], end=[]))
        n += 1
    at = 0
    for j in range(6):                                   # six steps: thirteen single tokens + a portion of the long prompt
        entries = [dict(id=rid, tokens=[seqs[rid][len(seqs[rid]) - 6 + j]], want=[0]) for rid in list(seqs)[:13]]
        m = (70, 2, 64, 33, 59, 2)[j]
        entries.append(dict(id="long", tokens=seqs["long"][at:at + m], want=list(range(m))))
        at += m
        steps.append(dict(step=n, entries=entries, end=list(seqs) if j == 5 else []))
        n += 1
    assert at == 230
    runner = runner_for(folder, "bfloat16", trace_budget(steps, 64) // 64, max_seqs=14)
    got = run_trace(runner, steps)
    assert calls.count(13) >= 6 * 2, calls               # every mixed step, every layer: thirteen tokens on the decode kernel
    for rid, seq in seqs.items():
        scale = float(ref[rid].abs().max())
        for pos in range(len(seq)):
            err = float((got[(rid, pos)] - ref[rid][pos]).abs().max())
            assert err <= ref.bound16[rid], (rid, pos, err, scale, ref.bound16[rid])


@pytest.mark.parametrize("graphs", [False, True])
def test_requests_of_unequal_length_decode_together(folder_and_plain, graphs, monkeypatch):
    """Four requests of 1,500, 40, 600 and 130 tokens decode their last tokens in the same steps.  The step's
    descriptor carries the decode kernel's work items: the long request is shared among several CTAs per kv head,
    the short ones take one each.  Every logit row against the plain model."""
    from prism_b200 import ops
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.weights.loader import load_model_folder
    folder, _, _ = folder_and_plain
    seen = []
    real = ops.attention_decode_bf16

    def spy(q, out, k, v, bt, pos, seg, npg, window, scale, nsplit, po, pml, err, items=None, starts=None):
        seen.append((q.shape[0], window, nsplit, None if items is None else items.shape[0],
                     None if starts is None or graphs else starts.tolist()))
        return real(q, out, k, v, bt, pos, seg, npg, window, scale, nsplit, po, pml, err, items=items, starts=starts)
    monkeypatch.setattr(ops, "attention_decode_bf16", spy)
    cfg, t = P.load_folder(folder, device="cuda:0")
    seqs = {"long": random_tokens(8192, 1500, 31), "tiny": random_tokens(8192, 40, 32),
            "mid": random_tokens(8192, 600, 33), "short": random_tokens(8192, 130, 34)}
    with torch.no_grad():
        ref = RefLogits(cfg, t, seqs, {k: P.forward(cfg, t, v) for k, v in seqs.items()})
        for k in seqs:
            ref[k] = ref[k].cpu()
    tail, steps = 6, []
    for rid, seq in seqs.items():
        steps.append(dict(step=len(steps), entries=[dict(id=rid, tokens=seq[:-tail], want=[len(seq) - tail - 1])], end=[]))
    for j in range(tail):
        steps.append(dict(step=len(steps), end=list(seqs) if j == tail - 1 else [],
                          entries=[dict(id=rid, tokens=[seq[len(seq) - tail + j]], want=[0]) for rid, seq in seqs.items()]))
    _, model, pool = load_model_folder(folder, "cuda:0", torch.bfloat16)
    runner = ModelRunner(model, "cuda:0", torch.bfloat16, 64, trace_budget(steps, 64) // 64, 4, max_seq_len=2048,
                         use_cuda_graph=graphs, graph_batch_sizes=(1, 4))
    got = run_trace(runner, steps)
    full = [s for s in seen if s[0] == 4 and s[1] is None]       # the layers that keep every key
    assert full and all(n is not None for _, _, _, n, _ in full), full[:4]
    if graphs:
        nkv = json.load(open(os.path.join(folder, "config.json")))["num_key_value_heads"]
        assert all(n == 2 * ops.num_sms() // nkv for _, _, _, n, _ in full)   # one wave of places per kv head
    else:
        # 1,494 + 34 + 594 + 124 keys: 24, 1, 10 and 2 tiles, at three tiles a CTA at least
        for _, _, ns, n, st in full[:2]:
            assert ns == 8 and n == 13 and [v >> 16 for v in st] == [8, 1, 3, 1], full[:2]
            assert sorted(v & 0xffff for v in st) == [0, 3, 11, 12]          # the longest CTAs (4 tiles each) first
    for rid, seq in seqs.items():
        for pos in range(len(seq) - tail - 1, len(seq)):
            err = float((got[(rid, pos)] - ref[rid][pos]).abs().max())
            assert err <= ref.bound16[rid], (rid, pos, err, ref.bound16[rid])
    assert runner.cache.pages_in_use() == 0


def test_generation_with_prompts_prefilled_in_portions(folder_and_plain):
    """``Engine.generate`` with ``prefill_chunk`` shorter than the prompts and a token budget that makes
    portions share steps with decoding requests, at these layer sizes, CUDA graphs and pipelined decoding on:
    every generated token is the plain model's best one for the same history (up to a near-tie)."""
    from prism_b200 import Engine, EngineConfig, SamplingParams, SchedulerConfig
    folder, _, _ = folder_and_plain
    cfg, t = P.load_folder(folder, device="cuda:0")
    ec = EngineConfig(kv_page_size=64, num_pages=24, max_seq_len=512, use_cuda_graph=True, graph_batch_sizes=(1, 2, 4),
                      scheduler=SchedulerConfig(max_batch_tokens=96, max_num_seqs=4, prefill_chunk=80))
    eng = Engine(folder, ec, dtype="bfloat16")
    prompts = [random_tokens(8192, n, 500 + n) for n in (200, 33, 150, 7, 90)]
    res = eng.generate(prompts, [SamplingParams(max_new_tokens=n) for n in (6, 14, 9, 20, 5)])
    assert eng.stats.prefill_tokens >= sum(len(p) for p in prompts) and eng.runner.graph_kernel_launches > 0
    assert eng.cache.pages_in_use() == 0
    with torch.no_grad():
        for p, r in zip(prompts, res):
            assert r.finish_reason == "length"
            lg = P.forward(cfg, t, list(p) + list(r.token_ids))            # one pass: row i predicts token i + 1
            for i, tok in enumerate(r.token_ids):
                row = lg[len(p) - 1 + i]
                assert float(row.max() - row[tok]) <= 0.03 * float(row.abs().max()), (len(p), i, tok)


def test_a_step_gives_the_same_bits_every_time():
    """The same prompt, prefilled again and again from recycled pages, gives bitwise the same
    logits.  A race shows here as a rare different result: a wait on a barrier whose phases are told
    apart by one parity bit once passed two phases early in the tcgen05 attention kernel when the
    neighbouring CTA kept the tensor pipe busy - about one step in ten, with four full-size layers and
    the full vocabulary (random weights made on the device; no plain model is needed for this)."""
    from prism_b200 import Engine, EngineConfig
    from prism_b200.engine.batch import Segment
    cfg = dict(SHAPE_7B, num_hidden_layers=4, vocab_size=152064)
    eng = Engine(None, EngineConfig(kv_page_size=64, num_pages=300, max_seq_len=4096, use_cuda_graph=False),
                 dtype="bfloat16", config=cfg, random_seed=0)
    runner = eng.runner
    prompt = random_tokens(150000, 200, 9)

    def once():
        runner.begin_request("r")
        a = runner.step([Segment("r", prompt, [199])]).clone()
        runner.end_request("r")
        return a

    ref = once()
    differ = [i for i in range(80) if not torch.equal(once(), ref)]
    runner.check_errors()
    assert not differ, differ


FAMILY_SHAPES = {
    "0.5B": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64, intermediate_size=4864,
                 vocab_size=151936, tie_word_embeddings=True),
    "32B": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=27648,
                vocab_size=152064, tie_word_embeddings=False),
}


@pytest.mark.parametrize("size", ["0.5B", "32B"])
def test_decode_graph_replay_gives_the_eager_logits(size):
    """Decode steps replayed from a captured graph against the same steps launched one kernel at a
    time, at the layer sizes of Qwen2.5-0.5B (14/2 heads of 64) and 32B (40/8 heads of 128), two
    layers each.  In a graph the kernels really
    overlap (programmatic dependent launch), and there decode attention once read q before the kernel
    that writes it had finished: the compiler had hoisted loads through a `const __restrict__`
    parameter above the dependency wait.  The logits were off by more than half their range."""
    from prism_b200 import Engine, EngineConfig
    from prism_b200.engine.batch import Segment
    cfg = dict(SHAPE_7B, **FAMILY_SHAPES[size])
    lens = (300, 17, 700, 64, 1)
    prompts = [random_tokens(150000, n, 20 + n) for n in lens]
    logits = {}
    for graph in (False, True):
        eng = Engine(None, EngineConfig(kv_page_size=256, num_pages=16, max_seq_len=4096, use_cuda_graph=graph,
                                        graph_batch_sizes=(16,)), dtype="bfloat16", config=cfg, random_seed=0)
        r = eng.runner
        for i, p in enumerate(prompts):
            r.begin_request(i)
            r.step([Segment(i, p, [])])
        logits[graph] = [r.step([Segment(i, [11 + s + i], [0]) for i in range(len(lens))]).float().cpu() for s in range(3)]
        r.check_errors()
        del eng, r
    for a, b in zip(logits[False], logits[True]):
        # the two differ by rounding only (the graph splits the keys over a different number of CTAs)
        assert float((a - b).abs().max()) <= 0.03 * float(a.abs().max()), float((a - b).abs().max())


def test_long_prompt_on_the_fast_kernels_against_the_generic_attention(monkeypatch):
    """6,000 tokens (too long for the plain model on the CPU): the tcgen05 prefill attention and the
    split-KV decode attention against the shape-generic kernel, which shares no code with them, whole,
    in portions of 1,024, and with a tail of short portions behind a long cache (whose key tiles several
    CTAs share, with a merge after them), followed by a few decode steps through graphs."""
    from prism_b200 import Engine, EngineConfig, ops
    from prism_b200.engine.batch import Segment
    cfg = dict(SHAPE_7B, vocab_size=152064)
    prompt = random_tokens(150000, 6000, 4)
    logits = {}
    calls = {"decode_tokens": [], "prefill_splits": []}
    real_decode, real_tc = ops.attention_decode_bf16, ops.attention_prefill_tc
    monkeypatch.setattr(ops, "attention_decode_bf16",
                        lambda q, *a, **k: (calls["decode_tokens"].append(q.shape[0]), real_decode(q, *a, **k))[1])
    monkeypatch.setattr(ops, "attention_prefill_tc",
                        lambda *a, **k: (calls["prefill_splits"].append(k.get("nsplit", 1)), real_tc(*a, **k))[1])
    for mode in ("fast", "generic", "portions", "short_portions", "tail_and_mixed"):
        monkeypatch.setattr(ops, "FORCE_GENERIC_ATTENTION", mode == "generic")
        eng = Engine(None, EngineConfig(kv_page_size=256, num_pages=32, max_seq_len=8192, use_cuda_graph=mode != "generic"),
                     dtype="bfloat16", config=cfg, random_seed=0)
        r = eng.runner
        r.begin_request(0)
        if mode == "portions":
            for c in range(0, 6000, 1024):
                part = prompt[c:c + 1024]
                lg = r.step([Segment(0, part, [len(part) - 1])])
        elif mode == "short_portions":
            assert ops.prefill_splits(1, 152, cfg["num_attention_heads"], 4936 + 152, None) > 1
            r.step([Segment(0, prompt[:4936], [])])
            for c in range(4936, 6000, 152):
                lg = r.step([Segment(0, prompt[c:c + 152], [151])])
        elif mode == "tail_and_mixed":
            # the prompt's last 32 tokens as a portion of their own: short, but behind 5,968 keys, so the
            # tcgen05 kernel with shared keys takes it; then the first decoded token beside another request's
            # prompt portion: one decoding request only, but a long one, so it goes to the decode kernel
            r.step([Segment(0, prompt[:5968], [])])
            calls["prefill_splits"].clear()
            lg = r.step([Segment(0, prompt[5968:], [31])])
            assert calls["prefill_splits"] and min(calls["prefill_splits"]) > 1, calls
            r.begin_request(1)
            calls["decode_tokens"].clear()
            first = r.step([Segment(0, [100], [0]), Segment(1, prompt[:100], [])])
            assert calls["decode_tokens"] and set(calls["decode_tokens"]) == {1}, calls
            outs = [lg.float().cpu(), first.float().cpu()]
            outs += [r.step([Segment(0, [100 + s], [0])]).float().cpu() for s in range(1, 4)]
            r.check_errors()
            logits[mode] = outs
            del eng, r
            continue
        else:
            lg = r.step([Segment(0, prompt, [5999])])
        outs = [lg.float().cpu()] + [r.step([Segment(0, [100 + s], [0])]).float().cpu() for s in range(4)]
        r.check_errors()
        logits[mode] = outs
        del eng, r
    scale = float(logits["fast"][0].abs().max())
    for mode in ("generic", "portions", "short_portions", "tail_and_mixed"):
        for a, b in zip(logits["fast"], logits[mode]):
            assert float((a - b).abs().max()) <= 0.03 * scale, (mode, float((a - b).abs().max()), scale)
