"""The engine against the plain implementation for every way of cutting the
work, in float32 and in bfloat16 (GPU)."""

import pytest
import torch

from helpers import (TINY, compare_with_plain, model_folder, random_tokens, run_trace, trace_budget,
                     trace_mixed, trace_portions, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu

# float32: the engine and the plain model differ by the order of float32 additions only.
# bfloat16: activations are rounded to 8 bits of mantissa where they are stored (norm out, qkv, attention
# out, SwiGLU out); weights are the same bf16 values on both sides.  The yardstick is what that rounding alone
# does to the plain model's logits of the same sequence (helpers.plain_rounding_error, about 3e-3 at a logit
# scale of 1): the engine measured 0.76 to 1.38 times that in every configuration and every way of cutting,
# and may be at most twice it.  (A constant bound would have to be ten times looser to hold everywhere.)
TOL = {"float32": dict(atol=2e-5, rtol=1e-5), "bfloat16": dict(rounding_slack=2.0)}
LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 40, 71, 130], "C": [3, 30, 64, 97, 150], "D": [2, 65, 128, 200, 333]}


def make_runner(name, dtype, num_pages, page_size=None, max_seqs=8, graphs=False):
    from prism_b200.weights.loader import load_model_folder
    from prism_b200.engine.runner import ModelRunner
    tdt = getattr(torch, dtype)
    cfg, model, pool = load_model_folder(model_folder(name), "cuda:0", tdt)
    ps = page_size or TINY[name][2]
    runner = ModelRunner(model, "cuda:0", tdt, ps, num_pages, max_seqs, use_cuda_graph=graphs, graph_batch_sizes=(1, 2, 4))
    runner._pool = pool
    return runner


def sequences(name):
    vocab = TINY[name][0]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, 100 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cutting(name, dtype, mode):
    seqs = sequences(name)
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions,
             "mixed": lambda s: trace_mixed(s, seed=7)}[mode](seqs)
    ps = TINY[name][2]
    budget = trace_budget(steps, ps)
    runner = make_runner(name, dtype, num_pages=budget // ps)
    got = run_trace(runner, steps)
    assert len(got) == sum(len(s) for s in seqs.values())
    compare_with_plain(name, seqs, got, **TOL[dtype])
    assert runner.cache.pages_in_use() == 0


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cutting_with_64_token_pages(mode, monkeypatch):
    """Head size 64 with pages of 64 tokens: portions of 64 tokens and more run on the
    tcgen05 attention kernel, shorter ones on the mma.sync kernel, and in mixed steps the
    decoding requests at the head of the batch go to the decode kernel."""
    from prism_b200 import ops
    monkeypatch.setattr(ops, "MIXED_SPLIT_MIN", 2)
    name, dtype, ps = "D", "bfloat16", 64
    seqs = sequences(name)
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions,
             "mixed": lambda s: trace_mixed(s, seed=11)}[mode](seqs)
    budget = trace_budget(steps, ps)
    runner = make_runner(name, dtype, num_pages=budget // ps, page_size=ps)
    got = run_trace(runner, steps)
    assert len(got) == sum(len(s) for s in seqs.values())
    compare_with_plain(name, seqs, got, **TOL[dtype])
    assert runner.cache.pages_in_use() == 0


@pytest.mark.parametrize("name,dtype,ps", [("D", "bfloat16", 64), ("C", "bfloat16", 16), ("B", "float32", 8)])
def test_replay_is_reproducible(name, dtype, ps):
    """The same trace on the same runner (pages recycled in between) gives bitwise the same logits."""
    seqs = sequences(name)
    steps = trace_mixed(seqs, seed=13)
    runner = make_runner(name, dtype, num_pages=trace_budget(steps, ps) // ps, page_size=ps)
    ref = run_trace(runner, steps)
    for _ in range(3):
        got = run_trace(runner, steps)
        assert all(torch.equal(got[k], ref[k]) for k in ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["tail", "mixed"])
def test_cutting_with_decode_graphs(name, dtype, mode):
    """The same with pure-decode steps replayed from captured CUDA graphs (buckets 1, 2, 4 with
    padded rows): inside a graph the kernels overlap, which launches from Python never do."""
    seqs = sequences(name)
    steps = {"tail": trace_tail, "mixed": lambda s: trace_mixed(s, seed=7)}[mode](seqs)
    ps = TINY[name][2]
    runner = make_runner(name, dtype, num_pages=trace_budget(steps, ps) // ps, graphs=True)
    got = run_trace(runner, steps)
    compare_with_plain(name, seqs, got, **TOL[dtype])
    assert runner.cache.pages_in_use() == 0 and runner.graph_kernel_launches > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_cutting_behind_a_backlog(name, dtype):
    """Mixed steps launched into a busy GPU: the step's kernels wait in the queue and then run
    back to back, so that programmatic dependent launch really overlaps them."""
    seqs = sequences(name)
    steps = trace_mixed(seqs, seed=7)
    ps = TINY[name][2]
    runner = make_runner(name, dtype, num_pages=trace_budget(steps, ps) // ps)
    big = torch.randn(4096, 4096, device="cuda:0")

    def busy():
        for _ in range(3):
            torch.mm(big, big)
    got = run_trace(runner, steps, before_step=busy)
    compare_with_plain(name, seqs, got, **TOL[dtype])


@pytest.mark.parametrize("which", ["all", "norms"])
def test_tensors_stored_in_float32_under_the_bf16_engine(which, tmp_path):
    """A model file whose tensors (all of them, or only the norms' weights and the biases) are stored
    in float32: the bf16 engine keeps those in float32 and still gives the plain model's logits,
    mixed steps and reused pages included."""
    from safetensors.torch import load_file, save_file
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.weights.loader import load_model_folder
    from prism_b200.weights.random_init import write_model_folder
    from helpers import P
    name = "D"
    cfg, seed, ps = TINY[name]
    d = str(tmp_path / "m")
    write_model_folder(cfg, seed, d, store_dtype=torch.float32)
    if which == "norms":
        t = load_file(d + "/model.safetensors")
        t = {k: (v if (v.dim() == 1) else v.to(torch.bfloat16)) for k, v in t.items()}
        assert any(v.dtype == torch.float32 for v in t.values()) and any(v.dtype == torch.bfloat16 for v in t.values())
        save_file(t, d + "/model.safetensors")
    pcfg, pt = P.load_folder(d)
    seqs = sequences(name)
    steps = trace_mixed(seqs, seed=5)
    _, model, pool = load_model_folder(d, "cuda:0", torch.bfloat16)
    kept = {p.dtype for p in pool.tensors.values() if p is not None}
    assert torch.float32 in kept and (which == "all" or torch.bfloat16 in kept)
    runner = ModelRunner(model, "cuda:0", torch.bfloat16, ps, trace_budget(steps, ps) // ps, 8)
    got = run_trace(runner, steps)
    for rid, seq in seqs.items():
        ref = P.forward(pcfg, pt, list(seq))
        # twice what rounding the stored activations to bfloat16 does to this model's own logits
        bound = TOL["bfloat16"]["rounding_slack"] * float(
            (P.forward(pcfg, pt, list(seq), store=lambda v: v.bfloat16().float()) - ref).abs().max())
        for pos in range(len(seq)):
            err = float((got[(rid, pos)] - ref[pos]).abs().max())
            assert err <= bound, (rid, pos, err, bound)
    assert len(got) == sum(len(s) for s in seqs.values())
