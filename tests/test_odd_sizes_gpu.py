"""Configurations whose sizes fit no kernel's favourite shape - widths that are no multiple of 8, an odd
vocabulary, head sizes 80, 112 and 256, 17 query heads on one kv head, a feed-forward of 17 - through the
runner in float32 and bfloat16, cut into portions and mixed, against the plain model (GPU).  Every size the
configuration allows is taken (by the fast kernels or by the generic ones) and gives the right logits."""

import tempfile
import warnings

import pytest
import torch

from helpers import P, random_tokens, round_bf16, run_trace, trace_budget, trace_mixed, trace_portions

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", rope_theta=10000.0, rms_norm_eps=1e-6,
            max_position_embeddings=512, use_sliding_window=False)
ODD = {
    "width 68, feed-forward 172, vocabulary 1001": dict(
        num_hidden_layers=2, hidden_size=68, num_attention_heads=2, num_key_value_heads=1, head_dim=32,
        intermediate_size=172, vocab_size=1001, tie_word_embeddings=False),
    "width 70, feed-forward 50, vocabulary 77": dict(
        num_hidden_layers=2, hidden_size=70, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
        intermediate_size=50, vocab_size=77, tie_word_embeddings=True),
    "width 33, feed-forward 17, vocabulary 19": dict(
        num_hidden_layers=1, hidden_size=33, num_attention_heads=1, num_key_value_heads=1, head_dim=16,
        intermediate_size=17, vocab_size=19, tie_word_embeddings=False),
    "head 80": dict(
        num_hidden_layers=1, hidden_size=160, num_attention_heads=2, num_key_value_heads=2, head_dim=80,
        intermediate_size=324, vocab_size=513, tie_word_embeddings=False),
    "head 112, 7 query heads on one kv head": dict(
        num_hidden_layers=2, hidden_size=96, num_attention_heads=7, num_key_value_heads=1, head_dim=112,
        intermediate_size=200, vocab_size=300, tie_word_embeddings=True),
    "head 256 (generic attention)": dict(
        num_hidden_layers=1, hidden_size=128, num_attention_heads=2, num_key_value_heads=1, head_dim=256,
        intermediate_size=136, vocab_size=260, tie_word_embeddings=False),
    "17 query heads on one kv head (generic attention)": dict(
        num_hidden_layers=1, hidden_size=136, num_attention_heads=17, num_key_value_heads=1, head_dim=64,
        intermediate_size=144, vocab_size=260, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", list(ODD))
def test_odd_sizes(name):
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.weights.loader import load_model_folder
    from prism_b200.weights.random_init import write_model_folder
    cfg = dict(BASE, **ODD[name])
    with tempfile.TemporaryDirectory(prefix="prism_odd_") as d:
        write_model_folder(cfg, 1, d)
        pc, pt = P.load_folder(d)
        seqs = {f"r{i}": random_tokens(cfg["vocab_size"], n, 10 + i) for i, n in enumerate((70, 33, 150, 9, 101))}
        ref = {k: P.forward(pc, pt, v) for k, v in seqs.items()}
        rounding = {k: float((P.forward(pc, pt, v, store=round_bf16) - ref[k]).abs().max()) for k, v in seqs.items()}
        for dtype in ("float32", "bfloat16"):
            for page, steps in ((16, trace_mixed(seqs, seed=3)), (64, trace_portions(seqs))):
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore", RuntimeWarning)       # "falls to the generic attention kernel"
                    _, model, pool = load_model_folder(d, "cuda:0", getattr(torch, dtype))
                runner = ModelRunner(model, "cuda:0", getattr(torch, dtype), page, trace_budget(steps, page) // page, 8,
                                     max_seq_len=512)
                got = run_trace(runner, steps)
                for rid, seq in seqs.items():
                    # float32: 2e-5 as everywhere; bfloat16: twice what rounding alone does to the plain model
                    bound = 2e-5 if dtype == "float32" else 2 * rounding[rid]
                    for pos in range(len(seq)):
                        err = float((got[(rid, pos)] - ref[rid][pos]).abs().max())
                        assert err <= bound, (name, dtype, page, rid, pos, err, bound)
                assert runner.cache.pages_in_use() == 0
