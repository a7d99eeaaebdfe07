"""Shared pieces of the tests: tiny configurations, model folders in a
temporary directory, trace builders and the comparison with the plain model."""

from __future__ import annotations

import os
import random
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

from plain import qwen2_plain as P  # noqa: E402

ARCH = ["Qwen2ForCausalLM"]

# Three tiny configurations that differ in every size and option.
TINY_A = dict(architectures=ARCH, model_type="qwen2", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=128, use_sliding_window=False)
TINY_B = dict(architectures=ARCH, model_type="qwen2", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=3, num_key_value_heads=1, intermediate_size=224,
              vocab_size=320, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=256, use_sliding_window=False)
# C: a sliding window on the upper layers, head_dim that is not hidden/heads, no q/k/v bias, odd vocabulary
TINY_C = dict(architectures=ARCH, model_type="qwen2", num_hidden_layers=4, hidden_size=80,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=176,
              vocab_size=389, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
              max_position_embeddings=512, use_sliding_window=True, sliding_window=24,
              max_window_layers=2, attention_bias=False)
# D: head size 64, which the tensor-core attention kernels take in bfloat16; window on every layer but the first
TINY_D = dict(architectures=ARCH, model_type="qwen2", num_hidden_layers=2, hidden_size=136,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=200,
              vocab_size=301, rope_theta=20000.0, rms_norm_eps=2e-6, tie_word_embeddings=True,
              max_position_embeddings=1024, use_sliding_window=True, sliding_window=70, max_window_layers=1)
TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 2, 8), "C": (TINY_C, 5, 16), "D": (TINY_D, 9, 32)}    # config, weight seed, page size

_folders = {}


def model_folder(name: str) -> str:
    """A model folder for a tiny configuration, made once per process in a
    temporary directory with the framework's random-weights mode."""
    if name not in _folders:
        from prism_b200.weights.random_init import write_model_folder
        cfg, seed, _ = TINY[name]
        d = tempfile.mkdtemp(prefix=f"prism_tiny_{name}_")
        write_model_folder(cfg, seed, d)
        _folders[name] = d
    return _folders[name]


_plain_cache = {}


def plain_model(name: str):
    if name not in _plain_cache:
        _plain_cache[name] = P.load_folder(model_folder(name))
    return _plain_cache[name]


def plain_logits(name: str, seq) -> torch.Tensor:
    cfg, t = plain_model(name)
    return P.forward(cfg, t, list(seq))


def round_bf16(v: torch.Tensor) -> torch.Tensor:
    return v.bfloat16().float()


_rounding_cache = {}


def plain_rounding_error(name: str, seq) -> float:
    """What rounding to bfloat16 alone does to a sequence's logits: the largest difference between the plain
    model with its stored activations rounded (``store=round_bf16``, arithmetic still float32) and itself in
    float32.  The yardstick for the engine's bfloat16 path: its distance from the float32 logits is rounding
    of the same kind plus the order of additions, so it may be a small multiple of this and no more."""
    key = (name, tuple(seq))
    if key not in _rounding_cache:
        cfg, t = plain_model(name)
        _rounding_cache[key] = float((P.forward(cfg, t, list(seq), store=round_bf16) - plain_logits(name, seq)).abs().max())
    return _rounding_cache[key]


def random_tokens(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# --------------------------------------------------------------------------
# traces: lists of steps {"step", "entries": [{"id","tokens","want"}], "end"}
# --------------------------------------------------------------------------

def trace_whole(seqs: dict):
    steps = []
    for i, (rid, seq) in enumerate(seqs.items()):
        steps.append(dict(step=i, entries=[dict(id=rid, tokens=list(seq), want=list(range(len(seq))))], end=[rid]))
    return steps


def trace_tail(seqs: dict, tail: int = 32):
    steps, n = [], 0
    for rid, seq in seqs.items():
        head = max(1, len(seq) - tail)
        steps.append(dict(step=n, entries=[dict(id=rid, tokens=list(seq[:head]), want=list(range(head)))], end=[]))
        n += 1
        for j in range(head, len(seq)):
            steps.append(dict(step=n, entries=[dict(id=rid, tokens=[seq[j]], want=[0])],
                              end=[rid] if j == len(seq) - 1 else []))
            n += 1
        if head == len(seq):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(seqs: dict, sizes=(7, 2, 16, 3, 2, 5, 11, 2, 1, 4)):
    steps, n = [], 0
    for rid, seq in seqs.items():
        at, k = 0, 0
        while at < len(seq):
            m = min(sizes[k % len(sizes)], len(seq) - at)
            k += 1
            steps.append(dict(step=n, entries=[dict(id=rid, tokens=list(seq[at:at + m]), want=list(range(m)))],
                              end=[rid] if at + m == len(seq) else []))
            at += m
            n += 1
    return steps


def trace_mixed(seqs: dict, seed: int, max_live: int = 4, decode_tail: int = 12):
    """Up to ``max_live`` live requests; each step every live request either
    sits out, feeds a portion of its prompt (2..17 tokens) or, in its last
    ``decode_tail`` tokens, a single token."""
    rng = random.Random(seed)
    waiting = list(seqs.items())
    live, at, steps, n = [], {}, [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, seq = waiting.pop(0)
            live.append(rid)
            at[rid] = 0
        entries, end = [], []
        for rid in list(live):
            seq = seqs[rid]
            left = len(seq) - at[rid]
            if rng.random() < 0.15 and len(live) > 1:
                continue
            m = 1 if left <= decode_tail else min(left - decode_tail, rng.randint(2, 17))
            entries.append(dict(id=rid, tokens=list(seq[at[rid]:at[rid] + m]), want=list(range(m))))
            at[rid] += m
            if at[rid] == len(seq):
                end.append(rid)
                live.remove(rid)
        if entries:
            steps.append(dict(step=n, entries=entries, end=end))
            n += 1
    return steps


def trace_budget(steps, unit: int) -> int:
    """Most tokens live requests hold at any time, each rounded up to ``unit``."""
    held, best = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        best = max(best, sum((v + unit - 1) // unit * unit for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return best


def run_trace(runner, steps, before_step=None):
    """Drive a ModelRunner through a trace in-process.  Returns
    ``{(request id, position): logits row (float32 CPU tensor)}``.
    ``before_step()`` is called before every step (e.g. to keep the GPU busy)."""
    from prism_b200.engine.batch import Segment
    out, live, fed = {}, set(), {}
    for st in steps:
        segs = []
        for e in st["entries"]:
            if e["id"] not in live:
                runner.begin_request(e["id"])
                live.add(e["id"])
                fed[e["id"]] = 0
            segs.append(Segment(e["id"], e["tokens"], e["want"]))
        if before_step is not None:
            before_step()
        logits = runner.step(segs)
        if logits is not None:
            logits = logits.float().cpu()
        r = 0
        for e in st["entries"]:
            for w in e["want"]:
                out[(e["id"], fed[e["id"]] + w)] = logits[r]
                r += 1
            fed[e["id"]] += len(e["tokens"])
        for rid in st["end"]:
            runner.end_request(rid)
            live.discard(rid)
        runner.check_errors()
        runner.cache.check_invariants()
    return out


def compare_with_plain(name: str, seqs: dict, got: dict, atol: float = 0.0, rtol: float = 0.0,
                       rounding_slack: float = None):
    """Every logits row the trace produced against the plain model on the whole
    sequence.  The bound on a row's largest error: ``atol + rtol * (largest logit of the sequence)``, plus,
    with ``rounding_slack``, that many times what rounding to bfloat16 alone does to the plain model's logits
    of that sequence (``plain_rounding_error``).  Returns the worst absolute error and where it was."""
    worst, where = 0.0, None
    for rid, seq in seqs.items():
        ref = plain_logits(name, seq)
        scale = float(ref.abs().max())
        bound = atol + rtol * scale
        if rounding_slack:
            bound += rounding_slack * plain_rounding_error(name, seq)
        for pos in range(len(seq)):
            if (rid, pos) not in got:
                continue
            err = float((got[(rid, pos)] - ref[pos]).abs().max())
            if err > worst:
                worst, where = err, (rid, pos)
            assert err <= bound, \
                f"request {rid} position {pos}: max abs error {err:.3e} > {bound:.3e} (logit scale {scale:.3f})"
    return worst, where
