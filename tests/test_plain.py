"""The plain implementation itself (CPU): against the recorded outputs of
andre-fu/prism's own executor (tests/golden), and the properties each of its
parts must have."""

import os

import pytest
import torch
from safetensors.torch import load_file

from helpers import HERE, P, TINY, plain_logits, plain_model, random_tokens

GOLDEN = os.path.join(HERE, "golden", "prefill_reference.safetensors")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_executor(name):
    """Same weights, same tokens, the executor's own (bf16-rounded) cos/sin:
    the plain forward and FlashAttnExecutorV3.prefill agree to float32 rounding,
    at the last position, at earlier positions, and for a prompt fed in two
    portions."""
    g = load_file(GOLDEN)
    cfg, t = plain_model(name)
    tokens = g[f"{name}.tokens"].tolist()
    assert tokens == random_tokens(TINY[name][0]["vocab_size"], len(tokens), 50)
    ours = P.forward(cfg, t, tokens, cos_sin=(g[f"{name}.cos"], g[f"{name}.sin"]))
    n = len(tokens)
    assert float((ours[-1] - g[f"{name}.last_logits"]).abs().max()) < 2e-6
    assert float((ours[-1] - g[f"{name}.last_logits_two_portions"]).abs().max()) < 2e-6
    rows = torch.stack([ours[0], ours[1], ours[n // 2 - 1]])
    assert float((rows - g[f"{name}.logits_at_1_2_half"]).abs().max()) < 2e-6
    # with float32 tables (what the engine computes) the difference is the table rounding only
    exact = P.forward(cfg, t, tokens)
    assert float((exact[-1] - g[f"{name}.last_logits"]).abs().max()) < 5e-4


def test_rms_norm():
    x = torch.randn(5, 96)
    w = torch.randn(96)
    y = P.rms_norm(x, w, 1e-5)
    assert torch.allclose(y, x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w, atol=1e-6)
    assert torch.allclose(P.rms_norm(3 * x, w, 0.0), P.rms_norm(x, w, 0.0), atol=1e-5)   # scale-free without eps


def test_rope_is_a_rotation_by_relative_position():
    hd = 32
    q, k = torch.randn(1, 1, hd), torch.randn(1, 1, hd)
    def score(pq, pk):
        cq, sq = P.rope_cos_sin(torch.tensor([pq]), hd, 1e4)
        ck, sk = P.rope_cos_sin(torch.tensor([pk]), hd, 1e4)
        return float((P.apply_rope(q, cq, sq) * P.apply_rope(k, ck, sk)).sum())
    assert abs(score(10, 3) - score(107, 100)) < 1e-4          # depends on the distance only
    c0, s0 = P.rope_cos_sin(torch.tensor([0]), hd, 1e4)
    assert torch.allclose(P.apply_rope(q, c0, s0), q)           # position 0: identity
    c, s = P.rope_cos_sin(torch.tensor([77]), hd, 1e6)
    assert abs(float(P.apply_rope(q, c, s).norm()) - float(q.norm())) < 1e-5


def test_attention_is_causal_grouped_and_windowed():
    T, nh, nkv, hd = 12, 4, 2, 8
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    o = P.attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[7:], v2[7:] = 9.0, -9.0                                   # the future does not reach the past
    assert torch.allclose(P.attention(q, k2, v2)[:7], o[:7])
    assert torch.allclose(o[0], v[0].repeat_interleave(2, dim=0))   # one key: its value; heads 0,1 -> kv head 0
    ow = P.attention(q, k, v, window=3)
    assert torch.allclose(ow[:3], o[:3], atol=1e-6) and not torch.allclose(ow[5], o[5])
    k3 = k.clone()
    k3[2] = 50.0                                                  # outside the window of position 5 .. 11
    assert torch.allclose(P.attention(q, k3, v, window=3)[5:], ow[5:])


def test_swiglu_and_sampling():
    g, u = torch.tensor([0.0, 1.0, -2.0]), torch.tensor([3.0, 2.0, 1.0])
    assert torch.allclose(P.swiglu(g, u), g * torch.sigmoid(g) * u)
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert P.sample(logits, 0.0, 0.3) == 1                       # ties: the lowest index
    p = torch.softmax(logits / 0.7, -1)
    c = torch.cumsum(p, -1)
    for u_ in (0.0, 0.2, 0.5, 0.9, 0.9999):
        tok = P.sample(logits, 0.7, u_)
        assert (c[tok - 1] if tok else 0.0) <= u_ < c[tok] + 1e-6


@pytest.mark.parametrize("name", ["A", "C"])
def test_prefix_of_a_sequence_has_the_same_logits(name):
    """No cache in the plain model, but causality makes a prefix's logits equal
    the longer sequence's at the same positions - the identity every cached run
    of the engine is later held to."""
    vocab = TINY[name][0]["vocab_size"]
    seq = random_tokens(vocab, 40, 3)
    full = plain_logits(name, seq)
    assert torch.allclose(plain_logits(name, seq[:17]), full[:17], atol=1e-5)
    cfg, t = plain_model(name)
    gen = P.generate(cfg, t, seq[:9], 4)
    assert gen[0] == int(plain_logits(name, seq[:9])[-1].argmax()) and len(gen) == 4
