"""Makes tests/golden/prefill_reference.safetensors: logits of andre-fu/prism's
own executor (engine/executor.py, FlashAttnExecutorV3.prefill) on tiny random
models, on the CPU in float32.

    python tests/golden/make_golden.py --reference <path of the andre-fu/prism checkout>

The executor imports there without a GPU, but two of the names it calls are
GPU-only and are replaced by CPU stand-ins before it runs:
``flash_attn_with_kvcache`` (append k, v at ``cache_seqlens``; causal,
grouped-query attention over the paged cache with scale hd^-1/2) and the
Triton ``fused_rms_norm``.  So the golden values anchor everything the
executor itself spells out - weight fusion order, q/k/v split offsets, bias,
norm placement, rotary pairing, SwiGLU order, residuals, the tied head, the
``prefix_len`` continuation - and not the attention arithmetic, which is the
stand-in's.  The executor rounds its rotary tables to bf16 (executor.py:53-54);
the tables are widened back to float32 copies of those rounded values, so the
comparison in tests/test_plain.py uses the same rounded cos/sin.

Only its prefill is recorded.  Its decode entry points store the new key one
slot late (executor.py:205-208) and are not a reference for anything.
"""

import argparse
import os
import sys
from types import SimpleNamespace

import torch


def cpu_flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, cache_seqlens=None, block_table=None,
                                causal=True):
    B, Sq, nh, hd = q.shape
    P, nkv = k_cache.shape[1], k_cache.shape[2]
    out = torch.empty_like(q)
    for b in range(B):
        n0 = int(cache_seqlens[b])
        for t in range(Sq):
            slot = n0 + t
            page = int(block_table[b, slot // P])
            k_cache[page, slot % P] = k[b, t]
            v_cache[page, slot % P] = v[b, t]
        idx = torch.arange(n0 + Sq)
        rows = block_table[b][idx // P].long() * P + idx % P
        K = k_cache.reshape(-1, nkv, hd)[rows].float()
        V = v_cache.reshape(-1, nkv, hd)[rows].float()
        g = nh // nkv
        for h in range(nh):
            s = (q[b, :, h].float() @ K[:, h // g].T) * hd ** -0.5
            mask = idx[None, :] <= (n0 + torch.arange(Sq))[:, None]
            s = s.masked_fill(~mask, float("-inf"))
            out[b, :, h] = (torch.softmax(s, -1) @ V[:, h // g]).to(q.dtype)
    return out


def cpu_rms_norm(x, w, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "prefill_reference.safetensors"))
    args = ap.parse_args()

    sys.path.insert(0, args.reference)
    import engine.executor as ex                     # andre-fu/prism's module
    from engine.kv_cache import FlashAttnKVCache
    from engine.weight_pool import StaticWeightPool
    ex.flash_attn_with_kvcache = cpu_flash_attn_with_kvcache
    ex.fused_rms_norm = cpu_rms_norm

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(1, os.path.dirname(here))        # tests/
    sys.path.insert(1, os.path.dirname(os.path.dirname(here)))   # the repository root, for prism_b200
    from helpers import TINY_A, TINY_B, random_tokens
    from prism_b200.weights.random_init import write_model_folder
    from safetensors.torch import load_file, save_file
    import tempfile

    out = {}
    for name, raw, seed, n_tok in (("A", TINY_A, 0, 33), ("B", TINY_B, 2, 40)):
        with tempfile.TemporaryDirectory() as d:
            write_model_folder(raw, seed, d)
            weights = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
        cfg = SimpleNamespace(num_hidden_layers=raw["num_hidden_layers"], hidden_size=raw["hidden_size"],
                              num_attention_heads=raw["num_attention_heads"],
                              num_key_value_heads=raw["num_key_value_heads"],
                              intermediate_size=raw["intermediate_size"], vocab_size=raw["vocab_size"],
                              rope_theta=raw["rope_theta"], rms_norm_eps=raw["rms_norm_eps"],
                              max_position_embeddings=raw["max_position_embeddings"])
        pool = StaticWeightPool(cfg, "cpu", torch.float32)
        pool.load_from_pinned(weights, cfg)
        hd = raw["hidden_size"] // raw["num_attention_heads"]
        kv = FlashAttnKVCache(raw["num_hidden_layers"], raw["num_key_value_heads"], hd, 16, 16, "cpu", torch.float32)
        E = ex.FlashAttnExecutorV3(pool, kv, "cpu", use_cuda_graph=False)
        E._cos, E._sin = E._cos.float(), E._sin.float()      # bf16-rounded values, float32 arithmetic
        ids = torch.tensor([random_tokens(raw["vocab_size"], n_tok, 50)])
        with torch.no_grad():
            kv.new_sequence(0)
            whole = E.prefill(ids, 0)[0, 0]
            # the same prompt in two portions through prefix_len (executor.py:82-101)
            kv.new_sequence(1)
            E.prefill(ids[:, :n_tok // 2], 1)
            cont = E.prefill(ids, 1, prefix_len=n_tok // 2)[0, 0]
            # shorter prompts give the logits at earlier positions
            rows = []
            for n in (1, 2, n_tok // 2):
                kv.new_sequence(10 + n)
                rows.append(E.prefill(ids[:, :n], 10 + n)[0, 0])
        out[f"{name}.tokens"] = ids[0].to(torch.int32)
        out[f"{name}.last_logits"] = whole.contiguous()
        out[f"{name}.last_logits_two_portions"] = cont.contiguous()
        out[f"{name}.logits_at_1_2_half"] = torch.stack(rows).contiguous()
        out[f"{name}.cos"] = E._cos[0, :n_tok, 0, :hd // 2].contiguous()
        out[f"{name}.sin"] = E._sin[0, :n_tok, 0, :hd // 2].contiguous()
        print(name, "max |whole - two portions| =", float((whole - cont).abs().max()))
    save_file(out, args.out)
    print("wrote", args.out, {k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
