"""The two serving workloads that the baseline names beside the headline configuration, through the
public entry point (`Engine.generate`: host token ids in, host token ids out), random weights:

    python benchmarks/workloads.py 14b    Qwen2.5-14B shape: 32 requests, prompts of 128..4,096 tokens, 256 new tokens each
    python benchmarks/workloads.py 32b    Qwen2.5-32B shape: 64 requests, prompts of 1,024 tokens, 512 new tokens each,
                                          the cache pool filling what the weights leave of the GPU's memory

Prints one JSON line: wall time, generated tokens per second, prompt tokens per second over the whole
run, steps, preemptions, the time to the first token (mean) and between tokens (mean).
"""

import argparse
import json
import os
import random
import sys
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from prism_b200 import Engine, EngineConfig, SamplingParams, SchedulerConfig  # noqa: E402

from bench import BASE, SHAPES  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which", choices=["14b", "32b"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in the output)")
    args = ap.parse_args()
    cfg = dict(BASE, **SHAPES[args.which])
    layers_of_model = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    rnd = random.Random(0)
    g = torch.Generator().manual_seed(0)
    if args.which == "14b":
        lens, new, budget_gb = [rnd.randint(128, 4096) for _ in range(32)], 256, 40.0
    else:
        lens, new, budget_gb = [1024] * 64, 512, None
    free, total = torch.cuda.mem_get_info(0)
    if budget_gb is None:
        # what the weights and a few GB of activations leave
        H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
        qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
        weights = 2 * (L * (qkv * H + cfg["num_attention_heads"] * cfg["head_dim"] * H + 3 * I * H) + 2 * V * H)
        budget_gb = max(4.0, (free - weights) / 1e9 - 12.0)
    ec = EngineConfig(kv_page_size=256, kv_cache_budget_gb=budget_gb, max_seq_len=8192, use_cuda_graph=True,
                      scheduler=SchedulerConfig(max_batch_tokens=4096, max_num_seqs=64, prefill_chunk=2048))
    eng = Engine(None, ec, dtype="bfloat16", config=cfg, random_seed=0)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    sp = SamplingParams(max_new_tokens=new, ignore_eos=True)
    # capture the decode graphs of every bucket before the timed run, as a server does when it starts
    eng.warmup()
    eng.generate([p[:16] for p in prompts[:4]], SamplingParams(max_new_tokens=3, ignore_eos=True))
    steps0, pre0 = eng.stats.steps, eng.stats.preemptions
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = eng.generate(prompts, sp)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    eng.runner.check_errors()
    gen = sum(len(r.token_ids) for r in res)
    print(json.dumps({
        "workload": args.which, "layers": cfg["num_hidden_layers"], "layers_of_model": layers_of_model, "requests": len(lens),
        "prompt_tokens": sum(lens), "generated_tokens": gen, "wall_s": round(wall, 3),
        "generated_tok_s": round(gen / wall, 1), "all_tok_s": round((gen + sum(lens)) / wall, 1),
        "steps": eng.stats.steps - steps0, "preemptions": eng.stats.preemptions - pre0,
        "ttft_mean_s": round(sum(r.ttft for r in res) / len(res), 3), "tbt_mean_ms": round(1e3 * sum(r.tbt for r in res) / len(res), 3),
        "kv_pool_gb": round(eng.runner.storage.bytes() / 1e9, 1), "dtype": "bf16", "data": "random weights, uniform-random token ids"}))


if __name__ == "__main__":
    main()
