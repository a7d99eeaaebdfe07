"""Decode steps of requests with unequal contexts against requests with equal contexts of the same total,
through the engine's own step function (CUDA graphs on), random weights:

    python benchmarks/ragged_decode.py 7b 64      Qwen2.5-7B shape, 64 requests: contexts of 128..4,096 tokens (one of
                                                  them 4,096), then 64 equal contexts of their mean

Prints one JSON line for each: milliseconds a step over 100 steps after 10 warm-ups (CUDA events).  With
``--no-plan`` the step's descriptor carries no work items for the decode attention kernel, and every request gets
the same number of CTAs, chosen from the longest context (the behaviour the items replaced).
"""

import argparse
import json
import os
import random
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from prism_b200 import Engine, EngineConfig, SchedulerConfig, ops  # noqa: E402
from prism_b200.engine.batch import Segment  # noqa: E402

from bench import BASE, SHAPES  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("model", choices=sorted(SHAPES))
    ap.add_argument("batch", type=int)
    ap.add_argument("--no-plan", action="store_true")
    args = ap.parse_args()
    B = args.batch
    cfg = dict(BASE, **SHAPES[args.model])
    rnd = random.Random(0)
    ragged = [rnd.randint(128, 4096) for _ in range(B)]
    ragged[0] = 4096
    uniform = [sum(ragged) // B] * B
    ec = EngineConfig(kv_page_size=256, num_pages=B * 18 + 8, max_seq_len=4608, use_cuda_graph=True,
                      graph_batch_sizes=(B,), scheduler=SchedulerConfig(max_num_seqs=B))
    eng = Engine(None, ec, dtype="bfloat16", config=cfg, random_seed=0)
    runner = eng.runner
    if args.no_plan:
        runner._decode_work = lambda cached, qlen, n_real=None: {}
    g = torch.Generator().manual_seed(1)
    out = torch.empty(B, dtype=torch.int32, device="cuda:0")
    for name, lens in (("equal", uniform), ("unequal", ragged)):
        ids = [f"{name}{i}" for i in range(B)]
        for rid, n in zip(ids, lens):
            runner.begin_request(rid)
            runner.step([Segment(rid, torch.randint(0, 1000, (n,), generator=g).tolist(), [])])

        def one():
            ops.sample(runner.step([Segment(rid, [1], [0]) for rid in ids]), None, None, out)
        for _ in range(10):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(100):
            one()
        e1.record()
        torch.cuda.synchronize()
        runner.check_errors()
        print(json.dumps({"model": args.model, "batch": B, "contexts": name, "plan": not args.no_plan,
                          "mean": round(sum(lens) / B, 1), "longest": max(lens),
                          "ms_per_step": round(e0.elapsed_time(e1) / 100, 4)}), flush=True)
        for rid in ids:
            runner.end_request(rid)


if __name__ == "__main__":
    main()
