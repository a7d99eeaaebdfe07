"""Prefill cost per token against the number of tokens a step carries (8 layers of the chosen shape, requests of
256 tokens each so that attention per token stays the same): the library GEMMs' tile grids fill the GPU's SMs
more or less well depending on the token count, and `SchedulerConfig.max_batch_tokens` decides which count a
loaded engine runs at.

    python benchmarks/prefill_step_sizes.py 7b|14b|32b
"""

import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from prism_b200 import Engine, EngineConfig, SchedulerConfig  # noqa: E402
from prism_b200.engine.batch import Segment  # noqa: E402

from bench import BASE, SHAPES  # noqa: E402


def main():
    model = sys.argv[1] if len(sys.argv) > 1 else "7b"
    cfg = dict(BASE, **SHAPES[model])
    cfg["num_hidden_layers"] = 8
    ec = EngineConfig(kv_page_size=256, num_pages=80, max_seq_len=4096, use_cuda_graph=False,
                      scheduler=SchedulerConfig(max_num_seqs=64))
    runner = Engine(None, ec, dtype="bfloat16", config=cfg, random_seed=0).runner
    g = torch.Generator().manual_seed(1)
    for m in (8, 9, 10, 11, 12, 14, 16, 20, 21, 22, 31, 32, 42):
        T, best = 256 * m, float("inf")
        for rep in range(4):
            ids = [f"m{m}_{rep}_{i}" for i in range(m)]
            segs = []
            for rid in ids:
                runner.begin_request(rid)
                segs.append(Segment(rid, torch.randint(0, 1000, (256,), generator=g).tolist(), []))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            runner.step(segs)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
            for rid in ids:
                runner.end_request(rid)
        print(f"{model}: {T:6d} tokens a step: {best:8.3f} ms for 8 layers, {best / T * 1e3:6.3f} us per token", flush=True)


if __name__ == "__main__":
    main()
