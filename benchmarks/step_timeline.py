"""Timeline of one decode step inside its CUDA graph: when each kernel starts and ends, from the
CUDA activity records that torch.profiler collects (no serialisation, no replays: the kernels
overlap as they do in production, so a kernel that was launched early and sat in its dependency
wait shows a long duration and a negative gap).

    python benchmarks/step_timeline.py [--batch 8] [--layers 28] [--context 2048] [--shape 7b|14b|32b]

Prints the kernels of the first two layers and of the step's end, then one layer's critical path:
for every kernel, how long after the end of the kernel before it its own end comes.
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from bench import BASE, SHAPES  # noqa: E402
from prism_b200 import Engine, EngineConfig, SchedulerConfig, ops  # noqa: E402
from prism_b200.engine.batch import Segment  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--shape", default="7b", choices=["7b", "14b", "32b"], help="layer sizes (Qwen2.5-7B / 14B / 32B)")
    args = ap.parse_args()
    B = args.batch
    cfg = dict(BASE, **SHAPES[args.shape])
    cfg["num_hidden_layers"] = args.layers
    pages = (args.context + 256) // 256 + 1
    ec = EngineConfig(kv_page_size=256, num_pages=B * pages + 8, max_seq_len=4096, use_cuda_graph=True,
                      graph_batch_sizes=(B,), scheduler=SchedulerConfig(max_num_seqs=B))
    eng = Engine(None, ec, dtype="bfloat16", config=cfg, random_seed=0)
    r = eng.runner
    g = torch.Generator().manual_seed(1)
    ids = list(range(B))
    for i in ids:
        r.begin_request(i)
        r.step([Segment(i, torch.randint(0, 1000, (args.context,), generator=g).tolist(), [])])
    out = torch.empty(B, dtype=torch.int32, device="cuda:0")

    def one():
        ops.sample(r.step([Segment(i, [1], [0]) for i in ids]), None, None, out)
    for _ in range(10):
        one()
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            one()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(ev) if "embed_kernel" in e.name]
    ev = ev[first[-1]:]                                    # the last of the three steps
    t0 = ev[0].time_range.start

    def short(name):
        return name.replace("void ", "").replace("prism::", "").split("(")[0][:44]
    print(f"{'kernel':44s} {'start':>8s} {'length':>7s} {'end':>8s} {'end - end of the one before':>28s}   (us)")
    prev_end = t0
    per_layer = max(1, (len(ev) - 6) // max(1, args.layers))
    for k, e in enumerate(ev):
        s, t = e.time_range.start - t0, e.time_range.end - t0
        if k < 3 + 2 * per_layer or k >= len(ev) - 4:
            print(f"{short(e.name):44s} {s:8.1f} {t - s:7.1f} {t:8.1f} {t - (prev_end - t0):28.1f}")
        prev_end = max(prev_end, e.time_range.end)
    print(f"whole step: {ev[-1].time_range.end - t0:.1f} us, {len(ev)} kernels")


if __name__ == "__main__":
    main()
