"""Trace replay: feed given token ids through the model step by step and write
the logits.  Nothing is sampled.  It drives the same model, step function,
cache manager and kernels that generation uses; andre-fu/prism's nearest
relatives are ``FlashAttnExecutorV3.generate`` (engine/executor.py:411-429)
and the all-positions verify pass of engine/speculative_executor.py:113-164.

Steps arrive on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the
logits at the wanted places (order of the entries and of ``want``) as
little-endian float32 ``[wanted, vocab]``.  After every step ``done <step>``
is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from .batch import Segment
from .runner import ModelRunner
from ..weights.loader import load_model_folder

ROUND = 64          # --max-tokens counts each request rounded up to this many tokens


def build_runner(model_dir: str, dtype: str, max_tokens: int, page_size: int, max_live: int, device="cuda:0"):
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    cfg, model, pool = load_model_folder(model_dir, device, tdt)
    if ROUND % page_size and page_size % ROUND:
        raise SystemExit(f"--page-size {page_size} must divide or be a multiple of {ROUND}")
    unit = max(page_size, ROUND)
    budget = (max_tokens + unit - 1) // unit * unit
    num_pages = max(1, budget // page_size)
    max_seq_len = min(model.spec.max_positions, num_pages * page_size)
    runner = ModelRunner(model, device, tdt, page_size, num_pages, max_live, max_seq_len, use_cuda_graph=False)
    return cfg, model, pool, runner


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=8, help="request slots")
    ap.add_argument("--gpu", type=int, default=0)
    args = ap.parse_args(argv)

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 1
    os.makedirs(args.out, exist_ok=True)
    device = f"cuda:{args.gpu}"
    torch.cuda.set_device(args.gpu)
    _, model, _, runner = build_runner(args.model, args.dtype, args.max_tokens, args.page_size,
                                       args.max_live, device)
    live = set()
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        segs = []
        for e in step.get("entries", []):
            if e["id"] not in live:
                runner.begin_request(e["id"])
                live.add(e["id"])
            if not e["tokens"] and not e.get("want"):
                continue                      # a request that brings no tokens this step: nothing to run
            segs.append(Segment(e["id"], e["tokens"], e.get("want", [])))
        logits = runner.step(segs)
        if logits is not None and logits.shape[0] > 0:
            data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step['step']}.f32.tmp")
            data.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step['step']}.f32"))
        for rid in step.get("end", []):
            if rid in live:
                runner.end_request(rid)
                live.discard(rid)
        runner.check_errors()
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
