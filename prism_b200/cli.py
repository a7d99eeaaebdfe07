"""Command line in the manner of andre-fu/prism's ``python -m engine``
(engine/__main__.py:15-22, which no longer imports there): ``--model``,
``--name``, ``--gpu``, ``--prompt``, ``--max-tokens`` (default 100),
``--dtype`` (default bfloat16) keep their names and meanings, and the same
figures are printed at the end (:117-124).  Added: token-id prompts (there is
no tokenizer without network), random-weights mode, sampling and cache knobs.
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="python -m prism_b200", description="Single-GPU inference engine (B200)")
    p.add_argument("--model", help="model folder: config.json + model.safetensors")
    p.add_argument("--name", default="", help="Model display name")
    p.add_argument("--gpu", type=int, default=0, help="GPU ID")
    p.add_argument("--prompt", default=None, help="Input prompt text (needs tokenizer files in the model folder)")
    p.add_argument("--prompt-ids", default=None, help="Input prompt as comma-separated token ids")
    p.add_argument("--prompt-len", type=int, default=None, help="Random prompt of this many tokens")
    p.add_argument("--prompt-seed", type=int, default=1)
    p.add_argument("--num-prompts", type=int, default=1, help="Copies of the prompt (random prompts differ)")
    p.add_argument("--max-tokens", type=int, default=100, help="Max new tokens")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="Model dtype")
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--sample-seed", type=int, default=0)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--random-weights", action="store_true", help="draw weights from --seed instead of reading them")
    p.add_argument("--config-json", help="config.json for --random-weights")
    p.add_argument("--seed", type=int, default=0, help="weight seed for --random-weights")
    p.add_argument("--write-model", metavar="DIR", help="with --random-weights: write the model folder and exit")
    p.add_argument("--page-size", type=int, default=64)
    p.add_argument("--num-pages", type=int, default=None)
    p.add_argument("--kv-budget-gb", type=float, default=35.0)
    p.add_argument("--max-batch-tokens", type=int, default=4096)
    p.add_argument("--prefill-chunk", type=int, default=2048)
    p.add_argument("--max-num-seqs", type=int, default=64)
    p.add_argument("--max-seq-len", type=int, default=None)
    p.add_argument("--no-cuda-graph", action="store_true")
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch
    from .config.engine_config import EngineConfig, ModelConfig, SchedulerConfig
    from .sampling.sampler import SamplingParams

    raw = None
    if args.random_weights:
        if not args.config_json:
            print("--random-weights needs --config-json", file=sys.stderr)
            return 2
        with open(args.config_json) as f:
            raw = json.load(f)
        if args.write_model:
            from .weights.random_init import write_model_folder
            write_model_folder(raw, args.seed, args.write_model)
            print(f"wrote {args.write_model}")
            return 0
    elif not args.model:
        print("give --model DIR or --random-weights --config-json FILE", file=sys.stderr)
        return 2

    from .engine.llm import Engine
    ec = EngineConfig(gpu_id=args.gpu, kv_page_size=args.page_size, num_pages=args.num_pages,
                      kv_cache_budget_gb=args.kv_budget_gb, max_seq_len=args.max_seq_len,
                      use_cuda_graph=not args.no_cuda_graph, seed=args.sample_seed,
                      scheduler=SchedulerConfig(args.max_batch_tokens, args.max_num_seqs, args.prefill_chunk))
    t0 = time.perf_counter()
    if raw is not None:
        eng = Engine(None, ec, dtype=args.dtype, config=raw, random_seed=args.seed)
    else:
        eng = Engine(ModelConfig(args.model, args.name, args.dtype), ec)
    t_load = time.perf_counter() - t0
    vocab = eng.model.spec.vocab_size

    tokenizer = None
    if args.prompt_ids:
        prompts = [[int(x) for x in args.prompt_ids.split(",")]] * args.num_prompts
    elif args.prompt_len:
        g = torch.Generator().manual_seed(args.prompt_seed)
        prompts = [torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist() for _ in range(args.num_prompts)]
    else:
        text = args.prompt if args.prompt is not None else "The capital of France is"
        try:
            from tokenizers import Tokenizer
            import os
            tokenizer = Tokenizer.from_file(os.path.join(args.model or "", "tokenizer.json"))
        except Exception as e:  # no tokenizer files offline
            print(f"no tokenizer in the model folder ({e}); use --prompt-ids or --prompt-len", file=sys.stderr)
            return 2
        prompts = [tokenizer.encode(text).ids] * args.num_prompts
    print(f"\nPrompt: {len(prompts)} x {len(prompts[0])} tokens; weights {eng.pool.total_gb:.2f} GB loaded in {t_load:.1f}s")

    sp = SamplingParams(max_new_tokens=args.max_tokens, temperature=args.temperature, seed=args.sample_seed,
                        ignore_eos=args.ignore_eos)
    print("Warming up...")
    eng.generate(prompts[:1], SamplingParams(max_new_tokens=min(5, args.max_tokens), ignore_eos=True))
    print("Generating...\n")
    torch.cuda.synchronize()
    t_start = time.perf_counter()
    results = eng.generate(prompts, sp)
    torch.cuda.synchronize()
    t_total = time.perf_counter() - t_start

    r0 = results[0]
    if tokenizer is not None:
        print(f"Output: {tokenizer.decode(prompts[0] + r0.token_ids)}")
    else:
        print(f"Output ids: {r0.token_ids}")
    n_gen = sum(len(r.token_ids) for r in results)
    ttft = max(r.ttft for r in results)
    n_dec = max(len(r0.token_ids) - 1, 1)
    t_dec = max(t_total - ttft, 1e-9)
    print()
    print("--- Performance ---")
    print(f"TTFT (prefill):    {ttft * 1000:.1f} ms ({len(prompts[0])} tokens)")
    print(f"Decode:            {t_dec:.3f}s ({n_dec} steps)")
    print(f"TBT:               {r0.tbt * 1000:.1f} ms")
    print(f"Decode tok/s:      {(n_gen - len(results)) / t_dec:.1f}")
    print(f"Total tok/s:       {n_gen / t_total:.1f}")
    print(f"KV pages used:     {eng.cache.pages_high_water} (high water)")
    print(f"GPU memory:        {torch.cuda.memory_allocated(args.gpu) / 1e9:.1f} GB")
    return 0
