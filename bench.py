"""Headline benchmark: decode tokens/s (batch 8 by default) and prefill
tokens/s at 2,048 tokens for a Qwen2.5-7B-shaped random-weight model in bf16
on one B200, each with its fraction of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout.  A "step" is one decode step of the whole batch.
Timing is on the device with CUDA events after W warm-up steps; every step
reads all weights (15 GB), far more than the 126 MB L2, so no flush is needed.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=3584,
                 num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
                 vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                 max_position_embeddings=32768, use_sliding_window=False)
CONTEXT, PROMPT, PAGE = 4096, 2048, 256
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                v = raw.get(k)
                if isinstance(v, dict):
                    v = v.get("value")
                if v:
                    out[k] = float(v)
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu=0):
        self.rows, self.proc, self.gpu = [], None, gpu

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


def model_bytes_flops(cfg, B, ctx_mean, T_prefill):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (nh + 2 * nkv) * hd
    per_layer = qkv * H + qkv + nh * hd * H + 2 * I * H + H * I + 2 * H
    # decode reads every weight it uses once: all layers, final norm, head; B embedding rows
    weight_bytes = 2 * (L * per_layer + H + V * H + B * H)
    kv_bytes = B * ctx_mean * L * 2 * nkv * hd * 2
    gemm_flops = 2 * T_prefill * L * (qkv * H + nh * hd * H + 2 * I * H + H * I) + 2 * V * H
    attn_flops = L * 4 * nh * hd * (T_prefill * (T_prefill + 1) // 2)
    return weight_bytes, kv_bytes, gemm_flops + attn_flops


def run(args):
    import torch
    from prism_b200 import Engine, EngineConfig, SamplingParams, SchedulerConfig, ops
    from prism_b200.engine.batch import Segment

    pk = peaks()
    cfg = dict(QWEN25_7B)
    layers_model = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    B, K, Wm = args.batch, args.steps, args.warmup
    pages_per_seq = CONTEXT // PAGE
    ec = EngineConfig(kv_page_size=PAGE, num_pages=64 * pages_per_seq + 8, max_seq_len=CONTEXT, use_cuda_graph=True,
                      graph_batch_sizes=(1, 8, 64),
                      scheduler=SchedulerConfig(max_batch_tokens=max(8, B) * PROMPT, max_num_seqs=64, prefill_chunk=PROMPT))
    eng = Engine(None, ec, dtype="bfloat16", config=cfg, random_seed=0)
    runner, dev = eng.runner, eng.device
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def prompts(n):
        return [torch.randint(0, V, (PROMPT,), generator=g).tolist() for _ in range(n)]

    sample_out = torch.empty(64, dtype=torch.int32, device=dev)

    def decode_bench(batch, steps, warmup, clocks=None):
        """Prefill `batch` prompts of PROMPT tokens, then time `steps` decode steps."""
        ids = [f"b{batch}_{i}" for i in range(batch)]
        for rid, p in zip(ids, prompts(batch)):
            runner.begin_request(rid)
            runner.step([Segment(rid, p, [])])
        toks = [1] * batch

        def one():
            logits = runner.step([Segment(rid, [t], [0]) for rid, t in zip(ids, toks)])
            ops.sample(logits, None, None, sample_out[:batch])
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        l0, g0 = ops.launch_count, runner.graph_kernel_launches
        if clocks:
            clocks.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        ck = clocks.stop() if clocks else None
        launches = (ops.launch_count - l0) + (runner.graph_kernel_launches - g0)
        ctx_mean = PROMPT + warmup + steps / 2
        for rid in ids:
            runner.end_request(rid)
        runner.check_errors()
        return ms, launches, ctx_mean, ck

    if args.quick == "prefill":
        # one prompt of PROMPT tokens, a few times, for profilers
        p = prompts(1)[0]
        times = []
        for i in range(max(2, K)):
            runner.begin_request("pf")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([Segment("pf", p, [PROMPT - 1])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            runner.end_request("pf")
        print(json.dumps({"quick": "prefill", "layers": cfg["num_hidden_layers"], "tokens": PROMPT,
                          "ms": round(min(times[1:]), 3)}))
        return
    if args.quick:
        # decode only, for profilers: no prefill timing, no other batch sizes, no end-to-end run
        ms, launches, ctx_mean, _ = decode_bench(B, K, Wm)
        print(json.dumps({"quick": True, "batch": B, "layers": cfg["num_hidden_layers"], "ms_per_step": round(ms, 4),
                          "tok_s": round(B / ms * 1e3, 1), "gpu_launches": int(launches)}))
        return
    # ---- prefill of one 2,048-token prompt -------------------------------------
    runner.begin_request("pf")
    p = prompts(1)[0]
    pre_ms = []
    for i in range(4):
        if i:
            runner.end_request("pf")
            runner.begin_request("pf")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([Segment("pf", p, [PROMPT - 1])])
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
    runner.end_request("pf")
    prefill_ms = min(pre_ms[1:])

    # ---- decode ------------------------------------------------------------------
    clocks = ClockSampler()
    ms, launches, ctx_mean, ck = decode_bench(B, K, Wm, clocks)
    wbytes, kvbytes, pf_flops = model_bytes_flops(cfg, B, ctx_mean, PROMPT)
    achieved = (wbytes + kvbytes) / (ms * 1e-3) / 1e9
    points = {}
    for b in (1, 64):
        if b == B:
            points[f"decode_b{b}"] = round(B / ms * 1e3, 1)
            continue
        m, _, _, _ = decode_bench(b, max(8, K // 4), 3)
        points[f"decode_b{b}"] = round(b / m * 1e3, 1)

    # ---- end to end through Engine.generate: host token ids in, host token ids out ----
    n_new = max(8, min(K, 256))      # the first ~20 steps after the prompts run at the lower clocks the prefill left
    res = eng.generate(prompts(B), SamplingParams(max_new_tokens=n_new, ignore_eos=True))   # warm
    t_first = time.perf_counter()
    res = eng.generate(prompts(B), SamplingParams(max_new_tokens=n_new, ignore_eos=True))
    # all B prompts are prefilled in one step (the token budget allows it), so every later step is a
    # pure decode step of the whole batch; tbt is the engine's own host clock between a request's tokens
    tbt = sum(r.tbt for r in res) / len(res)
    e2e = B / tbt if tbt > 0 else 0.0
    lay_total = runner.last_h2d_bytes            # the packed batch descriptor of a decode step

    out = {
        "metric": "decode tok/s (Qwen2.5-7B shape, bf16, batch %d, 2048-token prompts)" % B,
        "value": round(B / ms * 1e3, 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": Wm,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init weights normal(0,0.02), uniform-random token ids",
        "config": {"model": "Qwen2.5-7B-shaped", "global_batch": B, "seq_len": CONTEXT, "parallelism": "single-gpu",
                   "layers": cfg["num_hidden_layers"], "layers_of_model": layers_model, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": V,
                   "prompt_len": PROMPT, "page_size": PAGE, "cuda_graph": True,
                   "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": lay_total, "d2h_bytes_per_step": 4 * B},
        "gpu_launches": int(launches),
        "clocks": ck,
        "prefill": {"value": round(PROMPT / prefill_ms * 1e3, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(pf_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    # vs_baseline: the reference publishes 1,096 tok/s at batch 8 (H100, 5-token prompts); other batches: none
    published = {1: 150.0, 2: 286.0, 4: 564.0, 8: 1096.0, 16: 2133.0, 32: 4000.0}
    if B in published:
        out["vs_baseline"] = round(out["value"] / published[B], 3)
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--quick", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                    help="only the decode steps at --batch, or only the prefill (short runs under a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "andre-fu/prism has no setup.py/pyproject.toml (pip: 'not installable') and its stock path "
                          "fetches weights with huggingface_hub.snapshot_download; there is no network"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    run(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
