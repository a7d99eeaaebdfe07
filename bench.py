"""Headline benchmark: decode tokens/s (batch 8 by default; batch 1 and 64 as
``points``) and prefill tokens/s at 2,048 tokens for a Qwen2.5-7B-shaped
random-weight model in bf16 on one B200, each with its fraction of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
                    [--model 7b|14b|32b] [--prompt-len N] [--batch B]

One JSON line on stdout.  A "step" is one decode step of the whole batch.
Timing is on the device with CUDA events after W warm-up steps; every step
reads all weights (15 GB), far more than the 126 MB L2, so no flush is needed.

``--impl reference`` runs andre-fu/prism's own classes, unmodified, from a
copy of its tree under ``baseline/_ref`` (the classes its own GPU test drives,
tests/test_engine_correctness.py:14-55: ``StaticWeightPool`` +
``load_from_pinned``, ``FlashAttnKVCache``, ``FlashAttnExecutorV3`` with
``warmup_batch_graphs``, ``prefill`` and ``batched_decode_step``) on the same
shape, prompts and step counts, and prints the same line with
``"impl": "reference"``.  Nothing of ``prism_b200`` is imported on that path.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

BASE = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", head_dim=128, vocab_size=152064,
            rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=32768,
            use_sliding_window=False)
SHAPES = {
    "7b": dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944),
    "14b": dict(num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=27648),
}
PAGE = 256
POINT_STEPS, POINT_WARMUP = 128, 5        # decode steps timed for each of the other batch sizes
E2E_MIN_TOKENS = 256                       # new tokens per request of the end-to-end run, at least
# Both arms wait this long between the prompts and the decode steps: for about 75 ms after a burst of prefill
# GEMMs at the power cap the GPU runs ~10 % slower (batch 8: 3.28 instead of 2.98 ms a step for the first
# 23 steps; with 0.3 s of rest 2.98 from the second step on), and a short run (--steps 20) would measure that.
# The end-to-end figure has no such rest: a request's tokens follow its prompt at once.
SETTLE_S = 0.5
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)
# what the reference publishes for this model (docs/benchmarks.md:9-14): one H100, 5-token prompts
PUBLISHED_H100 = {1: 150.0, 2: 286.0, 4: 564.0, 8: 1096.0, 16: 2133.0, 32: 4000.0}


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
    """Bytes a decode step must read (every weight once, B embedding rows, the live requests' keys and
    values) and the flops of a prefill of ``T_prefill`` tokens."""
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (nh + 2 * nkv) * hd
    per_layer = qkv * H + qkv + nh * hd * H + 2 * I * H + H * I + 2 * H
    weight_bytes = 2 * (L * per_layer + H + V * H + B * H)
    kv_bytes = B * ctx_mean * L * 2 * nkv * hd * 2
    gemm_flops = 2 * T_prefill * L * (qkv * H + nh * hd * H + 2 * I * H + H * I) + 2 * V * H
    attn_flops = L * 4 * nh * hd * (T_prefill * (T_prefill + 1) // 2)
    return weight_bytes, kv_bytes, gemm_flops + attn_flops


def shape_of(args):
    cfg = dict(BASE, **SHAPES[args.model])
    layers_model = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    return cfg, layers_model


def result_line(args, cfg, layers_model, pk, B, ms, ctx_mean, prefill_ms, points, e2e, launches, ck, impl=None,
                extra_config=None):
    """The one JSON line; the same keys for both arms."""
    PROMPT = args.prompt_len
    wbytes, kvbytes, pf_flops = model_bytes_flops(cfg, B, ctx_mean, PROMPT)
    achieved = (wbytes + kvbytes) / (ms * 1e-3) / 1e9
    config = {"model": f"Qwen2.5-{args.model.upper()}-shaped", "global_batch": B, "seq_len": 2 * PROMPT,
              "parallelism": "single-gpu", "layers": cfg["num_hidden_layers"], "layers_of_model": layers_model,
              "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
              "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
              "prompt_len": PROMPT, "page_size": PAGE, "cuda_graph": True,
              "l2": "inputs larger than L2 (all weights are read every step)", "peaks": pk["source"],
              "settle_s": SETTLE_S}
    config.update(extra_config or {})
    out = {
        "metric": "decode tok/s (Qwen2.5-%s shape, bf16, batch %d, %d-token prompts)" % (args.model.upper(), B, PROMPT),
        "value": round(B / ms * 1e3, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        # the reference publishes numbers for an H100 and 5-token prompts only: another GPU and another
        # workload, so no ratio is formed; the ratio that counts is against the reference arm on this GPU
        "vs_baseline": None,
        "baseline_note": ("published by the reference: %s tok/s at batch %d on one H100 80GB with 5-token prompts "
                          "(docs/benchmarks.md:9-14); not comparable with this GPU and %d-token prompts"
                          % (PUBLISHED_H100.get(B, "nothing"), B, PROMPT)),
        "dtype": "bf16", "data": "synthetic: random-init weights normal(0,0.02), uniform-random token ids",
        "config": config, "e2e": e2e, "gpu_launches": int(launches), "clocks": ck,
        "prefill": {"value": round(PROMPT / prefill_ms * 1e3, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(pf_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        # decode at batch 1 and 64: tokens a second, and beside them the step time and the fraction of the
        # measured copy bandwidth (weights once + the live requests' keys and values over the step time)
        "points": {k: v and v["value"] for k, v in points.items()},
        "points_ms": {k: v and v["ms"] for k, v in points.items()},
        "points_frac": {k: v and v["frac"] for k, v in points.items()},
    }
    if impl:
        out["impl"] = impl
    return out


def point(cfg, pk, b, ms, ctx_mean, prompt_len):
    w, kv, _ = model_bytes_flops(cfg, b, ctx_mean, prompt_len)
    gbs = (w + kv) / (ms * 1e-3) / 1e9
    return {"value": round(b / ms * 1e3, 1), "ms": round(ms, 4), "frac": round(gbs / pk["hbm_gbs"], 4)}


# --------------------------------------------------------------------------
# this engine
# --------------------------------------------------------------------------

def run(args):
    sys.path.insert(0, ROOT)
    import torch
    from prism_b200 import Engine, EngineConfig, SamplingParams, SchedulerConfig, ops
    from prism_b200.engine.batch import Segment

    pk = peaks()
    cfg, layers_model = shape_of(args)
    PROMPT, CONTEXT = args.prompt_len, 2 * args.prompt_len
    B, K, Wm = args.batch, args.steps, args.warmup
    pages_per_seq = CONTEXT // PAGE
    # the cache pool holds the largest batch that is measured: 64 requests for the batch-64 point, unless only
    # --batch is asked for (--quick) or 64 requests of this context do not fit beside the weights - then the
    # batch-64 point is left out (null)
    w_bytes, kv_per_seq, _ = model_bytes_flops(cfg, 1, CONTEXT, PROMPT)
    room = torch.cuda.mem_get_info(0)[0] - w_bytes - (12 << 30)
    most = B if args.quick else max(64, B)
    if most * kv_per_seq > room:
        most = max(B, min(most, int(room // kv_per_seq)))
    ec = EngineConfig(kv_page_size=PAGE, num_pages=most * pages_per_seq + 8, max_seq_len=CONTEXT, use_cuda_graph=True,
                      graph_batch_sizes=tuple(sorted({1, 8, 64, B})),
                      scheduler=SchedulerConfig(max_batch_tokens=max(8, B) * PROMPT, max_num_seqs=most,
                                                prefill_chunk=PROMPT))
    eng = Engine(None, ec, dtype="bfloat16", config=cfg, random_seed=0)
    runner, dev = eng.runner, eng.device
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def prompts(n):
        return [torch.randint(0, V, (PROMPT,), generator=g).tolist() for _ in range(n)]

    sample_out = torch.empty(most, dtype=torch.int32, device=dev)

    def decode_bench(batch, steps, warmup, clocks=None):
        """Prefill `batch` prompts of PROMPT tokens, then time `steps` decode steps."""
        ids = [f"b{batch}_{i}" for i in range(batch)]
        for rid, p in zip(ids, prompts(batch)):
            runner.begin_request(rid)
            runner.step([Segment(rid, p, [])])
        toks = [1] * batch
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)

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
        print(json.dumps(dict(point(cfg, pk, B, ms, ctx_mean, PROMPT), quick=True, batch=B, layers=cfg["num_hidden_layers"],
                              gpu_launches=int(launches))))
        return
    # ---- prefill of one prompt ---------------------------------------------------
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
    points = {}
    for b in (1, 64):
        if b == B:
            points[f"decode_b{b}"] = point(cfg, pk, b, ms, ctx_mean, PROMPT)
            continue
        if b > most:
            points[f"decode_b{b}"] = None              # that many requests of this context do not fit
            continue
        m, _, c, _ = decode_bench(b, POINT_STEPS, POINT_WARMUP)
        points[f"decode_b{b}"] = point(cfg, pk, b, m, c, PROMPT)

    # ---- end to end through Engine.generate: host token ids in, host token ids out ----
    # At least E2E_MIN_TOKENS new tokens per request whatever --steps is: the first steps after the
    # prompts run at the lower clocks the prefill left, and a short run would measure mostly that.
    n_new = max(E2E_MIN_TOKENS, min(K, 256))
    res = eng.generate(prompts(B), SamplingParams(max_new_tokens=n_new, ignore_eos=True))   # warm
    res = eng.generate(prompts(B), SamplingParams(max_new_tokens=n_new, ignore_eos=True))
    # all B prompts are prefilled in one step (the token budget allows it), so every later step is a
    # pure decode step of the whole batch; tbt is the engine's own host clock between a request's tokens
    tbt = sum(r.tbt for r in res) / len(res)
    e2e = {"value": round(B / tbt if tbt > 0 else 0.0, 1), "unit": "tok/s", "new_tokens": n_new,
           "h2d_bytes_per_step": runner.last_h2d_bytes, "d2h_bytes_per_step": 4 * B}
    print(json.dumps(result_line(args, cfg, layers_model, pk, B, ms, ctx_mean, prefill_ms, points, e2e, launches, ck)))


# --------------------------------------------------------------------------
# the reference arm
# --------------------------------------------------------------------------

def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def run_reference(args):
    ref = os.environ.get("PRISM_REFERENCE_DIR") or os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref, "engine", "executor.py")):
        return unavailable(f"no copy of andre-fu/prism under baseline/_ref (engine/executor.py not found in {ref}); "
                           "it has no setup.py/pyproject.toml, so pip cannot install it: copy its tree there")
    # the reference's package is called `engine`, as is this repository's forwarder for `python -m engine`:
    # its tree goes first on the path, and this repository's root is taken off it
    sys.path[:] = [ref] + [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    try:
        import torch
        from types import SimpleNamespace
        from engine.executor import FlashAttnExecutorV3
        from engine.kv_cache import FlashAttnKVCache
        from engine.weight_pool import StaticWeightPool
    except Exception as e:                                      # noqa: BLE001  (flash_attn, triton or transformers missing)
        return unavailable(f"the reference does not import here: {type(e).__name__}: {e}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    try:
        return _run_reference(args, torch, SimpleNamespace, StaticWeightPool, FlashAttnKVCache, FlashAttnExecutorV3)
    except Exception as e:                                      # noqa: BLE001
        return unavailable(f"the reference's own path failed on this GPU: {type(e).__name__}: {e}")


def _run_reference(args, torch, SimpleNamespace, StaticWeightPool, FlashAttnKVCache, FlashAttnExecutorV3):
    pk = peaks()
    cfg, layers_model = shape_of(args)
    PROMPT = args.prompt_len
    B, K, Wm = args.batch, args.steps, args.warmup
    dev = "cuda:0"
    torch.cuda.set_device(0)
    hf = SimpleNamespace(num_hidden_layers=cfg["num_hidden_layers"], hidden_size=cfg["hidden_size"],
                         num_attention_heads=cfg["num_attention_heads"], num_key_value_heads=cfg["num_key_value_heads"],
                         intermediate_size=cfg["intermediate_size"], vocab_size=cfg["vocab_size"],
                         rope_theta=cfg["rope_theta"], rms_norm_eps=cfg["rms_norm_eps"],
                         max_position_embeddings=cfg["max_position_embeddings"])
    nh, nkv, H, I, V = hf.num_attention_heads, hf.num_key_value_heads, hf.hidden_size, hf.intermediate_size, hf.vocab_size
    hd = H // nh                                                 # the reference's own rule (executor.py:37)
    if hd != cfg["head_dim"]:
        return unavailable(f"the reference fixes head_dim = hidden/heads = {hd}, this shape has {cfg['head_dim']}")
    if 2 * PROMPT > 4096:
        return unavailable("the reference caps its rotary table at 4,096 positions (executor.py:46)")

    class RandomWeights:
        """HF tensor names -> normal(0, 0.02) tensors drawn on the GPU when asked for (``load_from_pinned``
        only indexes and tests membership), so the 15 GB never sit in host memory."""

        def __init__(self):
            self.shapes = {"model.embed_tokens.weight": (V, H), "lm_head.weight": (V, H), "model.norm.weight": (H,)}
            for i in range(hf.num_hidden_layers):
                p = f"model.layers.{i}."
                self.shapes.update({
                    p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
                    p + "self_attn.q_proj.weight": (nh * hd, H), p + "self_attn.k_proj.weight": (nkv * hd, H),
                    p + "self_attn.v_proj.weight": (nkv * hd, H), p + "self_attn.q_proj.bias": (nh * hd,),
                    p + "self_attn.k_proj.bias": (nkv * hd,), p + "self_attn.v_proj.bias": (nkv * hd,),
                    p + "self_attn.o_proj.weight": (H, nh * hd), p + "mlp.gate_proj.weight": (I, H),
                    p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I)})
            self.gen = torch.Generator(device=dev).manual_seed(0)

        def __contains__(self, name):
            return name in self.shapes

        def __getitem__(self, name):
            t = torch.randn(self.shapes[name], generator=self.gen, device=dev, dtype=torch.float32) * 0.02
            return (t + 1.0 if name.endswith("norm.weight") else t).to(torch.bfloat16)

    pool = StaticWeightPool(hf, dev, torch.bfloat16)
    pool.load_from_pinned(RandomWeights(), hf)
    most = max(64, B)
    pages_per_seq = 2 * PROMPT // PAGE
    kv = FlashAttnKVCache(hf.num_hidden_layers, nkv, hd, most * pages_per_seq + 8, PAGE, dev, torch.bfloat16)
    ex = FlashAttnExecutorV3(pool, kv, dev)
    g = torch.Generator().manual_seed(1)

    def prompt():
        return torch.randint(0, V, (1, PROMPT), generator=g).to(dev)

    launches = [0]

    def decode_bench(batch, steps, warmup, clocks=None, host_tokens=False):
        """`batch` sequences prefilled one after the other (the reference has no batched prefill), then
        `steps` steps of its decode entry point: `decode_step` for one sequence, `batched_decode_step`
        (graph of that batch size, `warmup_batch_graphs`) for more, as its scheduler calls them
        (engine/scheduler.py:255-264).  `host_tokens`: each step's token ids go through host lists."""
        kv.free_all()
        seqs = list(range(batch))
        with torch.no_grad():
            for s in seqs:
                kv.new_sequence(s)
                ex.prefill(prompt(), s)
            if batch > 1:
                ex.warmup_batch_graphs([batch])
            toks = [1] * batch
            torch.cuda.synchronize()
            time.sleep(SETTLE_S)

            def one():
                nonlocal toks
                if batch == 1:
                    logits = ex.decode_step(torch.tensor([[toks[0]]], device=dev), 0)[:, -1, :]
                else:
                    logits = ex.batched_decode_step(toks, seqs)
                nxt = logits.argmax(dim=-1)
                if host_tokens:
                    toks = nxt.tolist()
            for _ in range(warmup):
                one()
            torch.cuda.synchronize()
            if clocks:
                clocks.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) / steps
        ms = e0.elapsed_time(e1) / steps
        ck = clocks.stop() if clocks else None
        ex.invalidate_graph()
        return ms, PROMPT + warmup + steps / 2, ck, wall

    # ---- prefill ---------------------------------------------------------------------
    pre_ms = []
    with torch.no_grad():
        for i in range(4):
            kv.free_all()
            kv.new_sequence(0)
            ids = prompt()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            ex.prefill(ids, 0)
            e1.record()
            torch.cuda.synchronize()
            pre_ms.append(e0.elapsed_time(e1))
    prefill_ms = min(pre_ms[1:])
    # ---- decode ----------------------------------------------------------------------
    ms, ctx_mean, ck, _ = decode_bench(B, K, Wm, ClockSampler())
    points = {}
    for b in (1, 64):
        if b == B:
            points[f"decode_b{b}"] = point(cfg, pk, b, ms, ctx_mean, PROMPT)
            continue
        m, c, _, _ = decode_bench(b, POINT_STEPS, POINT_WARMUP)
        points[f"decode_b{b}"] = point(cfg, pk, b, m, c, PROMPT)
    # ---- end to end: host token ids into every step, host token ids out of it -----------
    n_new = max(E2E_MIN_TOKENS, min(K, 256))
    decode_bench(B, n_new, Wm, host_tokens=True)
    _, _, _, wall = decode_bench(B, n_new, Wm, host_tokens=True)
    e2e = {"value": round(B / wall, 1), "unit": "tok/s", "new_tokens": n_new,
           "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B}
    line = result_line(args, cfg, layers_model, pk, B, ms, ctx_mean, prefill_ms, points, e2e, 0, ck, impl="reference",
                       extra_config={"reference": "andre-fu/prism FlashAttnExecutorV3, unmodified"})
    line["gpu_launches"] = None          # the reference's kernels are libraries' (cuBLAS, flash-attn, Triton): not counted
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="7b", choices=sorted(SHAPES), help="layer sizes (default: the headline's)")
    ap.add_argument("--prompt-len", type=int, default=2048, help="prompt tokens (context = twice as many)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--quick", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                    help="only the decode steps at --batch, or only the prefill (short runs under a profiler)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.prompt_len % PAGE:
        ap.error(f"--prompt-len must be a multiple of the page size {PAGE}")
    if args.impl == "reference":
        return run_reference(args)
    run(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
