"""Each part alone against the plain implementation's function of the same
name, and toy parts - a mixer with state of its own, a position encoding with
weights, a feed-forward with routing - defined here, registered, built and
stepped without touching the framework's files (GPU)."""

import tempfile

import pytest
import torch

from helpers import P, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_ctx(segs, dtype, W=8, page_size=8, tables=None, max_positions=4096):
    """A StepContext for segments [(cached_len, q_len)] of requests 0, 1, ...; tables: per-request page lists."""
    from prism_b200.engine.batch import BatchLayout, StepContext, pack_batch
    tok, pos, seg_of, seg_start, cached, qlen = [], [], [], [0], [], []
    for i, (c, n) in enumerate(segs):
        tok += [0] * n
        pos += list(range(c, c + n))
        seg_of += [i] * n
        seg_start.append(len(tok))
        cached.append(c)
        qlen.append(n)
    S = len(segs)
    layout = BatchLayout(len(tok), S, len(tok), W, [0])
    rows = tables or [list(range(i * W, (i + 1) * W)) for i in range(S)]
    host = pack_batch(layout, tok, pos, seg_of, seg_start, cached, qlen, list(range(S)), list(range(len(tok))),
                      {0: rows}, {0: S * W})
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = StepContext(layout, host.to(DEV), dtype, torch.device(DEV), err, max_positions,
                      dict(seg_start=seg_start, cached_len=cached, q_len=qlen, slots=list(range(S)), tok_seg=seg_of),
                      max(qlen), max(c + n for c, n in segs))
    return ctx


def build(category, kind, args, tensors, dtype):
    from prism_b200.parts import PartSpec, build_part
    part = build_part(category, PartSpec(kind, args))
    names = {q for q, _ in part.named_params()}
    assert names == set(tensors), (names, set(tensors))
    part.bind({k: v.to(DEV).to(dtype if v.is_floating_point() else v.dtype) for k, v in tensors.items()},
              torch.device(DEV), dtype)
    return part


TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    H, T = 200, 7
    w = torch.randn(H) * 0.1 + 1
    part = build("norm", "rmsnorm", dict(width=H, eps=4e-6), {"weight": w}, dtype)
    ctx = make_ctx([(0, T)], dtype)
    res = torch.randn(T, H, device=DEV)
    delta = torch.randn(T, H, device=DEV).to(dtype)
    want_res = res.cpu() + delta.float().cpu()
    out = part.forward(ctx, res, delta)
    wq = w.to(dtype).float()
    assert torch.allclose(res.cpu(), want_res, atol=1e-6)
    assert torch.allclose(out.float().cpu(), P.rms_norm(want_res, wq, 4e-6), atol=TOL[dtype], rtol=TOL[dtype])


def test_rotary_part_matches_the_plain_angles():
    part = build("position", "rotary", dict(head_dim=48, theta=50000.0), {}, torch.float32)
    rp = part.rotary()
    want = 1.0 / (50000.0 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert rp.rotary_dim == 48 and torch.equal(rp.inv_freq.cpu(), want)
    pos = torch.tensor([0, 1, 77, 4095])
    assert torch.equal(torch.outer(pos.float(), rp.inv_freq.cpu()), P.rope_angles(pos, 48, 50000.0))
    with pytest.raises(ValueError):
        build("position", "rotary", dict(head_dim=48, theta=1e4, rotary_dim=50), {}, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 40])
def test_swiglu_part(dtype, T):
    H, I = 72, 200
    g, u, d = torch.randn(I, H) * 0.1, torch.randn(I, H) * 0.1, torch.randn(H, I) * 0.1
    part = build("feed_forward", "swiglu", dict(hidden_size=H, intermediate_size=I),
                 {"gate_up_w": torch.cat([g, u]), "down_w": d}, dtype)
    x = (torch.randn(T, H)).to(dtype)
    out = part.forward(make_ctx([(0, T)], dtype), x.to(DEV))
    q = lambda t: t.to(dtype).float()
    xf = x.float()
    want = P.swiglu(xf @ q(g).T, xf @ q(u).T) @ q(d).T
    assert torch.allclose(out.float().cpu(), want, atol=TOL[dtype] * float(want.abs().max() + 1), rtol=TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    V, H = 77, 40
    E = torch.randn(V, H)
    emb = build("embedding", "token", dict(vocab_size=V, hidden_size=H), {"weight": E}, dtype)
    ctx = make_ctx([(0, 5)], dtype)
    ids = torch.tensor([3, 76, 0, 3, 9], dtype=torch.int32, device=DEV)
    ctx.token_ids.copy_(ids)
    out = emb.forward(ctx)
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), P.embed(ids.cpu().long(), E.to(dtype).float()))
    head = build("head", "linear", dict(vocab_size=V, hidden_size=H), {"weight": E}, dtype)
    h = torch.randn(4, H).to(dtype)
    logits = head.forward(ctx, h.to(DEV))
    assert logits.dtype == torch.float32
    assert torch.allclose(logits.cpu(), h.float() @ E.to(dtype).float().T, atol=TOL[dtype], rtol=TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window,bias", [(4, 2, 16, None, True), (6, 3, 64, 9, False), (3, 1, 48, None, True)])
def test_attention_part_whole_and_in_portions(dtype, nh, nkv, hd, window, bias):
    """The attention mixer alone over a cache of its own: a whole sequence in one
    call, then the same sequence in three portions into fresh pages."""
    from prism_b200.cache.storage import PagedCacheView
    from prism_b200.parts import PartSpec
    H, T, Pg, W = 56, 29, 8, 6
    qs, kvs = nh * hd, nkv * hd
    wq, wk, wv, wo = (torch.randn(qs, H) * 0.2, torch.randn(kvs, H) * 0.2, torch.randn(kvs, H) * 0.2,
                      torch.randn(H, qs) * 0.2)
    tensors = {"qkv_w": torch.cat([wq, wk, wv]), "o_w": wo}
    bq = bk = bv = None
    if bias:
        bq, bk, bv = torch.randn(qs) * 0.2, torch.randn(kvs) * 0.2, torch.randn(kvs) * 0.2
        tensors["qkv_b"] = torch.cat([bq, bk, bv])
    part = build("mixer", "gqa_attention",
                 dict(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, qkv_bias=bias, window=window,
                      position=PartSpec("rotary", dict(head_dim=hd, theta=1e4))), tensors, dtype)
    assert part.cache_need().kind == "paged" and part.cache_need().window == window
    x = torch.randn(T, H).to(dtype)
    rd = lambda t: None if t is None else t.to(dtype).float()
    xf = x.float()
    q = xf @ rd(wq).T + (rd(bq) if bias else 0)
    k = xf @ rd(wk).T + (rd(bk) if bias else 0)
    v = xf @ rd(wv).T + (rd(bv) if bias else 0)
    cos, sin = P.rope_cos_sin(torch.arange(T), hd, 1e4)
    a = P.attention(P.apply_rope(q.view(T, nh, hd), cos, sin), P.apply_rope(k.view(T, nkv, hd), cos, sin),
                    v.view(T, nkv, hd), window)
    want = a.reshape(T, qs) @ rd(wo).T
    tol = TOL[dtype] * float(want.abs().max() + 1)

    def cache_view(ctx, pages=W):
        kc = torch.full((pages + 1, Pg, nkv, hd), float("nan"), dtype=dtype, device=DEV)
        return PagedCacheView(kc, kc.clone(), ctx.block_tables[0], pages + 1, Pg, True, window, 0)

    ctx = make_ctx([(0, T)], dtype, W=W, page_size=Pg, tables=[[4, 2, 0, 5]])
    out = part.forward(ctx, x.to(DEV), cache_view(ctx))
    assert int(ctx.err) == 0 and torch.allclose(out.float().cpu(), want, atol=tol, rtol=TOL[dtype])
    view, got, at = None, [], 0
    for n in (11, 2, 16):
        ctx = make_ctx([(at, n)], dtype, W=W, page_size=Pg, tables=[[1, 3, 5, 0]])
        view = cache_view(ctx) if view is None else PagedCacheView(view.k, view.v, ctx.block_tables[0], W + 1, Pg,
                                                                   True, window, 0)
        got.append(part.forward(ctx, x[at:at + n].to(DEV), view))
        at += n
    assert torch.allclose(torch.cat(got).float().cpu(), want, atol=tol, rtol=TOL[dtype])


# --------------------------------------------------------------------------
# a toy architecture made of a new mixer (state of its own), the stock attention
# and feed-forward, a layer that runs twice and a run that reads another run's cache
# --------------------------------------------------------------------------

DECAY = 0.75


def register_toy():
    from prism_b200.model_registry import register_architecture
    from prism_b200.models.decoder import ModelSpec, ScheduleEntry
    from prism_b200.parts import CacheNeed, Mixer, ParamSpec, PartSpec, WeightSource, register_part

    @register_part("mixer", "toy_decay")
    class ToyDecay(Mixer):
        """s_t = DECAY * s_{t-1} + W x_t per request; output s_t.  The state is
        one vector per request in a cache slot."""

        def __init__(self, hidden_size):
            self.h = hidden_size

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.h,), state_dtype="float32")

        def params(self):
            return [ParamSpec("w_in", (WeightSource("w_in", (self.h, self.h)),))]

        def forward(self, ctx, x, cache):
            u = x.float() @ self.w["w_in"].float().T
            out = torch.empty_like(u)
            starts = ctx.host["seg_start"]
            for s, slot in enumerate(ctx.host["slots"]):
                st = cache.state[slot].clone()
                for t in range(starts[s], starts[s + 1]):
                    st = DECAY * st + u[t]
                    out[t] = st
                cache.state[slot] = st
            return out.to(x.dtype)

    @register_part("mixer", "toy_decay_on_device")
    class ToyDecayOnDevice(ToyDecay):
        """The same mixer for models that want their decode steps replayed from CUDA graphs: a step in
        which every request brings one token is computed from the device's slot array alone (gather the
        states, advance them, scatter them back), so nothing of it depends on the host's copy of the step."""
        graph_safe = True

        def forward(self, ctx, x, cache):
            if not ctx.decode_only:
                return super().forward(ctx, x, cache)
            u = x.float() @ self.w["w_in"].float().T
            slots = cache.slots.long()
            st = DECAY * cache.state[slots] + u
            cache.state.index_copy_(0, slots, st)          # padded rows of a graph all point at the spare slot
            return st.to(x.dtype)

    def spec(cfg):
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        norm = lambda p: PartSpec("rmsnorm", dict(width=H, eps=1e-5), prefix=p)
        ff = lambda p: PartSpec("swiglu", dict(hidden_size=H, intermediate_size=cfg["intermediate_size"]), prefix=p)
        l0 = PartSpec("prenorm", dict(mixer=PartSpec(cfg.get("mixer_kind", "toy_decay"), dict(hidden_size=H), prefix="l0.mix."),
                                      feed_forward=ff("l0.ff."), mixer_norm=norm("l0.n1."), ff_norm=norm("l0.n2.")))
        l1 = PartSpec("prenorm", dict(
            mixer=PartSpec("gqa_attention", dict(hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16,
                                                 qkv_bias=False, position=PartSpec("rotary", dict(head_dim=16, theta=1e4))),
                           prefix="l1.attn."),
            feed_forward=ff("l1.ff."), mixer_norm=norm("l1.n1."), ff_norm=norm("l1.n2.")))
        return ModelSpec("ToyDecayForCausalLM", H, V, 512,
                         PartSpec("token", dict(vocab_size=V, hidden_size=H), prefix="emb."), [l0, l1],
                         norm("final."), PartSpec("linear", dict(vocab_size=V, hidden_size=H, tied_to="embedding.weight"),
                                                  prefix="head."),
                         schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=1)])

    register_architecture("ToyDecayForCausalLM", lambda raw: raw, spec)


def toy_plain(t, tokens):
    """The toy model on a whole sequence, no cache, float32."""
    T = len(tokens)
    x = t["emb.embed_tokens.weight"][torch.tensor(tokens)]
    cos, sin = P.rope_cos_sin(torch.arange(T), 16, 1e4)

    def ffn(x, p):
        h = P.rms_norm(x, t[p + "n2.weight"], 1e-5)
        return x + P.swiglu(h @ t[p + "ff.gate_proj.weight"].T, h @ t[p + "ff.up_proj.weight"].T) @ t[p + "ff.down_proj.weight"].T

    def l0(x):
        u = P.rms_norm(x, t["l0.n1.weight"], 1e-5) @ t["l0.mix.w_in"].T
        s, out = torch.zeros(x.shape[1]), []
        for i in range(T):
            s = DECAY * s + u[i]
            out.append(s)
        return ffn(x + torch.stack(out), "l0.")

    def l1(x, kv=None):
        h = P.rms_norm(x, t["l1.n1.weight"], 1e-5)
        q = P.apply_rope((h @ t["l1.attn.q_proj.weight"].T).view(T, 4, 16), cos, sin)
        if kv is None:
            kv = (P.apply_rope((h @ t["l1.attn.k_proj.weight"].T).view(T, 2, 16), cos, sin),
                  (h @ t["l1.attn.v_proj.weight"].T).view(T, 2, 16))
        a = P.attention(q, kv[0], kv[1])
        return ffn(x + a.reshape(T, 64) @ t["l1.attn.o_proj.weight"].T, "l1."), kv

    x = l0(x)
    x, kv = l1(x)
    x = l0(x)
    x, _ = l1(x, kv)                      # reads the keys and values of the first run
    return P.rms_norm(x, t["final.weight"], 1e-5) @ t["emb.embed_tokens.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from safetensors.torch import load_file
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.weights.loader import load_model_folder
    from prism_b200.weights.random_init import write_model_folder
    from helpers import run_trace, trace_mixed, trace_portions, trace_whole, trace_budget
    register_toy()
    raw = dict(architectures=["ToyDecayForCausalLM"], hidden_size=48, intermediate_size=80, vocab_size=97)
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(raw, 11, d, store_dtype=torch.float32)
        t = load_file(d + "/model.safetensors")
        assert "l0.mix.w_in" in t and "head.weight" not in t
        seqs = {f"r{i}": random_tokens(97, n, 40 + i) for i, n in enumerate([5, 23, 41, 64])}
        for make in (trace_whole, trace_portions, lambda s: trace_mixed(s, seed=3)):
            steps = make(seqs)
            _, model, pool = load_model_folder(d, DEV, torch.float32)
            assert [n.kind if n else None for n in model.cache_needs()] == ["state", "paged", "state", None]
            runner = ModelRunner(model, DEV, torch.float32, 8, trace_budget(steps, 8) // 8, 4)
            assert [g.kind for g in runner.groups] == ["state", "paged"] and runner.groups[0].num_planes == 2
            got = run_trace(runner, steps)
            for rid, seq in seqs.items():
                ref = toy_plain(t, seq)
                for pos in range(len(seq)):
                    err = float((got[(rid, pos)] - ref[pos]).abs().max())
                    assert err < 5e-5, (rid, pos, err)


def test_toy_state_mixer_with_cuda_graphs_requested():
    """A mixer that keeps per-request state reads the host's copy of the step (its slots), which a
    captured graph does not have: asked for graphs, the runner runs such a model eagerly instead of
    capturing it - the decoded tokens' logits are those of the plain model, not a crash."""
    from safetensors.torch import load_file
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.weights.loader import load_model_folder
    from prism_b200.weights.random_init import write_model_folder
    from helpers import run_trace, trace_tail, trace_budget
    register_toy()
    raw = dict(architectures=["ToyDecayForCausalLM"], hidden_size=48, intermediate_size=80, vocab_size=97)
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(raw, 11, d, store_dtype=torch.float32)
        t = load_file(d + "/model.safetensors")
        seqs = {f"r{i}": random_tokens(97, n, 50 + i) for i, n in enumerate([19, 33])}
        steps = trace_tail(seqs, 12)                     # the last 12 tokens one by one: pure-decode steps
        _, model, pool = load_model_folder(d, DEV, torch.float32)
        runner = ModelRunner(model, DEV, torch.float32, 8, trace_budget(steps, 8) // 8, 4, use_cuda_graph=True,
                             graph_batch_sizes=(1, 2))
        assert not runner.graph_safe and not runner.use_cuda_graph
        got = run_trace(runner, steps)
        assert not runner._graphs
        for rid, seq in seqs.items():
            ref = toy_plain(t, seq)
            for pos in range(len(seq)):
                assert float((got[(rid, pos)] - ref[pos]).abs().max()) < 5e-5, (rid, pos)
        # the variant of the mixer that works from the device's slot array declares itself safe: graphs are captured
        with tempfile.TemporaryDirectory() as d2:
            write_model_folder(dict(raw, mixer_kind="toy_decay_on_device"), 11, d2, store_dtype=torch.float32)
            _, model2, pool2 = load_model_folder(d2, DEV, torch.float32)
            runner2 = ModelRunner(model2, DEV, torch.float32, 8, trace_budget(steps, 8) // 8, 4, use_cuda_graph=True,
                                  graph_batch_sizes=(1, 2))
            assert runner2.graph_safe and runner2.use_cuda_graph
            got2 = run_trace(runner2, steps)
            assert runner2._graphs and runner2.graph_kernel_launches > 0
            for rid, seq in seqs.items():
                ref = toy_plain(t, seq)
                for pos in range(len(seq)):
                    assert float((got2[(rid, pos)] - ref[pos]).abs().max()) < 5e-5, (rid, pos)
    # the stock attention model keeps its graphs
    from helpers import model_folder
    _, m2, pool2 = load_model_folder(model_folder("A"), DEV, torch.float32)
    r2 = ModelRunner(m2, DEV, torch.float32, 16, 8, 4, use_cuda_graph=True, graph_batch_sizes=(1, 2))
    assert r2.graph_safe and r2.use_cuda_graph


# --------------------------------------------------------------------------
# a second toy architecture: a position encoding with weights of its own (a learned
# table added to q and k) and a feed-forward with routing (top-1 of small experts,
# router logits in float32), beside the stock parts; different mixers' settings and
# feed-forwards in different layers
# --------------------------------------------------------------------------

N_EXPERTS, EXPERT_WIDTH, MAX_POS = 3, 24, 160


def register_toy_routed():
    from prism_b200.model_registry import register_architecture
    from prism_b200.models.decoder import ModelSpec
    from prism_b200.parts import FeedForward, ParamSpec, PartSpec, PositionEncoding, WeightSource, register_part

    @register_part("position", "toy_learned")
    class ToyLearnedPositions(PositionEncoding):
        """q[t, h] += table[pos_t]; k[t, h] += table[pos_t].  Not a rotary encoding: the mixer
        calls ``apply``."""

        def __init__(self, head_dim, max_positions):
            self.hd, self.n = head_dim, max_positions

        def params(self):
            return [ParamSpec("table", (WeightSource("table", (self.n, self.hd)),))]

        def apply(self, ctx, q, k):
            add = self.w["table"][ctx.positions.long()].to(q.dtype)[:, None, :]
            q += add
            k += add

    @register_part("feed_forward", "toy_top1_experts")
    class ToyTop1Experts(FeedForward):
        """Each token goes to the expert whose router logit (float32) is largest; its output is
        scaled by that expert's softmax probability."""

        def __init__(self, hidden_size, experts, expert_width):
            self.h, self.e, self.w_ = hidden_size, experts, expert_width

        def params(self):
            ps = [ParamSpec("router", (WeightSource("router.weight", (self.e, self.h)),))]
            for i in range(self.e):
                ps.append(ParamSpec(f"up{i}", (WeightSource(f"experts.{i}.up.weight", (self.w_, self.h)),)))
                ps.append(ParamSpec(f"down{i}", (WeightSource(f"experts.{i}.down.weight", (self.h, self.w_)),)))
            return ps

        def forward(self, ctx, x):
            logits = x.float() @ self.w["router"].float().T
            prob = torch.softmax(logits, -1)
            pick = logits.argmax(-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for i in range(self.e):
                rows = (pick == i).nonzero().flatten()
                if rows.numel():
                    h = torch.nn.functional.silu(x[rows].float() @ self.w[f"up{i}"].float().T)
                    out[rows] = (h @ self.w[f"down{i}"].float().T) * prob[rows, i:i + 1]
            return out.to(x.dtype)

    def spec(cfg):
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        norm = lambda p, eps: PartSpec("rmsnorm", dict(width=H, eps=eps), prefix=p)
        l0 = PartSpec("prenorm", dict(
            mixer=PartSpec("gqa_attention", dict(hidden_size=H, num_heads=3, num_kv_heads=1, head_dim=16, qkv_bias=True,
                                                 position=PartSpec("toy_learned", dict(head_dim=16, max_positions=MAX_POS),
                                                                   prefix="l0.attn.pos.")),
                           prefix="l0.attn."),
            feed_forward=PartSpec("toy_top1_experts", dict(hidden_size=H, experts=N_EXPERTS, expert_width=EXPERT_WIDTH),
                                  prefix="l0.moe."),
            mixer_norm=norm("l0.n1.", 1e-5), ff_norm=norm("l0.n2.", 1e-5)))
        l1 = PartSpec("prenorm", dict(
            mixer=PartSpec("gqa_attention", dict(hidden_size=H, num_heads=2, num_kv_heads=2, head_dim=32, qkv_bias=False,
                                                 window=19, position=PartSpec("rotary", dict(head_dim=32, theta=5e3, rotary_dim=16))),
                           prefix="l1.attn."),
            feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=cfg["intermediate_size"]), prefix="l1.ff."),
            mixer_norm=norm("l1.n1.", 1e-6), ff_norm=norm("l1.n2.", 1e-6)))
        return ModelSpec("ToyRoutedForCausalLM", H, V, MAX_POS,
                         PartSpec("token", dict(vocab_size=V, hidden_size=H), prefix="emb."), [l0, l1],
                         norm("final.", 1e-6), PartSpec("linear", dict(vocab_size=V, hidden_size=H), prefix="head."))

    register_architecture("ToyRoutedForCausalLM", lambda raw: raw, spec)


def toy_routed_plain(t, tokens):
    T = len(tokens)
    x = t["emb.embed_tokens.weight"][torch.tensor(tokens)]
    # layer 0: learned positions, one kv head, routed feed-forward
    h = P.rms_norm(x, t["l0.n1.weight"], 1e-5)
    add = t["l0.attn.pos.table"][:T][:, None, :]
    q = (h @ t["l0.attn.q_proj.weight"].T + t["l0.attn.q_proj.bias"]).view(T, 3, 16) + add
    k = (h @ t["l0.attn.k_proj.weight"].T + t["l0.attn.k_proj.bias"]).view(T, 1, 16) + add
    v = (h @ t["l0.attn.v_proj.weight"].T + t["l0.attn.v_proj.bias"]).view(T, 1, 16)
    x = x + P.attention(q, k, v).reshape(T, 48) @ t["l0.attn.o_proj.weight"].T
    h = P.rms_norm(x, t["l0.n2.weight"], 1e-5)
    logits = h @ t["l0.moe.router.weight"].T
    prob, pick = torch.softmax(logits, -1), logits.argmax(-1)
    out = torch.zeros_like(h)
    for i in range(T):
        e = int(pick[i])
        out[i] = (torch.nn.functional.silu(h[i] @ t[f"l0.moe.experts.{e}.up.weight"].T)
                  @ t[f"l0.moe.experts.{e}.down.weight"].T) * prob[i, e]
    x = x + out
    # layer 1: partial rotary (16 of 32), window 19, dense feed-forward
    h = P.rms_norm(x, t["l1.n1.weight"], 1e-6)
    cos, sin = P.rope_cos_sin(torch.arange(T), 16, 5e3)
    q = (h @ t["l1.attn.q_proj.weight"].T).view(T, 2, 32).clone()
    k = (h @ t["l1.attn.k_proj.weight"].T).view(T, 2, 32).clone()
    q[..., :16], k[..., :16] = P.apply_rope(q[..., :16], cos, sin), P.apply_rope(k[..., :16], cos, sin)
    v = (h @ t["l1.attn.v_proj.weight"].T).view(T, 2, 32)
    x = x + P.attention(q, k, v, 19).reshape(T, 64) @ t["l1.attn.o_proj.weight"].T
    h = P.rms_norm(x, t["l1.n2.weight"], 1e-6)
    x = x + P.swiglu(h @ t["l1.ff.gate_proj.weight"].T, h @ t["l1.ff.up_proj.weight"].T) @ t["l1.ff.down_proj.weight"].T
    return P.rms_norm(x, t["final.weight"], 1e-6) @ t["head.weight"].T


def test_toy_position_encoding_and_routed_feed_forward():
    """Another position encoding (with weights of its own) and a feed-forward with routing,
    defined here and registered, make a model with the stock attention: built from a
    configuration, written and loaded by tensor name, stepped whole, in portions and mixed."""
    from safetensors.torch import load_file
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.weights.loader import load_model_folder
    from prism_b200.weights.random_init import write_model_folder
    from helpers import run_trace, trace_mixed, trace_portions, trace_whole, trace_budget
    register_toy_routed()
    raw = dict(architectures=["ToyRoutedForCausalLM"], hidden_size=40, intermediate_size=56, vocab_size=83)
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(raw, 5, d, store_dtype=torch.float32)
        t = load_file(d + "/model.safetensors")
        assert t["l0.attn.pos.table"].shape == (MAX_POS, 16) and t["l0.moe.experts.2.down.weight"].shape == (40, EXPERT_WIDTH)
        seqs = {f"r{i}": random_tokens(83, n, 60 + i) for i, n in enumerate([4, 27, 50, 90])}
        for make in (trace_whole, trace_portions, lambda s: trace_mixed(s, seed=9)):
            steps = make(seqs)
            _, model, pool = load_model_folder(d, DEV, torch.float32)
            assert [n.window for n in model.cache_needs()] == [None, 19]
            runner = ModelRunner(model, DEV, torch.float32, 8, trace_budget(steps, 8) // 8, 4)
            assert len(runner.groups) == 2                        # all keys / a window of them
            got = run_trace(runner, steps)
            for rid, seq in seqs.items():
                ref = toy_routed_plain(t, seq)
                for pos in range(len(seq)):
                    err = float((got[(rid, pos)] - ref[pos]).abs().max())
                    assert err < 5e-5, (rid, pos, err)
            assert runner.cache.pages_in_use() == 0
