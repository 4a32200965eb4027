"""Each part of a block alone against the plain implementation's function for it, and the
generality of the parts: a run order that names a layer twice, a layer that reads another
layer's cache, an attention window, and toy parts that are defined and registered here,
without any change to the framework's files: a mixer with state of its own, a feed-forward with
routing, a position encoding.  Run on the CPU with the
torch statements of the kernels and on the GPU with the kernels."""

from __future__ import annotations

import torch

import plain_model as pm
from helpers import TINY, TEST_STD, random_ids
from qwen3_runtime_b200.cache import CacheManager
from qwen3_runtime_b200.cache.layout import CacheLayout, StateLayerSpec
from qwen3_runtime_b200.cache.storage import CacheStorage
from qwen3_runtime_b200.config import LayerRun, ModelSpec, PartSpec
from qwen3_runtime_b200.engine.batch import BatchBuilder, StepEntry
from qwen3_runtime_b200.engine.factory import build_runtime
from qwen3_runtime_b200.models.qwen3 import qwen3_spec
from qwen3_runtime_b200.parts import (BuildContext, DecoderModel, ParamSpec, Part, ResidualStream, build_part,
                                      register_part, unregister_part)
from qwen3_runtime_b200.weights import DictSource, load_into
from qwen3_runtime_b200.weights.loader import place

TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype, scale):
    return (2e-5 if dtype == "float32" else 2e-2) * max(1.0, scale)


def ctx_for(dtype, ops, device):
    return BuildContext(dtype=TD[dtype], device=torch.device(device), ops=ops)


def load_part(part, tensors, ctx):
    part.load({n: place(tensors[n], ps, ctx.dtype, ctx.device) for n, ps in part.param_specs().items()})


def draw(specs, seed):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for n, ps in specs.items():
        t = torch.randn(ps.shape, generator=g)
        out[n] = (1 + 0.1 * t if ps.kind == "vector" else TEST_STD * t).to(torch.bfloat16)
    return out


class OnePartHarness:
    """A cache and a step context for a single mixer: two sequences, one mid-way (portion after
    some cached tokens), one fresh."""

    def __init__(self, mixer, ctx, page_size=4):
        self.layout = CacheLayout({0: mixer.cache_spec()})
        self.cache = CacheManager(self.layout.group_specs, page_size, 32, 4)
        self.storage = CacheStorage(self.layout, page_size, 32, 4, ctx.dtype, ctx.device)
        self.builder = BatchBuilder(self.cache, ctx.device, vocab_size=1 << 20, max_positions=4096)
        self.handles = {}

    def step(self, spans):
        entries = []
        for rid, n in spans:
            rc = self.handles.get(rid) or self.handles.setdefault(rid, self.cache.open(rid))
            self.cache.reserve(rc, n)
            entries.append(StepEntry(rc, [0] * n, []))
        step = self.builder.build(entries)
        return step, entries

    def commit(self, entries):
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))


def case_norm_part(dtype, ops, device):
    ctx = ctx_for(dtype, ops, device)
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=80, eps=3e-5)), ctx)
    t = draw(norm.param_specs(), 1)
    load_part(norm, t, ctx)
    table = (torch.randn(50, 80) * 0.5).to(ctx.dtype).to(ctx.device)
    ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32, device=ctx.device)
    stream = ResidualStream(4, 80, ids=ids, table=table)
    h = norm.add_norm(stream)
    x = table.float().cpu()[ids.cpu().long()]
    want = pm.rmsnorm(x, t["weight"].float(), 3e-5)
    assert float((h.float().cpu() - want).abs().max()) <= tol(dtype, float(want.abs().max()))
    assert torch.equal(stream.resid.cpu(), x) and stream.embed is None
    pend = (torch.randn(4, 80) * 0.3).to(ctx.dtype).to(ctx.device)
    stream.pending = pend
    h2 = norm.add_norm(stream)
    x2 = x + pend.float().cpu()
    want2 = pm.rmsnorm(x2, t["weight"].float(), 3e-5)
    assert float((h2.float().cpu() - want2).abs().max()) <= tol(dtype, float(want2.abs().max()))
    assert torch.equal(stream.resid.cpu(), x2) and stream.pending is None
    # what is pending may be partial sums: float32 planes, added in order, then to the residual
    planes = (torch.randn(3, 4, 80) * 0.3).to(ctx.device)
    stream.pending = planes
    h3 = norm.add_norm(stream)
    x3 = x2 + ((planes[0] + planes[1]) + planes[2]).cpu()
    want3 = pm.rmsnorm(x3, t["weight"].float(), 3e-5)
    assert float((h3.float().cpu() - want3).abs().max()) <= tol(dtype, float(want3.abs().max()))
    assert torch.equal(stream.resid.cpu(), x3) and stream.pending is None


def case_position_part(dtype, ops, device):
    ctx = ctx_for(dtype, ops, device)
    pos = build_part("position", PartSpec("rope_neox", dict(rotary_dim=48, theta=5e5, max_positions=300)), ctx)
    cos, sin = pos.rotation_tables()
    c, s = pm.rope_tables(48, 5e5, torch.arange(300))
    assert float((cos.cpu() - c).abs().max()) < 2e-6 and float((sin.cpu() - s).abs().max()) < 2e-6
    assert pos.rotation_tables()[0] is cos  # one table per (dim, theta, length), shared by the layers
    assert build_part("position", PartSpec("none"), ctx).rotation_tables() is None


def case_mixer_part(dtype, ops, device, name="C"):
    """The attention part alone: a request fed in two portions equals the plain attention part
    on the whole sequence."""
    cfg = TINY[name]["config"]
    ctx = ctx_for(dtype, ops, device)
    spec = qwen3_spec(cfg).blocks[0]["mixer"]
    mixer = build_part("mixer", spec, ctx)
    t = draw(mixer.param_specs(), 2)
    load_part(mixer, t, ctx)
    T = 23
    x = (torch.randn(T, cfg.hidden_size, generator=torch.Generator().manual_seed(3))).to(ctx.dtype)
    harness = OnePartHarness(mixer, ctx)
    outs = []
    for lo, hi in ((0, 9), (9, T)):
        step, entries = harness.step([("a", hi - lo)])
        outs.append(mixer.forward(x[lo:hi].to(ctx.device).contiguous(), step, harness.storage.view(0)).float().cpu())
        harness.commit(entries)
    got = torch.cat(outs)
    act = torch.bfloat16 if dtype == "bfloat16" else None
    w = {"p." + k: v for k, v in t.items()}
    want, _ = pm.attention_part(x.float(), {k: v.float() for k, v in w.items()}, "p.", cfg.to_hf_config(),
                                torch.arange(T), act_dtype=act)
    assert float((got - want).abs().max()) <= tol(dtype, float(want.abs().max()))


def case_feed_forward_part(dtype, ops, device):
    ctx = ctx_for(dtype, ops, device)
    ff = build_part("feed_forward", PartSpec("gated_mlp", dict(hidden_size=80, intermediate_size=112)), ctx)
    t = draw(ff.param_specs(), 4)
    load_part(ff, t, ctx)
    x = torch.randn(9, 80, generator=torch.Generator().manual_seed(5)).to(ctx.dtype)
    got = ff.forward(x.to(ctx.device), None).float().cpu()
    act = torch.bfloat16 if dtype == "bfloat16" else None
    want = pm.swiglu_part(x.float(), {"p." + k: v.float() for k, v in t.items()}, "p.", act_dtype=act)
    assert float((got - want).abs().max()) <= tol(dtype, float(want.abs().max()))


def _toy_model(spec: ModelSpec, cfg, dtype, ops, device, seed=9):
    ctx = ctx_for(dtype, ops, device)
    model = DecoderModel(spec, ctx)
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for n, ps in model.expected_tensors().items():
        t = torch.randn(ps.shape, generator=g)
        tensors[n] = (1 + 0.05 * t if ps.kind == "vector" else TEST_STD * t).to(torch.bfloat16)
    load_into(model, DictSource(tensors))
    return model, tensors


def _run_cut(model, cfg, ids, page_size=4, cuts=(5, 2, 9, 1, 1, 30)):
    rt = build_runtime(model, max_positions=cfg.max_position_embeddings, block_size=page_size, num_kv_blocks=40,
                       max_num_seqs=2)
    rc = rt.cache.open("a")
    outs, i = [], 0
    for n in cuts:
        n = min(n, len(ids) - i)
        if n <= 0:
            break
        rt.cache.reserve(rc, n)
        outs.append(rt.runner.run([StepEntry(rc, ids[i:i + n], list(range(n)))]).float().cpu())
        i += n
    rt.cache.check_invariants()
    return torch.cat(outs), rt


def case_run_order_layer_twice_and_shared_cache(dtype, ops, device):
    """Order is data: block 0 runs twice (weights shared, a cache layer per run), and the last
    run reads the keys and values that block 1 stored instead of storing its own."""
    cfg = TINY["A"]["config"]
    base = qwen3_spec(cfg)
    order = (LayerRun(0, 0), LayerRun(1, 1), LayerRun(0, 2), LayerRun(1, 1, writes=False))
    spec = ModelSpec(base.vocab_size, base.hidden_size, base.blocks, order, base.final_norm, True)
    model, tensors = _toy_model(spec, cfg, dtype, ops, device)
    ids = random_ids(cfg.vocab_size, 40, 21)
    got, rt = _run_cut(model, cfg, ids)
    assert len(rt.model.cache_layout().groups[0].cache_ids) == 3  # three cache layers for four runs
    act = torch.bfloat16 if dtype == "bfloat16" else None
    want = pm.forward_logits(cfg.to_hf_config(), tensors, ids, act_dtype=act,
                             order=[(r.block, r.cache, r.writes) for r in order])
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) <= (3e-5 if dtype == "float32" else 0.03) * max(1.0, scale)


def case_window_attention(dtype, ops, device, window=7):
    """A window is a parameter of the attention part; its cache group returns pages behind the window."""
    cfg = TINY["A"]["config"]
    base = qwen3_spec(cfg)
    blocks = []
    for i, b in enumerate(base.blocks):  # layer 0 keeps everything, layer 1 looks back `window` tokens
        mixer = PartSpec("paged_attention", {**b["mixer"].params, "window": window if i == 1 else None})
        blocks.append(PartSpec("pre_norm", {**b.params, "mixer": mixer}))
    spec = ModelSpec(base.vocab_size, base.hidden_size, tuple(blocks), base.order, base.final_norm, True)
    model, tensors = _toy_model(spec, cfg, dtype, ops, device)
    ids = random_ids(cfg.vocab_size, 48, 22)
    got, rt = _run_cut(model, cfg, ids)
    kinds = [g.spec.kind for g in rt.model.cache_layout().groups]
    assert kinds == ["full", "window"]
    rc = next(iter(rt.cache.live.values()))
    assert len([p for p in rc.tables[0] if p >= 0]) == 12 and len([p for p in rc.tables[1] if p >= 0]) <= 3
    act = torch.bfloat16 if dtype == "bfloat16" else None
    raw = cfg.to_hf_config()
    # the plain model with the window in layer 1 only: run it layer by layer
    h, wc = pm.forward_hidden({**raw, "num_hidden_layers": 1}, tensors, ids, act_dtype=act)
    w1 = {k.replace("model.layers.1.", "model.layers.0."): v for k, v in tensors.items() if ".layers.1." in k}
    w1["model.embed_tokens.weight"] = torch.eye(1)  # unused below
    pos = torch.arange(len(ids))
    wf = {k: v.float() for k, v in tensors.items()}
    n = pm._round(pm.rmsnorm(h, wf["model.layers.1.input_layernorm.weight"], raw["rms_norm_eps"]), act)
    a, _ = pm.attention_part(n, wf, "model.layers.1.self_attn.", raw, pos, act_dtype=act, window=window)
    h = h + a
    n = pm._round(pm.rmsnorm(h, wf["model.layers.1.post_attention_layernorm.weight"], raw["rms_norm_eps"]), act)
    h = h + pm.swiglu_part(n, wf, "model.layers.1.mlp.", act_dtype=act)
    want = pm._round(pm.rmsnorm(h, wf["model.norm.weight"], raw["rms_norm_eps"]), act) @ wf["model.embed_tokens.weight"].T
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) <= (3e-5 if dtype == "float32" else 0.03) * max(1.0, scale)


class FinishedOnlyNorm(Part):
    """A toy norm that does not add partial sums (it does not say ``adds_partial_sums``): the parts
    that feed it must hand it finished products."""

    category = "norm"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.inner = build_part("norm", PartSpec("rmsnorm", spec.params), ctx)
        self.seen = 0

    def param_specs(self):
        return self.inner.param_specs()

    def load(self, tensors):
        self.inner.load(tensors)

    def kernel_groups(self):
        return self.inner.kernel_groups()

    def add_norm(self, stream, rows=None, num_rows=None):
        assert stream.pending is None or stream.pending.dim() == 2, "this norm was promised finished products"
        self.seen += 1
        return self.inner.add_norm(stream, rows=rows, num_rows=num_rows)


def case_partial_sums(dtype, ops, device):
    """A sublayer may hand its last product to the next norm as partial sums, if that norm adds
    them: who may is settled when the model is put together, from the run order.  The logits
    are the plain model's either way."""
    cfg = TINY["A"]["config"]
    base = qwen3_spec(cfg)
    ids = random_ids(cfg.vocab_size, 40, 23)
    act = torch.bfloat16 if dtype == "bfloat16" else None
    limit = (3e-5 if dtype == "float32" else 0.03)
    # (1) every norm adds partial sums: every mixer and feed-forward may produce them
    model, tensors = _toy_model(base, cfg, dtype, ops, device)
    assert all(b.mixer.partial_sums_ok and b.feed_forward.partial_sums_ok for b in model.blocks)
    want = pm.forward_logits(cfg.to_hf_config(), tensors, ids, act_dtype=act)
    scale = max(1.0, float(want.abs().max()))
    emulated = hasattr(ops, "partial_parts")
    try:
        if emulated:  # the stand-in for the kernels cuts every such product into three ranges
            ops.partial_parts = 3
        got, _ = _run_cut(model, cfg, ids)
    finally:
        if emulated:
            ops.partial_parts = 0
    assert float((got - want).abs().max()) <= limit * scale
    # (2) a norm that does not: block 1's second norm and the final norm
    register_part("norm", "finished_only", FinishedOnlyNorm)
    try:
        blocks = list(base.blocks)
        ffn = base.blocks[1]["feed_forward_norm"]
        blocks[1] = PartSpec("pre_norm", {**base.blocks[1].params,
                                          "feed_forward_norm": PartSpec("finished_only", ffn.params)})
        spec = ModelSpec(base.vocab_size, base.hidden_size, tuple(blocks), base.order,
                         PartSpec("finished_only", base.final_norm.params), True)
        model, tensors = _toy_model(spec, cfg, dtype, ops, device)
        flags = [(b.mixer.partial_sums_ok, b.feed_forward.partial_sums_ok) for b in model.blocks]
        assert flags == [(True, True), (False, False)]
        try:
            if emulated:
                ops.partial_parts = 3
            got, _ = _run_cut(model, cfg, ids)
        finally:
            if emulated:
                ops.partial_parts = 0
        assert model.final_norm.seen > 0 and model.blocks[1].feed_forward_norm.seen > 0
        want = pm.forward_logits(cfg.to_hf_config(), tensors, ids, act_dtype=act)
        assert float((got - want).abs().max()) <= limit * scale
        # (3) a block that runs twice hands on to two norms: both must add partial sums
        order = (LayerRun(0, 0), LayerRun(1, 1), LayerRun(0, 2))
        spec = ModelSpec(base.vocab_size, base.hidden_size, base.blocks, order,
                         PartSpec("finished_only", base.final_norm.params), True)
        model, _ = _toy_model(spec, cfg, dtype, ops, device)
        flags = [(b.mixer.partial_sums_ok, b.feed_forward.partial_sums_ok) for b in model.blocks]
        assert flags == [(True, False), (True, True)]
    finally:
        unregister_part("norm", "finished_only")


class DecayStateMixer(Part):
    """A toy mixer with fixed-size state of its own: s_t = decay * s_{t-1} + x_t W_in, out_t = s_t W_out.
    It keeps one vector per request in a state slot, reads it at the start of a portion and writes
    it back at the end.  (Plain torch on whatever device it is given; it is a test fixture, not a
    model of anything.)"""

    category = "mixer"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden, self.width, self.decay = int(spec["hidden_size"]), int(spec["state_size"]), float(spec["decay"])

    def param_specs(self):
        return {"in_proj.weight": ParamSpec((self.width, self.hidden)), "out_proj.weight": ParamSpec((self.hidden, self.width))}

    def load(self, tensors):
        self.w_in, self.w_out = tensors["in_proj.weight"].float(), tensors["out_proj.weight"].float()

    def cache_spec(self):
        return StateLayerSpec((self.width,), "float32")

    def forward(self, h, step, cache):
        u = h.float() @ self.w_in.t()
        if step.decode_only and h.is_cuda:
            # one token per sequence: device-side gather and scatter of the slots, nothing read
            # back to the host, so the step can be captured into a CUDA graph
            slots = step.state_slots.long()
            s = self.decay * cache.state.index_select(0, slots) + u
            if cache.writes:
                cache.state.index_copy_(0, slots, s)
            return (s @ self.w_out.t()).to(h.dtype)
        out = torch.empty_like(h)
        slots = step.state_slots.tolist()
        for b in range(step.num_seqs):
            lo, hi = step.host_cu_seqlens[b], step.host_cu_seqlens[b + 1]
            s = cache.state[slots[b]].clone()
            for t in range(lo, hi):
                s = self.decay * s + u[t]
                out[t] = (s @ self.w_out.t()).to(h.dtype)
            if cache.writes:
                cache.state[slots[b]] = s
        return out


def case_toy_state_mixer(dtype, ops, device):
    """Register, build and step a mixer with per-request state next to an attention layer."""
    cfg = TINY["A"]["config"]
    base = qwen3_spec(cfg)
    register_part("mixer", "toy_decay_state", DecayStateMixer)
    try:
        toy = PartSpec("toy_decay_state", dict(hidden_size=cfg.hidden_size, state_size=24, decay=0.8))
        blocks = (base.blocks[0], PartSpec("pre_norm", {**base.blocks[1].params, "mixer": toy}))
        spec = ModelSpec(base.vocab_size, base.hidden_size, blocks, base.order, base.final_norm, True)
        model, tensors = _toy_model(spec, cfg, dtype, ops, device)
        assert "model.layers.1.self_attn.in_proj.weight" in tensors
        layout = model.cache_layout()
        assert [g.spec.kind for g in layout.groups] == ["full", "state"]
        rt = build_runtime(model, max_positions=512, block_size=4, num_kv_blocks=40, max_num_seqs=3)
        reqs = {"a": random_ids(cfg.vocab_size, 30, 31), "b": random_ids(cfg.vocab_size, 17, 32)}

        def run(plan):
            handles, got = {}, {k: [] for k in reqs}
            done = {k: 0 for k in reqs}
            for spans in plan:
                entries = []
                for rid, n in spans:
                    rc = handles.get(rid) or handles.setdefault(rid, rt.cache.open(rid))
                    rt.cache.reserve(rc, n)
                    entries.append(StepEntry(rc, reqs[rid][done[rid]:done[rid] + n], list(range(n))))
                logits = rt.runner.run(entries).float().cpu()
                row = 0
                for rid, n in spans:
                    got[rid].append(logits[row:row + n])
                    row += n
                    done[rid] += n
            for rc in handles.values():
                rt.cache.close(rc)
            return {k: torch.cat(v) for k, v in got.items()}

        whole = run([[("a", 30)], [("b", 17)]])
        # portions and decode steps mixed in one batch; the slots were used before, so the state
        # must have been zeroed when the requests started again
        mixed = run([[("a", 7), ("b", 2)], [("a", 1), ("b", 9)], [("b", 1)], [("a", 20), ("b", 5)], [("a", 2)]])
        t = 3e-5 if dtype == "float32" else 0.03 * float(whole["a"].abs().max())
        for k in reqs:
            assert float((whole[k] - mixed[k]).abs().max()) <= t
        # and the state matters: with another decay the logits move
        assert float((whole["a"][5:] - whole["a"][:-5]).abs().max()) > 1e-3
    finally:
        unregister_part("mixer", "toy_decay_state")


def case_toy_state_mixer_in_captured_steps(dtype, ops, device):
    """A model with a state layer decodes through captured graphs, with the engine running ahead
    and not: the same tokens as without graphs.  A graph is warmed up and captured on padding
    rows only, so the state of a live request is advanced exactly once per token; were it
    advanced by the warm-up as well, the first decode step of every new graph would count its
    token twice and the tokens would differ."""
    from qwen3_runtime_b200.engine.factory import build_engine

    cfg = TINY["A"]["config"]
    base = qwen3_spec(cfg)
    register_part("mixer", "toy_decay_state", DecayStateMixer)
    try:
        toy = PartSpec("toy_decay_state", dict(hidden_size=cfg.hidden_size, state_size=24, decay=0.8))
        blocks = (base.blocks[0], PartSpec("pre_norm", {**base.blocks[1].params, "mixer": toy}))
        spec = ModelSpec(base.vocab_size, base.hidden_size, blocks, base.order, base.final_norm, True)
        model, _ = _toy_model(spec, cfg, dtype, ops, device)
        prompts = [random_ids(cfg.vocab_size, n, 40 + n) for n in (9, 21, 4)]

        def tokens(cuda_graph, run_ahead):
            eng = build_engine(model=model, config=cfg, dtype=dtype, device=device, block_size=4, num_kv_blocks=60,
                               max_num_seqs=3, max_num_batched_tokens=16, cuda_graph=cuda_graph, run_ahead=run_ahead)
            out = eng.generate_batch(prompts, max_tokens=40)  # 40 tokens: the block tables outgrow a graph's width
            replays = eng.runner.graphs.replays if eng.runner.graphs is not None else 0
            return out, replays, eng.num_run_ahead

        want, _, _ = tokens(False, False)
        for run_ahead in (False, True):
            got, replays, ahead = tokens(True, run_ahead)
            assert replays >= 30 and (ahead >= 30) == run_ahead
            if dtype == "float32":
                assert got == want, f"captured steps (run_ahead={run_ahead}) changed the tokens"
            else:  # a logit within rounding may swap; the first steps after each capture must agree
                assert [g[:3] for g in got] == [w[:3] for w in want]
    finally:
        unregister_part("mixer", "toy_decay_state")


def _plain_layers(raw, tensors, ids, act, *, positions=None, feed_forward=None):
    """The plain model written out layer by layer, with the rotation's positions and the
    feed-forward open to replacement (tests of toy parts)."""
    ids_t = torch.as_tensor(ids, dtype=torch.long)
    pos = torch.arange(len(ids)) if positions is None else positions
    wf = {k: v.float() for k, v in tensors.items()}
    h = wf["model.embed_tokens.weight"][ids_t]
    eps = raw["rms_norm_eps"]
    for layer in range(raw["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        n = pm._round(pm.rmsnorm(h, wf[p + "input_layernorm.weight"], eps), act)
        a, _ = pm.attention_part(n, wf, p + "self_attn.", raw, pos, act_dtype=act)
        h = h + a
        n = pm._round(pm.rmsnorm(h, wf[p + "post_attention_layernorm.weight"], eps), act)
        ff = feed_forward(layer, n, wf) if feed_forward is not None else None
        h = h + (ff if ff is not None else pm.swiglu_part(n, wf, p + "mlp.", act_dtype=act))
    head = wf.get("lm_head.weight", wf["model.embed_tokens.weight"])
    return pm._round(pm.rmsnorm(h, wf["model.norm.weight"], eps), act) @ head.T


class Top1ExpertsFeedForward(Part):
    """A toy feed-forward with routing: a router picks one of E small SwiGLU experts per token
    (router logits and their softmax in fp32) and the expert's output is scaled by the router's
    probability.  The experts' products go through the framework's kernel table, with however
    many tokens each expert happens to get.  A test fixture, not a model of anything."""

    category = "feed_forward"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden, self.inter, self.experts = int(spec["hidden_size"]), int(spec["intermediate_size"]), int(spec["experts"])

    def param_specs(self):
        specs = {"router.weight": ParamSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            specs[f"experts.{e}.gate_up.weight"] = ParamSpec((2 * self.inter, self.hidden))
            specs[f"experts.{e}.down.weight"] = ParamSpec((self.hidden, self.inter))
        return specs

    def load(self, tensors):
        self.router = tensors["router.weight"].float()
        self.gate_up = [tensors[f"experts.{e}.gate_up.weight"].contiguous() for e in range(self.experts)]
        self.down = [tensors[f"experts.{e}.down.weight"].contiguous() for e in range(self.experts)]

    def kernel_groups(self):
        return (["norm", "gemm_f32"] if self.ctx.dtype == torch.float32
                else ["norm", "gemm_small_m", "gemm_stream", "gemm_tcgen05"])

    def forward(self, h, step):
        probs = torch.softmax(h.float() @ self.router.t(), dim=-1)
        weight, choice = probs.max(dim=-1)
        out = torch.zeros_like(h)
        for e in range(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel() == 0:
                continue
            x = h[rows].contiguous()
            mid = torch.empty((x.shape[0], self.inter), dtype=h.dtype, device=h.device)
            self.ops.gated_linear(x, self.gate_up[e], mid)
            y = self.ops.linear(mid, self.down[e])
            out[rows] = (y.float() * weight[rows, None]).to(h.dtype)
        return out


def case_toy_routed_feed_forward(dtype, ops, device):
    """Register, build and step a feed-forward with routing in layer 1, next to the dense one in
    layer 0: against the plain arithmetic, and the same logits however the tokens are cut."""
    cfg = TINY["A"]["config"]
    base = qwen3_spec(cfg)
    E, inter = 3, 48
    register_part("feed_forward", "toy_top1_experts", Top1ExpertsFeedForward)
    try:
        toy = PartSpec("toy_top1_experts", dict(hidden_size=cfg.hidden_size, intermediate_size=inter, experts=E))
        blocks = (base.blocks[0], PartSpec("pre_norm", {**base.blocks[1].params, "feed_forward": toy}))
        spec = ModelSpec(base.vocab_size, base.hidden_size, blocks, base.order, base.final_norm, True)
        model, tensors = _toy_model(spec, cfg, dtype, ops, device)
        assert "model.layers.1.mlp.router.weight" in tensors and "model.layers.1.mlp.gate_proj.weight" not in tensors
        ids = random_ids(cfg.vocab_size, 40, 41)
        whole, _ = _run_cut(model, cfg, ids, cuts=(40,))
        cut, _ = _run_cut(model, cfg, ids, cuts=(5, 2, 9, 1, 1, 30))
        act = torch.bfloat16 if dtype == "bfloat16" else None
        chosen = []

        def routed(layer, n, wf):
            if layer != 1:
                return None
            p = "model.layers.1.mlp."
            probs = torch.softmax(n.float() @ wf[p + "router.weight"].T, dim=-1)
            weight, choice = probs.max(dim=-1)
            chosen.append(choice)
            out = torch.zeros_like(n)
            for e in range(E):
                rows = choice == e
                gu = n[rows] @ wf[p + f"experts.{e}.gate_up.weight"].T
                g, u = pm._round(gu[:, :inter], act), pm._round(gu[:, inter:], act)
                mid = pm._round(g * torch.sigmoid(g) * u, act)
                y = pm._round(mid @ wf[p + f"experts.{e}.down.weight"].T, act)
                out[rows] = pm._round(y * weight[rows, None], act)
            return out

        want = _plain_layers(cfg.to_hf_config(), tensors, ids, act, feed_forward=routed)
        assert len(set(chosen[0].tolist())) == E, "the test wants every expert to get tokens"
        scale = max(1.0, float(want.abs().max()))
        if dtype == "float32":
            assert float((whole - want).abs().max()) <= 3e-5 * scale
            assert float((whole - cut).abs().max()) <= 3e-5 * scale
        else:  # a token whose two best experts are close may go the other way in bfloat16: compare most rows
            close_rows = ((whole - want).abs().amax(dim=1) <= 0.03 * scale).float().mean()
            assert float(close_rows) >= 0.9
            assert float(((whole - cut).abs().amax(dim=1) <= 0.03 * scale).float().mean()) >= 0.9
    finally:
        unregister_part("feed_forward", "toy_top1_experts")


class SlowedRotary(Part):
    """A toy position encoding: rotate-half rotary embedding whose angle grows `rate` times as
    fast as the position (rate < 1: positions squeezed together).  It hands the attention kernel
    its own tables; nothing else in the framework knows about it."""

    category = "position"
    style = "rotary"
    pairing = "half"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.dim, self.theta = int(spec["rotary_dim"]), float(spec["theta"])
        self.rate, self.max_positions = float(spec["rate"]), int(spec["max_positions"])
        self.pairing = spec.get("pairing", "half")

    def position_limit(self):
        return self.max_positions

    def kernel_groups(self):
        return ["rope_kv"]

    def rotation_tables(self):
        key = ("toy_slowed_rotary", self.dim, self.theta, self.rate, self.max_positions)
        if key not in self.ctx.shared:
            inv = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float) / self.dim))
            angle = (torch.arange(self.max_positions, dtype=torch.float) * self.rate)[:, None] * inv[None, :]
            self.ctx.shared[key] = (angle.cos().to(self.ctx.device), angle.sin().to(self.ctx.device))
        return self.ctx.shared[key]


def case_toy_position_encoding(dtype, ops, device):
    """Register a position encoding of the test's own and give it to the attention of both layers."""
    cfg = TINY["A"]["config"]
    base = qwen3_spec(cfg)
    rate = 0.25
    register_part("position", "toy_slowed_rotary", SlowedRotary)
    try:
        toy = PartSpec("toy_slowed_rotary", dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta, rate=rate,
                                                 max_positions=cfg.max_position_embeddings))
        blocks = tuple(
            PartSpec("pre_norm", {**b.params, "mixer": PartSpec("paged_attention", {**b["mixer"].params, "position": toy})})
            for b in base.blocks)
        spec = ModelSpec(base.vocab_size, base.hidden_size, blocks, base.order, base.final_norm, True)
        model, tensors = _toy_model(spec, cfg, dtype, ops, device)
        ids = random_ids(cfg.vocab_size, 40, 42)
        got, _ = _run_cut(model, cfg, ids)
        act = torch.bfloat16 if dtype == "bfloat16" else None
        raw = cfg.to_hf_config()
        want = _plain_layers(raw, tensors, ids, act, positions=torch.arange(len(ids), dtype=torch.float) * rate)
        ordinary = _plain_layers(raw, tensors, ids, act)
        scale = max(1.0, float(want.abs().max()))
        assert float((got - want).abs().max()) <= (3e-5 if dtype == "float32" else 0.03) * scale
        assert float((want - ordinary).abs().max()) > 1e-2, "the encoding has to matter for the test to mean anything"
    finally:
        unregister_part("position", "toy_slowed_rotary")


def case_interleaved_pairs_biases_and_capped_logits(dtype, ops, device):
    """Three seams as parameters, with toy parts: a position encoding that rotates neighbouring
    elements (2i, 2i + 1) instead of halves; projections with biases (q/k/v, o, down); a head
    whose logits are scaled and soft-capped.  Whole prompt, cut into portions, and decoded token
    by token (the decode kernel makes the newest token's q and k itself, with the same pairing)
    against plain arithmetic written out here."""
    cfg = TINY["D"]["config"]  # head size 64: bfloat16 decode steps take the fused split-KV kernel
    base = qwen3_spec(cfg)
    register_part("position", "toy_slowed_rotary", SlowedRotary)
    try:
        toy = PartSpec("toy_slowed_rotary", dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta, rate=1.0,
                                                 max_positions=cfg.max_position_embeddings, pairing="interleaved"))
        blocks = tuple(PartSpec("pre_norm", {
            **b.params,
            "mixer": PartSpec("paged_attention", {**b["mixer"].params, "position": toy, "qkv_bias": True, "o_bias": True}),
            "feed_forward": PartSpec("gated_mlp", {**b["feed_forward"].params, "down_bias": True})}) for b in base.blocks)
        spec = ModelSpec(base.vocab_size, base.hidden_size, blocks, base.order, base.final_norm, True,
                         logit_scale=0.5, logit_softcap=3.0)
        model, tensors = _toy_model(spec, cfg, dtype, ops, device)
        assert "model.layers.0.self_attn.q_proj.bias" in tensors and "model.layers.1.mlp.down_proj.bias" in tensors
        assert model.position_limit() == cfg.max_position_embeddings
        # the biases drawn by _toy_model are "vectors" around 1: make them ordinary small offsets
        for name in [n for n in tensors if n.endswith(".bias")]:
            tensors[name] = (tensors[name].float() - 1.0).to(torch.bfloat16)
        load_into(model, DictSource(tensors))
        ids = random_ids(cfg.vocab_size, 40, 43)
        whole, _ = _run_cut(model, cfg, ids, page_size=16, cuts=(40,))
        cut, _ = _run_cut(model, cfg, ids, page_size=16, cuts=(5, 2, 9, 1, 1, 1, 1, 30))
        act = torch.bfloat16 if dtype == "bfloat16" else None
        r = lambda x: pm._round(x, act)  # noqa: E731
        wf = {k: v.float() for k, v in tensors.items()}
        nq, nkv, D, eps = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps
        T = len(ids)
        cos, sin = pm.rope_tables(D, cfg.rope_theta, torch.arange(T))

        def rotate_neighbours(x):  # x [T, heads, D]: pair i = (2i, 2i + 1)
            x1, x2 = x[..., 0::2], x[..., 1::2]
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).flatten(-2)

        h = wf["model.embed_tokens.weight"][torch.as_tensor(ids)]
        for layer in range(cfg.num_hidden_layers):
            p = f"model.layers.{layer}."
            n = r(pm.rmsnorm(h, wf[p + "input_layernorm.weight"], eps))
            proj = lambda name: r(r(n @ wf[p + f"self_attn.{name}.weight"].T) + wf[p + f"self_attn.{name}.bias"])  # noqa: E731
            q, k, v = proj("q_proj").view(T, nq, D), proj("k_proj").view(T, nkv, D), proj("v_proj").view(T, nkv, D)
            q = r(rotate_neighbours(pm.rmsnorm(q, wf[p + "self_attn.q_norm.weight"], eps)))
            k = r(rotate_neighbours(pm.rmsnorm(k, wf[p + "self_attn.k_norm.weight"], eps)))
            ctx_ = r(pm.causal_attention(q, k, v, act_dtype=act))
            h = h + r(r(ctx_ @ wf[p + "self_attn.o_proj.weight"].T) + wf[p + "self_attn.o_proj.bias"])
            n = r(pm.rmsnorm(h, wf[p + "post_attention_layernorm.weight"], eps))
            g, u = n @ wf[p + "mlp.gate_proj.weight"].T, n @ wf[p + "mlp.up_proj.weight"].T
            if act is not None:
                g, u = r(g), r(u)
            m = r(g * torch.sigmoid(g) * u)
            h = h + r(r(m @ wf[p + "mlp.down_proj.weight"].T) + wf[p + "mlp.down_proj.bias"])
        logits = r(pm.rmsnorm(h, wf["model.norm.weight"], eps)) @ wf["model.embed_tokens.weight"].T
        want = 3.0 * torch.tanh(0.5 * logits / 3.0)
        tol = 3e-5 if dtype == "float32" else 0.03 * max(1.0, float(want.abs().max()))
        assert float((whole - want).abs().max()) <= tol and float((cut - want).abs().max()) <= tol
        assert float(want.abs().max()) < 3.0 and float((want - 0.5 * logits).abs().max()) > 1e-3, "the cap has to bite"
    finally:
        unregister_part("position", "toy_slowed_rotary")
