"""Engine-versus-plain comparisons, written once and run twice: on the CPU with the torch
statements of the kernels (tests/emulated_ops.py) in place of the kernel table -- that
checks batching, cache and scheduling -- and on the GPU with the real kernels, in
float32 and bfloat16."""

from __future__ import annotations


import torch

import plain_model as pm
from helpers import (TINY, first_mismatch, make_model_dir, peak_live, peak_tokens, random_ids, run_trace,
                     trace_mixed, trace_portions, trace_tail_decode, trace_whole)
from qwen3_runtime_b200.engine.factory import build_engine, build_runtime, load_model

# Tolerances, fixed in advance.  float32: the engine and the plain implementation do the
# same arithmetic in different orders; observed differences are a few 1e-6 on logits of
# magnitude ~4.  bfloat16: activations are rounded to 8 bits of mantissa between kernels, which
# moves the logits; how far is measured for every case, as the distance between the plain
# implementation with bfloat16 activations and the plain implementation in float32 on the same
# tokens (the rounding noise of that case).  The engine rounds at the same places, with sums in
# other orders, so its logits are another draw of the same noise: it has to stay within
# BF16_NOISE_FACTOR times the measured noise of the plain bfloat16 logits.  (On the two golden
# models the reference's own bfloat16 model lies 0.027..0.049 from its float32 logits, the plain
# bfloat16 logits 0.019..0.036, and the two 0.031..0.046 from each other: tests/test_plain_model.py.)
TOL_F32 = 3e-5
BF16_NOISE_FACTOR = 3.0


class Expected(dict):
    """``{request: plain logits}`` with the tolerance that goes with them."""

    tol: float = 0.0
    noise: float | None = None


def tolerance_f32(scale: float) -> float:
    return TOL_F32 * max(1.0, scale / 4.0)


def bf16_tolerance(rounded, exact) -> tuple[float, float]:
    """(tolerance, noise) from the plain logits with bfloat16 activations and in float32."""
    noise = max(float((a.double() - b.double()).abs().max()) for a, b in zip(rounded, exact))
    return BF16_NOISE_FACTOR * noise, noise


def check_greedy_within_rounding(raw, w, prompt, tokens, what, dtype="bfloat16"):
    """bfloat16 greedy tokens: two logits within rounding of each other may swap, after which a
    recomputed sequence goes another way, so whole sequences are not compared.  Instead every
    token is checked at its own place: given the tokens the engine chose before it, the plain
    model's logit for it is the largest, or below the largest by no more than the two logits'
    tolerances together."""
    rows = pm.forward_logits(raw, w, list(prompt) + list(tokens[:-1]),
                             rows=list(range(len(prompt) - 1, len(prompt) + len(tokens) - 1)),
                             act_dtype=torch.bfloat16 if dtype == "bfloat16" else None)
    assert rows.shape[0] == len(tokens)
    if dtype == "bfloat16":  # two logits may each be off by the tolerance, in opposite directions
        exact = pm.forward_logits(raw, w, list(prompt) + list(tokens[:-1]),
                                  rows=list(range(len(prompt) - 1, len(prompt) + len(tokens) - 1)))
        tol = 2 * bf16_tolerance([rows], [exact])[0]
    else:
        tol = 2 * tolerance_f32(float(rows.abs().max()))
    for i, tok in enumerate(tokens):
        gap = float(rows[i].max() - rows[i][tok])
        assert gap <= tol, f"{what}: token {i} ({tok}) is {gap:.3g} below the plain argmax (allowed {tol:.3g})"


def plain_logits(folder, requests, dtype, rows=None):
    """The plain implementation's logits for every request (``rows``: {request: positions}, default
    all) and the tolerance the engine is held to."""
    raw, w = pm.read_model_dir(folder)
    return expected_logits(raw, w, requests, dtype, rows)


def expected_logits(raw, w, requests, dtype, rows=None):
    pick = (lambda rid: None) if rows is None else (lambda rid: rows[rid])
    exact = {rid: pm.forward_logits(raw, w, toks, rows=pick(rid)) for rid, toks in requests.items()}
    if dtype == "float32":
        out = Expected(exact)
        out.tol = tolerance_f32(max(float(v.abs().max()) for v in exact.values()))
        return out
    out = Expected({rid: pm.forward_logits(raw, w, toks, rows=pick(rid), act_dtype=torch.bfloat16)
                    for rid, toks in requests.items()})
    out.tol, out.noise = bf16_tolerance(list(out.values()), [exact[rid] for rid in out])
    return out


def requests_for(name, lengths, seed=0):
    vocab = TINY[name]["config"].vocab_size
    return {f"r{i}": random_ids(vocab, n, seed * 100 + i) for i, n in enumerate(lengths)}


def make_runtime(folder, name, dtype, ops, device, *, num_pages, max_live=4, cuda_graph=False):
    model, cfg, _ = load_model(folder, dtype=dtype, device=device, ops=ops)
    rt = build_runtime(model, block_size=TINY[name]["page_size"], num_kv_blocks=num_pages, max_num_seqs=max_live,
                       cuda_graph=cuda_graph)
    assert rt.max_positions == cfg.max_position_embeddings  # taken from the model's own position part
    return rt


def check_against(got, want, dtype, what, positions=None):
    """``positions``: how many logit rows ``got`` has to hold (default: every position of ``want``)."""
    scale = max(float(v.abs().max()) for v in want.values())
    tol = want.tol
    bad = first_mismatch(got, want, tol)
    assert bad is None, (f"{what}: request {bad[0]} position {bad[1]} differs by {bad[2]:.3g} "
                         f"(tolerance {tol:.3g}, logits up to {scale:.3g}, rounding noise {want.noise})")
    if want.noise:
        from helpers import max_abs_diff

        print(f"{what}: worst difference {max_abs_diff(got, want) / want.noise:.2f} x the rounding noise "
              f"{want.noise:.3g} (allowed {BF16_NOISE_FACTOR})")
    n = sum(len(v) for v in got.values())
    expect = sum(v.shape[0] for v in want.values()) if positions is None else positions
    assert n == expect, f"{what}: {n} positions compared, {expect} expected"


def case_four_schedules(tmp_path, name, dtype, ops, device, lengths=(100, 37, 61, 150, 45, 83)):
    """Whole / tail decoded one by one / changing portions / mixed with page reuse, each
    against the plain implementation, and against the whole-sequence run."""
    folder = make_model_dir(tmp_path, name)
    requests = requests_for(name, lengths)
    want = plain_logits(folder, requests, dtype)
    ps = TINY[name]["page_size"]
    results = {}
    for kind, steps in (("whole", trace_whole(requests)), ("tail", trace_tail_decode(requests)),
                        ("portions", trace_portions(requests, seed=1)), ("mixed", trace_mixed(requests, seed=2))):
        # a pool that holds exactly the peak: pages are returned and handed out again
        pages = peak_tokens(steps, 64) // ps
        rt = make_runtime(folder, name, dtype, ops, device, num_pages=pages)
        got = run_trace(rt, steps, poison=True)
        check_against(got, want, dtype, f"{name} {dtype} {kind}")
        assert rt.cache.num_free_pages == rt.cache.num_pages
        results[kind] = got
    # cutting and batching change nothing beyond rounding
    whole = {rid: torch.stack([rows[p] for p in sorted(rows)]) for rid, rows in results["whole"].items()}
    scale = max(float(v.abs().max()) for v in whole.values())
    if dtype == "float32":
        # the float32 kernels reduce in an order that depends on the position only: bit-identical
        cut_tol = 0.0 if getattr(ops, "name", "").startswith("cuda") else tolerance_f32(scale)
    else:
        cut_tol = want.tol
    for kind in ("tail", "portions", "mixed"):
        bad = first_mismatch(results[kind], whole, cut_tol)
        assert bad is None, f"{name} {dtype} {kind} vs whole: request {bad[0]} position {bad[1]} differs by {bad[2]:.3g}"
    return results


def case_many_live(tmp_path, name, dtype, ops, device, max_live, *, cuda_graph=False, seed=0):
    """The mixed schedule with ``max_live`` requests live at once (portions of some beside single
    tokens of many others), in a pool of exactly the peak so that pages are handed on, every
    returned page poisoned; and the same requests' last tokens decoded together, one token per
    request and step, which is the batch a captured decode step of that size serves."""
    import random as _random

    folder = make_model_dir(tmp_path, name)
    rnd = _random.Random(1000 * max_live + seed)
    requests = requests_for(name, [rnd.randint(14, 60) for _ in range(2 * max_live + 3)], seed=seed + 20)
    want = plain_logits(folder, requests, dtype)
    ps = TINY[name]["page_size"]
    steps = trace_mixed(requests, seed=seed + 3, max_live=max_live, admit=0.97)
    assert peak_live(steps) == max_live, f"the trace was meant to hold {max_live} requests at once"
    rt = make_runtime(folder, name, dtype, ops, device, num_pages=peak_tokens(steps, 64) // ps, max_live=max_live,
                      cuda_graph=cuda_graph)
    got = run_trace(rt, steps, poison=True)
    check_against(got, want, dtype, f"{name} {dtype} mixed with {max_live} live")
    assert rt.cache.num_free_pages == rt.cache.num_pages
    # max_live requests decoding side by side: prompts whole (one step each), then 6 steps of
    # one token for every request at once
    batch = dict(list(requests.items())[:max_live])
    together = []
    for i, (rid, toks) in enumerate(batch.items()):
        head = len(toks) - 6
        together.append({"step": i, "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
    for j in range(6):
        together.append({"step": max_live + j, "end": list(batch) if j == 5 else [],
                         "entries": [{"id": rid, "tokens": [toks[len(toks) - 6 + j]], "want": [0]}
                                     for rid, toks in batch.items()]})
    rt = make_runtime(folder, name, dtype, ops, device, num_pages=peak_tokens(together, 64) // ps, max_live=max_live,
                      cuda_graph=cuda_graph)
    got = run_trace(rt, together)
    check_against(got, want, dtype, f"{name} {dtype} {max_live} requests decoding together", positions=7 * max_live)
    if cuda_graph and rt.runner.graphs is not None and max_live <= max(rt.runner.graphs.sizes):
        assert rt.runner.graphs.replays == 6, "the six decode steps were meant to replay a captured graph"
    return got


def case_mixed_lengths_decoding_together(tmp_path, name, dtype, ops, device, *, cuda_graph=True,
                                         lengths=(790, 57, 300, 90, 48, 520), tail=40):
    """Requests of very different lengths decoding side by side: the split-KV kernel cuts the
    longest into the step's slice count and the shorter ones into fewer slices; the count is chosen
    from the lengths of the moment, changes while the requests grow, and with captured steps each
    value has a graph of its own."""
    folder = make_model_dir(tmp_path, name)
    requests = requests_for(name, lengths, seed=41)
    want = plain_logits(folder, requests, dtype)
    ps = TINY[name]["page_size"]
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        head = len(toks) - tail
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
    for j in range(tail):
        steps.append({"step": len(requests) + j, "end": list(requests) if j == tail - 1 else [],
                      "entries": [{"id": rid, "tokens": [toks[len(toks) - tail + j]], "want": [0]}
                                  for rid, toks in requests.items()]})
    rt = make_runtime(folder, name, dtype, ops, device, num_pages=peak_tokens(steps, 64) // ps + 1,
                      max_live=len(requests), cuda_graph=cuda_graph)
    got = run_trace(rt, steps)
    check_against(got, want, dtype, f"{name} {dtype} mixed lengths decoding together",
                  positions=(tail + 1) * len(requests))
    return rt


def case_greedy_many(tmp_path, name, dtype, ops, device, num_requests, *, cuda_graph=True, max_tokens=6):
    """Greedy generation of ``num_requests`` requests side by side under the scheduler (a token
    budget that cuts the prompts, a decode batch of that size, captured or not)."""
    folder = make_model_dir(tmp_path, name)
    raw, w = pm.read_model_dir(folder)
    ps = TINY[name]["page_size"]
    prompts = list(requests_for(name, [5 + (7 * i) % 23 for i in range(num_requests)], seed=31).values())
    act = torch.bfloat16 if dtype == "bfloat16" else None
    eng = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps,
                       num_kv_blocks=num_requests * (-(-40 // ps) + 1), max_num_seqs=num_requests,
                       max_num_batched_tokens=48, cuda_graph=cuda_graph)
    got = eng.generate_batch(prompts, max_tokens=max_tokens)
    assert eng.cache.num_free_pages == eng.cache.num_pages
    for p, toks in zip(prompts, got):
        if dtype == "float32":
            assert toks == pm.greedy_generate(raw, w, p, max_tokens, act_dtype=act)
        else:
            check_greedy_within_rounding(raw, w, p, toks, f"{name} {num_requests} side by side")
    return eng


def case_first_tokens(tmp_path, name, dtype, ops, device):
    """The first tokens of a sequence: length-1 and length-2 requests, and position 0 alone."""
    folder = make_model_dir(tmp_path, name)
    requests = requests_for(name, (1, 2, 3, 1), seed=3)
    want = plain_logits(folder, requests, dtype)
    rt = make_runtime(folder, name, dtype, ops, device, num_pages=16)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:1], "want": [0]} for r, t in requests.items()], "end": []},
             {"step": 1, "entries": [{"id": r, "tokens": t[1:], "want": list(range(len(t) - 1))}
                                     for r, t in requests.items() if len(t) > 1], "end": list(requests)}]
    check_against(run_trace(rt, steps), want, dtype, f"{name} {dtype} first tokens")


def case_long_decode(tmp_path, name, dtype, ops, device, prompt=5, total=300):
    """Long decoding: a short prompt, then hundreds of single-token steps across many pages."""
    folder = make_model_dir(tmp_path, name)
    requests = requests_for(name, (total,), seed=4)
    want = plain_logits(folder, requests, dtype)
    rt = make_runtime(folder, name, dtype, ops, device, num_pages=-(-total // TINY[name]["page_size"]) + 1)
    got = run_trace(rt, trace_tail_decode(requests, tail=total - prompt), check=False)
    check_against(got, want, dtype, f"{name} {dtype} long decode")


def case_greedy_generation(tmp_path, name, dtype, ops, device, *, cuda_graph=False):
    """Greedy generation through the engine equals recomputing the whole sequence for every token
    with the plain implementation -- alone, batched, and with so few pages that a request is
    preempted and recomputed."""
    folder = make_model_dir(tmp_path, name)
    raw, w = pm.read_model_dir(folder)
    ps = TINY[name]["page_size"]
    prompts = list(requests_for(name, (7, 19, 5, 13), seed=5).values())
    act = torch.bfloat16 if dtype == "bfloat16" else None
    want = [pm.greedy_generate(raw, w, p, 8, act_dtype=act) for p in prompts]
    eng = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps, num_kv_blocks=64, max_num_seqs=4,
                       max_num_batched_tokens=6, cuda_graph=cuda_graph)
    alone = [eng.generate(p, max_tokens=8) for p in prompts]
    batched = eng.generate_batch(prompts, max_tokens=8)
    assert eng.cache.num_free_pages == eng.cache.num_pages
    # so few pages that they run out: two prompts that fill the pool exactly, so that neither can
    # take its first decoded token; the younger is preempted and later recomputed from its start
    vocab = TINY[name]["config"].vocab_size
    tight_prompts = [random_ids(vocab, 2 * ps, 77), random_ids(vocab, ps, 78)]
    tight_want = [pm.greedy_generate(raw, w, p, 8, act_dtype=act) for p in tight_prompts]
    tight = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps, num_kv_blocks=3,
                         max_num_seqs=4, max_num_batched_tokens=64, cuda_graph=cuda_graph)
    squeezed = tight.generate_batch(tight_prompts, max_tokens=8)
    assert tight.scheduler.num_preemptions >= 1, "the tight pool was meant to force a preemption"
    assert tight.cache.num_free_pages == tight.cache.num_pages
    roomy = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps, num_kv_blocks=64,
                         max_num_seqs=4, max_num_batched_tokens=64, cuda_graph=cuda_graph)
    unsqueezed = roomy.generate_batch(tight_prompts, max_tokens=8)
    assert roomy.scheduler.num_preemptions == 0
    if dtype == "float32":
        assert alone == want and batched == want and squeezed == tight_want and unsqueezed == tight_want
    else:
        # greedy ids may flip where two logits are within bfloat16 rounding of each other
        for p, toks in zip(prompts, alone):
            check_greedy_within_rounding(raw, w, p, toks, f"{name} alone")
        for p, toks in zip(tight_prompts, squeezed):
            check_greedy_within_rounding(raw, w, p, toks, f"{name} squeezed")
        assert batched == alone and squeezed == unsqueezed
    return alone


def case_temperature_sampling(tmp_path, name, dtype, ops, device):
    """Temperature sampling with a seed: the same tokens alone and in a batch, and equal to
    the plain implementation drawing with the same uniform numbers."""
    from qwen3_runtime_b200 import SamplingParams
    from qwen3_runtime_b200.engine.request import make_generator

    folder = make_model_dir(tmp_path, name)
    raw, w = pm.read_model_dir(folder)
    ps = TINY[name]["page_size"]
    prompts = list(requests_for(name, (5, 13, 30), seed=6).values())
    sp = [SamplingParams(temperature=0.8, seed=40 + i) for i in range(3)]
    eng = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps, num_kv_blocks=64, max_num_seqs=3,
                       max_num_batched_tokens=6, cuda_graph=False)
    batched = eng.generate_batch(prompts, max_tokens=8, sampling=sp)
    alone = [eng.generate(p, max_tokens=8, sampling=s) for p, s in zip(prompts, sp)]
    assert batched == alone
    if dtype != "float32":
        return
    for p, s, got in zip(prompts, sp, alone):
        gen = make_generator(s.seed)
        ids = list(p)
        for tok in got:
            u = float(torch.rand((), dtype=torch.float32, generator=gen))
            probs = pm.temperature_probs(pm.forward_logits(raw, w, ids)[-1], s.temperature)
            cdf = probs.double().cumsum(0)
            lo = float(cdf[tok - 1]) if tok > 0 else 0.0
            # the chosen token's interval of the CDF contains u (up to float32 rounding of the sums)
            assert lo - 1e-5 <= u <= float(cdf[tok]) + 1e-5, (tok, u, lo, float(cdf[tok]))
            ids.append(tok)


def case_run_ahead(tmp_path, name, dtype, ops, device, *, cuda_graph=False):
    """The engine puts the next decode step on the device before it reads the tokens of the last
    one.  The tokens are those of the engine that does not, step by step: with requests of
    different lengths, a stop token that ends one of them while a step is already running for
    it, seeded temperature sampling, a request that arrives later, one that is aborted, and so
    few pages that a request is preempted."""
    from qwen3_runtime_b200 import SamplingParams

    folder = make_model_dir(tmp_path, name)
    ps = TINY[name]["page_size"]
    vocab = TINY[name]["config"].vocab_size
    prompts = list(requests_for(name, (7, 19, 5, 13), seed=8).values())

    def engine(run_ahead, pages=64, eos=None):
        return build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps, num_kv_blocks=pages,
                            max_num_seqs=4, max_num_batched_tokens=16, cuda_graph=cuda_graph, run_ahead=run_ahead,
                            eos_token_id=eos)

    def scenario(eng, stop=(), late=True, abort=False):
        lengths = (12, 5, 9, 12)
        sampling = [SamplingParams(), SamplingParams(temperature=0.9, seed=3), SamplingParams(),
                    SamplingParams(temperature=0.7, top_k=20, seed=4)]
        ids = [eng.add_request(p, max_tokens=n, sampling=s, ignore_eos=not stop, stop_token_ids=tuple(stop))
               for p, n, s in zip(prompts[:3], lengths, sampling)]
        reqs = [eng.get_request(i) for i in ids]
        steps = []
        for i in range(200):
            if late and i == 6:  # arrives while the others decode
                ids.append(eng.add_request(prompts[3], max_tokens=lengths[3], sampling=sampling[3]))
                reqs.append(eng.get_request(ids[-1]))
            if abort and i == 9 and reqs[0].status.name != "FINISHED":
                eng.abort_request(ids[0])
            out = eng.step()
            if not out:
                break
            first = ids[0]
            steps.append(sorted((rid - first, tok, fin) for rid, tok, fin in out))
        assert eng.is_finished() and eng.cache.num_free_pages == eng.cache.num_pages
        eng.cache.check_invariants()
        return steps, [r.output_token_ids for r in reqs], [r.finish_reason for r in reqs]

    # (1) plain: lengths differ, one request arrives late
    want = scenario(engine(False))
    eng = engine(True)
    got = scenario(eng)
    assert got == want
    assert eng.num_run_ahead >= 4, "decode steps were meant to run ahead"
    assert got[2] == ["length"] * 4
    # (2) a stop token: the third output token of the first request (it decodes greedily)
    stop = [want[1][0][2]]
    want_stop = scenario(engine(False), stop=stop)
    eng = engine(True)
    got_stop = scenario(eng, stop=stop)
    assert got_stop == want_stop and "stop" in got_stop[2] and eng.num_run_ahead >= 1
    assert len(got_stop[1][0]) <= 3
    # (3) aborted while a step may be running for it
    want_abort = scenario(engine(False), abort=True)
    got_abort = scenario(engine(True), abort=True)
    assert got_abort == want_abort and got_abort[2][0] == "abort"
    # (4) so few pages that somebody is preempted: never runs ahead into a pool that cannot take it
    tight_prompts = [random_ids(vocab, 2 * ps, 77), random_ids(vocab, ps, 78)]

    def squeeze(run_ahead):
        eng = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps, num_kv_blocks=3, max_num_seqs=4,
                           max_num_batched_tokens=64, cuda_graph=cuda_graph, run_ahead=run_ahead)
        out = eng.generate_batch(tight_prompts, max_tokens=8)
        assert eng.scheduler.num_preemptions >= 1 and eng.cache.num_free_pages == eng.cache.num_pages
        return out

    assert squeeze(True) == squeeze(False)
    # (5) long enough to cross many pages and to outgrow a captured block-table width
    def long_run(run_ahead):
        eng = engine(run_ahead)
        out = eng.generate_batch(prompts[:2], max_tokens=150)
        assert eng.cache.num_free_pages == eng.cache.num_pages
        return out, eng.num_run_ahead

    (long_ahead, n_ahead), (long_plain, _) = long_run(True), long_run(False)
    assert long_ahead == long_plain and n_ahead >= 140
    # (6) an engine that is left with a step in flight (everybody stopped) starts afresh
    eng = engine(True)
    first = eng.generate(prompts[0], max_tokens=6, ignore_eos=False, stop_token_ids=(want[1][0][2],))
    again = eng.generate(prompts[2], max_tokens=6)
    assert first == want[1][0][:len(first)] and first[-1] == want[1][0][2] and again == want[1][2][:6], (first, again, want[1])


def case_run_ahead_random(tmp_path, name, dtype, ops, device, seed, *, cuda_graph=False):
    """Random arrivals, lengths, stop tokens, samplers and aborts: the engine that runs ahead gives
    every request the tokens and the end that the engine that does not gives it, and every page
    back.  The steps themselves may differ: a request that arrives while a step is already running
    ahead joins one step later (so an abort at a fixed step cuts it one token earlier)."""
    import random as _random

    from qwen3_runtime_b200 import SamplingParams

    folder = make_model_dir(tmp_path, name)
    ps = TINY[name]["page_size"]
    vocab = TINY[name]["config"].vocab_size
    rnd = _random.Random(seed)
    plan = []
    for i in range(rnd.randint(3, 6)):
        kind = rnd.choice(["greedy", "greedy", "temperature", "top_k", "penalty"])
        sampling = {"greedy": SamplingParams(),
                    "temperature": SamplingParams(temperature=0.8, seed=100 + i),
                    "top_k": SamplingParams(temperature=0.9, top_k=rnd.randint(2, 30), seed=200 + i),
                    "penalty": SamplingParams(repetition_penalty=1.3)}[kind]
        plan.append(dict(arrive=rnd.randint(0, 12), prompt=random_ids(vocab, rnd.randint(1, 40), 1000 * seed + i),
                         max_tokens=rnd.randint(1, 25), sampling=sampling,
                         stop=tuple(rnd.sample(range(vocab), rnd.randint(0, vocab // 8))) if rnd.random() < 0.5 else (),
                         abort=rnd.randint(3, 30) if rnd.random() < 0.25 else None))
    pages = rnd.choice([6, 12, 64])
    budget = rnd.choice([8, 16, 64])
    seqs = rnd.choice([2, 4])

    def run(run_ahead):
        eng = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=ps, num_kv_blocks=pages,
                           max_num_seqs=seqs, max_num_batched_tokens=budget, cuda_graph=cuda_graph,
                           run_ahead=run_ahead)
        reqs = {}
        for step in range(400):
            for i, p in enumerate(plan):
                if p["arrive"] == step and eng.cache.fits_at_all(len(p["prompt"]) + p["max_tokens"]):
                    rid = eng.add_request(p["prompt"], max_tokens=p["max_tokens"], sampling=p["sampling"],
                                          ignore_eos=not p["stop"], stop_token_ids=p["stop"])
                    reqs[i] = eng.get_request(rid)
                if p["abort"] == step and i in reqs:
                    eng.abort_request(reqs[i].request_id)
            if not eng.step() and step > max(p["arrive"] for p in plan):
                break
        assert eng.is_finished() and eng.cache.num_free_pages == eng.cache.num_pages
        eng.cache.check_invariants()
        return {i: (r.output_token_ids, r.finish_reason) for i, r in reqs.items()}, eng.num_run_ahead

    plain, none = run(False)
    ahead, count = run(True)
    assert none == 0 and plain.keys() == ahead.keys()
    for i in plain:
        (toks_p, why_p), (toks_a, why_a) = plain[i], ahead[i]
        if "abort" in (why_p, why_a):
            n = min(len(toks_p), len(toks_a))
            assert toks_p[:n] == toks_a[:n] and abs(len(toks_p) - len(toks_a)) <= 1, (seed, i, toks_p, toks_a)
        else:
            assert (toks_p, why_p) == (toks_a, why_a), (seed, i, plain[i], ahead[i])
    return count
