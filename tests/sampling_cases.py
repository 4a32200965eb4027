"""Sampler behaviour, run on the CPU (torch statements of the kernels) and on the GPU (kernels).
What is checked follows qwen3-runtime's tests/cpu/test_sampling.py:23-260: greedy ties, temperature
0 is greedy, top_k=1 is argmax, seeds, logit bias, penalties, min_p, top_p."""

from __future__ import annotations

from types import SimpleNamespace

import torch

from qwen3_runtime_b200 import SamplingParams
from qwen3_runtime_b200.engine.request import make_generator
from qwen3_runtime_b200.sampling.sampler import Sampler


def req(params, token_ids=(1, 2, 3)):
    return SimpleNamespace(sampling=params, rng=make_generator(params.seed), token_ids=list(token_ids), logprobs=[])


def rows(R, V, seed, device, scale=2.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(R, V, generator=g) * scale).to(device)


def case_greedy_and_equivalents(ops, device):
    s = Sampler(ops, device)
    x = rows(4, 301, 1, device)
    x[0, 7] = x[0, 200] = 50.0
    want = x.argmax(-1).tolist()
    want[0] = 7  # lowest id on ties
    assert s.sample(x, [req(SamplingParams()) for _ in range(4)])[0] == want
    assert s.sample(x, [req(SamplingParams(temperature=0.0, top_k=5, top_p=0.3)) for _ in range(4)])[0] == want
    assert s.sample(x, [req(SamplingParams(temperature=0.9, top_k=1, seed=i)) for i in range(4)])[0] == want
    toks, lps = s.sample(x, [req(SamplingParams(logprobs=True)) for _ in range(4)])
    ref = torch.log_softmax(x.float().cpu(), -1)
    assert all(abs(lp - float(ref[i, t])) < 1e-4 for i, (t, lp) in enumerate(zip(toks, lps)))


def case_seeded_draws(ops, device):
    s = Sampler(ops, device)
    x = rows(3, 4099, 2, device)
    a = s.sample(x, [req(SamplingParams(temperature=0.8, seed=5 + i)) for i in range(3)])[0]
    b = s.sample(x, [req(SamplingParams(temperature=0.8, seed=5 + i)) for i in range(3)])[0]
    c = s.sample(x, [req(SamplingParams(temperature=0.8, seed=50 + i)) for i in range(3)])[0]
    assert a == b and a != c
    # a request keeps its generator: consecutive draws differ but replay identically
    r1, r2 = req(SamplingParams(temperature=1.5, seed=9)), req(SamplingParams(temperature=1.5, seed=9))
    seq1 = [s.sample(x[:1], [r1])[0][0] for _ in range(6)]
    seq2 = [s.sample(x[:1], [r2])[0][0] for _ in range(6)]
    assert seq1 == seq2 and len(set(seq1)) > 1
    # greedy and sampling rows side by side
    mixed = s.sample(x, [req(SamplingParams()), req(SamplingParams(temperature=0.8, seed=6)), req(SamplingParams())])[0]
    assert mixed[0] == int(x[0].argmax()) and mixed[2] == int(x[2].argmax()) and mixed[1] == a[1]


def case_filters_restrict_the_support(ops, device):
    s = Sampler(ops, device)
    V = 301
    x = rows(1, V, 3, device)
    order = torch.argsort(x[0].cpu(), descending=True)
    probs = torch.softmax(x[0].double().cpu() / 1.3, -1)
    for trial in range(40):
        t = s.sample(x, [req(SamplingParams(temperature=1.3, top_k=5, seed=trial))])[0][0]
        assert t in order[:5].tolist()
    # nucleus: a token is kept iff the mass ranked before it is <= top_p
    cum_before = probs[order].cumsum(0) - probs[order]
    nucleus = set(order[cum_before <= 0.5].tolist())
    seen = {s.sample(x, [req(SamplingParams(temperature=1.3, top_p=0.5, seed=trial))])[0][0] for trial in range(60)}
    assert seen <= nucleus and len(seen) > 1
    # min_p: nothing below min_p * p_max
    allowed = set(torch.nonzero(probs >= 0.2 * probs.max()).flatten().tolist())
    seen = {s.sample(x, [req(SamplingParams(temperature=1.3, min_p=0.2, seed=trial))])[0][0] for trial in range(60)}
    assert seen <= allowed
    # the input logits are not modified
    before = x.clone()
    s.sample(x, [req(SamplingParams(temperature=0.7, top_k=3, top_p=0.9, min_p=0.05, seed=1))])
    assert torch.equal(x, before)


def case_bias_and_penalties(ops, device):
    s = Sampler(ops, device)
    V = 64
    x = rows(2, V, 4, device, scale=1.0)
    top = int(x[0].argmax())
    forced = (top + 5) % V
    assert s.sample(x[:1], [req(SamplingParams(logit_bias={forced: 100.0}))])[0][0] == forced
    # repetition penalty pushes the argmax down when it was already generated
    second = int(torch.topk(x[0], 2).indices[1])
    assert s.sample(x[:1], [req(SamplingParams(repetition_penalty=50.0), token_ids=[top, top])])[0][0] != top
    # presence / frequency: subtract per seen token / per occurrence (checked on the processed row)
    r = req(SamplingParams(presence_penalty=0.5, frequency_penalty=0.25, repetition_penalty=2.0), token_ids=[3, 3, 9])
    out = s._process(x[:1], [r], [0])[0].cpu()
    want = x[0].cpu().clone()
    for tok, cnt in ((3, 2), (9, 1)):
        v = want[tok]
        v = v / 2.0 if v > 0 else v * 2.0
        want[tok] = v - 0.5 - 0.25 * cnt
    assert float((out - want).abs().max()) < 1e-6
    assert second != top
