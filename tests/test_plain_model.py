"""The plain implementation against the reference's own model code (golden files made by
tests/golden/make_golden.py) and against itself."""

from pathlib import Path

import torch
from safetensors.torch import load_file

import plain_model as pm
from helpers import make_model_dir

GOLDEN = Path(__file__).parent / "golden"


def _golden(name):
    return load_file(str(GOLDEN / f"tiny_{name}.safetensors"))


def test_plain_logits_match_reference_model(tmp_path):
    for name in ("A", "B"):
        raw, w = pm.read_model_dir(make_model_dir(tmp_path, name))
        g = _golden(name)
        i = 0
        while f"prompt{i}.ids" in g:
            ids = g[f"prompt{i}.ids"].tolist()
            got = pm.forward_logits(raw, w, ids)
            torch.testing.assert_close(got, g[f"prompt{i}.logits"], atol=1e-5, rtol=1e-5)
            i += 1
        assert i >= 2


def test_plain_greedy_matches_reference_engine(tmp_path):
    for name in ("A", "B"):
        raw, w = pm.read_model_dir(make_model_dir(tmp_path, name))
        g = _golden(name)
        i = 0
        while f"prompt{i}.ids" in g:
            ids = g[f"prompt{i}.ids"].tolist()
            assert pm.greedy_generate(raw, w, ids, 8) == g[f"prompt{i}.greedy"].tolist()
            i += 1


def test_plain_bfloat16_against_the_reference_model_in_bfloat16(tmp_path):
    """The reference converted to bfloat16 (``model.to(bfloat16)``) also keeps its residual stream in
    bfloat16 (layers/ops.py:28-37); the plain implementation with ``act_dtype=bfloat16`` rounds
    where this engine stores and keeps the residual sum in float32.  Measured here, on the
    reference's own logits: both are rounding-noise away from the float32 logits, the plain
    variant no further than the reference's own, and they are as far from each other as two
    draws of that noise are."""
    worst = dict(ref=0.0, plain=0.0, apart=0.0)
    for name in ("A", "B"):
        raw, w = pm.read_model_dir(make_model_dir(tmp_path, name))
        g = _golden(name)
        i = 0
        while f"prompt{i}.ids" in g:
            ids = g[f"prompt{i}.ids"].tolist()
            exact, ref16 = g[f"prompt{i}.logits"], g[f"prompt{i}.logits_bf16"]
            plain16 = pm.forward_logits(raw, w, ids, act_dtype=torch.bfloat16)
            ref_err = float((ref16 - exact).abs().max())
            plain_err = float((plain16 - exact).abs().max())
            apart = float((plain16 - ref16).abs().max())
            scale = float(exact.abs().max())
            assert 0.002 * scale < ref_err < 0.02 * scale      # bfloat16 noise: about a percent of the range
            assert plain_err <= 1.1 * ref_err                  # the float32 residual sum is no worse
            assert apart <= ref_err + plain_err and apart <= 1.5 * ref_err
            worst = dict(ref=max(worst["ref"], ref_err), plain=max(worst["plain"], plain_err),
                         apart=max(worst["apart"], apart))
            i += 1
    print("bfloat16 distances from the float32 logits: reference", worst["ref"], "plain", worst["plain"],
          "between them", worst["apart"])


def test_float64_agrees_with_float32(tmp_path):
    raw, w = pm.read_model_dir(make_model_dir(tmp_path, "C"))
    ids = list(range(3, 40))
    a = pm.forward_logits(raw, w, ids)
    b = pm.forward_logits(raw, w, ids, compute=torch.float64)
    assert float((a.double() - b).abs().max()) < 1e-4


def test_causality(tmp_path):
    """Logits at a position do not change when later tokens change."""
    raw, w = pm.read_model_dir(make_model_dir(tmp_path, "A"))
    a = pm.forward_logits(raw, w, [5, 6, 7, 8, 9, 10])
    b = pm.forward_logits(raw, w, [5, 6, 7, 8, 200, 201])
    torch.testing.assert_close(a[:4], b[:4], atol=1e-6, rtol=0)
    assert float((a[4:] - b[4:]).abs().max()) > 1e-3


def test_parts_individually():
    x = torch.randn(3, 8)
    w = torch.rand(8) + 0.5
    y = pm.rmsnorm(x, w, 1e-6)
    torch.testing.assert_close(y, x / x.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt() * w)
    # rotation preserves the norm of each (i, i + D/2) pair and is the identity at position 0
    cos, sin = pm.rope_tables(8, 1e4, torch.arange(5))
    q = torch.randn(5, 2, 8)
    r = pm.rope_neox(q, cos, sin)
    torch.testing.assert_close(r[0], q[0])
    torch.testing.assert_close(r[..., :4] ** 2 + r[..., 4:] ** 2, q[..., :4] ** 2 + q[..., 4:] ** 2, atol=1e-5, rtol=1e-5)
    # a window of 1 attends to the token itself only
    k = torch.randn(5, 1, 8)
    v = torch.randn(5, 1, 8)
    out = pm.causal_attention(q, k, v, window=1)
    torch.testing.assert_close(out.view(5, 2, 8), v.expand(5, 2, 8))
    # inverse CDF picks the first index whose cumulative probability exceeds u
    p = torch.tensor([0.1, 0.2, 0.3, 0.4])
    assert [pm.inverse_cdf(p, u) for u in (0.0, 0.05, 0.1, 0.29, 0.3, 0.61, 0.999)] == [0, 0, 1, 1, 2, 3, 3]
