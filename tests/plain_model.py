"""A plain, slow implementation of the Qwen3 dense decoder for the tests.

Whole sequences, no cache, no batching, one function per part, written from the
formulas of yuzheng310/qwen3-runtime (file:line cited per function, paths within
that project).  It shares no code with the engine: it reads ``config.json`` and
``model.safetensors`` itself and keeps weights under their Hugging Face names.

``act_dtype`` (optional) rounds activations to that dtype at the places where a
reduced-precision engine stores them (norm outputs, projection outputs, q and k
after rotation, attention output, the SwiGLU product); all arithmetic between
those places stays in ``compute`` precision (float32 or float64), which is how
the reference's own ops behave when the model dtype is bfloat16
(qwen3_runtime/layers/ops.py:17-49).  The residual stream is never rounded.

tests/golden/ holds logits that the reference's own model code produced on the
CPU for two tiny models; tests/test_plain_model.py compares this file with them.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors.torch import load_file


def read_model_dir(model_dir):
    """``(config dict, {hf_name: tensor})`` straight from the files."""
    model_dir = Path(model_dir)
    raw = json.loads((model_dir / "config.json").read_text())
    tensors = {}
    for f in sorted(model_dir.glob("*.safetensors")):
        tensors.update(load_file(str(f)))
    return raw, tensors


def head_dim_of(raw) -> int:
    # qwen3_runtime/models/qwen3.py:46 -- optional key, default hidden // heads
    return int(raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"])


def _round(x: torch.Tensor, act_dtype) -> torch.Tensor:
    if act_dtype is None:
        return x
    return x.to(act_dtype).to(x.dtype)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """qwen3_runtime/layers/ops.py:17-20 -- mean of squares, rsqrt(var+eps), then times weight."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    y = x * torch.rsqrt(var + eps)
    return y * weight.to(x.dtype)


def rope_tables(head_dim: int, theta: float, positions: torch.Tensor):
    """qwen3_runtime/layers/rope.py:17-22 -- inv_j = 1/theta^(2j/D) and angle p*inv_j, in float32."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    freqs = torch.einsum("i,j->ij", positions.to(torch.float), inv)
    return freqs.cos(), freqs.sin()


def rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """qwen3_runtime/layers/rope.py:7-11 -- rotate-half (not interleaved); x is [T, heads, D]."""
    x1, x2 = x.chunk(2, dim=-1)
    c = cos.to(x.dtype).unsqueeze(1)
    s = sin.to(x.dtype).unsqueeze(1)
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def causal_attention(q, k, v, *, window=None, act_dtype=None):
    """qwen3_runtime/attention/pytorch.py:12-47 and reference/dense_attention.py:10-46.

    q: [T, nq, D]; k, v: [T, nkv, D].  Query head h reads kv head h // (nq // nkv);
    scores = q.k / sqrt(D); key j is allowed for query i iff j <= i (and, with a
    window w, j > i - w); softmax in full precision; probabilities rounded to the
    activation dtype before the product with v (pytorch.py:45).
    """
    T, nq, D = q.shape
    group = nq // k.shape[1]
    kh = k.repeat_interleave(group, dim=1).transpose(0, 1)  # [nq, T, D]
    vh = v.repeat_interleave(group, dim=1).transpose(0, 1)
    qh = q.transpose(0, 1)
    scores = torch.matmul(qh, kh.transpose(-2, -1)) * (1.0 / math.sqrt(D))
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    allowed = j <= i
    if window is not None:
        allowed = allowed & (j > i - window)
    scores = scores.masked_fill(~allowed, float("-inf"))
    probs = _round(torch.softmax(scores, dim=-1), act_dtype)
    return torch.matmul(probs, vh).transpose(0, 1).reshape(T, nq * D)


def attention_part(x, w, prefix, raw, positions, *, act_dtype=None, window=None, shared_kv=None):
    """qwen3_runtime/models/qwen3.py:96-117 -- q/k/v projections, per-head RMSNorm on
    q and k over D, then RoPE on q and k, attention, output projection.
    Returns ``(output, (k, v))``; with ``shared_kv`` the keys and values of another
    layer are used instead of this layer's own."""
    T = x.shape[0]
    nq, nkv, D = raw["num_attention_heads"], raw["num_key_value_heads"], head_dim_of(raw)
    eps = raw["rms_norm_eps"]
    cos, sin = rope_tables(D, raw["rope_theta"], positions)
    q = _round(x @ w[prefix + "q_proj.weight"].to(x.dtype).T, act_dtype).view(T, nq, D)
    q = _round(rope_neox(rmsnorm(q, w[prefix + "q_norm.weight"], eps), cos, sin), act_dtype)
    if shared_kv is None:
        k = _round(x @ w[prefix + "k_proj.weight"].to(x.dtype).T, act_dtype).view(T, nkv, D)
        v = _round(x @ w[prefix + "v_proj.weight"].to(x.dtype).T, act_dtype).view(T, nkv, D)
        k = _round(rope_neox(rmsnorm(k, w[prefix + "k_norm.weight"], eps), cos, sin), act_dtype)
    else:
        k, v = shared_kv
    ctx = _round(causal_attention(q, k, v, window=window, act_dtype=act_dtype), act_dtype)
    out = _round(ctx @ w[prefix + "o_proj.weight"].to(x.dtype).T, act_dtype)
    return out, (k, v)


def swiglu_part(x, w, prefix, *, act_dtype=None):
    """qwen3_runtime/models/qwen3.py:137-138 and layers/ops.py:23-25 --
    down(silu(gate x) * up x), silu(z) = z * sigmoid(z)."""
    g = x @ w[prefix + "gate_proj.weight"].to(x.dtype).T
    u = x @ w[prefix + "up_proj.weight"].to(x.dtype).T
    if act_dtype is not None:
        g, u = _round(g, act_dtype), _round(u, act_dtype)
    m = _round(g * torch.sigmoid(g) * u, act_dtype)
    return _round(m @ w[prefix + "down_proj.weight"].to(x.dtype).T, act_dtype)


def forward_hidden(raw, w, ids, *, compute=torch.float32, act_dtype=None, order=None, window=None):
    """The residual stream before the final norm, [T, H]
    (qwen3_runtime/models/qwen3.py:243-260; textbook form tests/cpu/reference_qwen3.py:79-110).

    ``order`` is a list of ``(block, cache, writes)``; default: each layer once, in
    order, with its own keys and values.
    """
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    w = {k: v.to(compute) if v.is_floating_point() else v for k, v in w.items()}
    h = w["model.embed_tokens.weight"][ids]
    eps = raw["rms_norm_eps"]
    L = raw["num_hidden_layers"]
    order = order or [(i, i, True) for i in range(L)]
    kv = {}
    for block, cache, writes in order:
        p = f"model.layers.{block}."
        n = _round(rmsnorm(h, w[p + "input_layernorm.weight"], eps), act_dtype)
        a, own = attention_part(
            n, w, p + "self_attn.", raw, positions,
            act_dtype=act_dtype, window=window, shared_kv=None if writes else kv[cache],
        )
        if writes:
            kv[cache] = own
        h = h + a
        n = _round(rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps), act_dtype)
        h = h + swiglu_part(n, w, p + "mlp.", act_dtype=act_dtype)
    return h, w


def forward_logits(raw, w, ids, rows=None, **kw):
    """Logits at every position, [T, V] (qwen3_runtime/models/qwen3.py:263-266): final
    RMSNorm, then the tied embedding or ``lm_head.weight``.  ``rows``: only those positions
    (the reference, too, gives the head only the rows that sample, :262-264)."""
    h, wc = forward_hidden(raw, w, ids, **kw)
    if rows is not None:
        h = h[torch.as_tensor(rows, dtype=torch.long)]
    n = _round(rmsnorm(h, wc["model.norm.weight"], raw["rms_norm_eps"]), kw.get("act_dtype"))
    head = wc["model.embed_tokens.weight"] if raw["tie_word_embeddings"] else wc["lm_head.weight"]
    return n @ head.T


def greedy_generate(raw, w, prompt, max_tokens, **kw):
    """Recompute the whole sequence for every new token; argmax, lowest id on ties
    (qwen3_runtime/sampling.py:28-32)."""
    ids = list(prompt)
    out = []
    for _ in range(max_tokens):
        tok = int(torch.argmax(forward_logits(raw, w, ids, rows=[len(ids) - 1], **kw)[0]).item())
        ids.append(tok)
        out.append(tok)
    return out


def temperature_probs(logits_row: torch.Tensor, temperature: float) -> torch.Tensor:
    """qwen3_runtime/sampling.py:120-135, 265 -- softmax(logits.float() / temperature)."""
    return torch.softmax(logits_row.float() / temperature, dim=-1)


def inverse_cdf(probs: torch.Tensor, u: float) -> int:
    """qwen3_runtime/sampling.py:208-227 -- searchsorted(cumsum(p), u, right=True), clamped."""
    cdf = probs.float().cumsum(0)
    idx = int(torch.searchsorted(cdf, torch.tensor(u, dtype=torch.float32), right=True).item())
    return max(0, min(idx, probs.numel() - 1))
