"""Shared by the tests: tiny configurations, model folders, traces and comparisons."""

from __future__ import annotations

import random

import torch

from qwen3_runtime_b200.config import Qwen3Config
from qwen3_runtime_b200.weights import write_random_model

# Tiny configurations that differ in every size and option the architecture has:
# layers, width, head counts and group size, head size, q width vs width, feed-forward
# width, vocabulary (one not a power of two, one odd), rope_theta, eps, tying, page size.
TINY = {
    "A": dict(
        config=Qwen3Config(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, intermediate_size=128, rms_norm_eps=1e-6,
                           rope_theta=1e4, max_position_embeddings=512, tie_word_embeddings=True),
        page_size=16, vector_std=0.02, seed=11),
    "B": dict(
        config=Qwen3Config(vocab_size=384, hidden_size=96, num_hidden_layers=3, num_attention_heads=8,
                           num_key_value_heads=2, head_dim=32, intermediate_size=160, rms_norm_eps=1e-5,
                           rope_theta=1e6, max_position_embeddings=512, tie_word_embeddings=False),
        page_size=8, vector_std=0.05, seed=12),
    "C": dict(
        config=Qwen3Config(vocab_size=301, hidden_size=80, num_hidden_layers=2, num_attention_heads=6,
                           num_key_value_heads=3, head_dim=48, intermediate_size=112, rms_norm_eps=3e-5,
                           rope_theta=5e5, max_position_embeddings=512, tie_word_embeddings=False),
        page_size=4, vector_std=0.1, seed=13),
    # head sizes 64 and 128: the only tiny models whose bfloat16 steps take the split-KV decode
    # kernel (with the newest token's q/k/v made inside it), the tensor-core prefill kernels and,
    # with rows of 16-byte multiples, the weight-streaming products
    "D": dict(
        config=Qwen3Config(vocab_size=320, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=64, intermediate_size=192, rms_norm_eps=1e-6,
                           rope_theta=1e6, max_position_embeddings=1024, tie_word_embeddings=True),
        page_size=16, vector_std=0.05, seed=14),
    "E": dict(
        config=Qwen3Config(vocab_size=411, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=1, head_dim=128, intermediate_size=320, rms_norm_eps=1e-5,
                           rope_theta=1e6, max_position_embeddings=1024, tie_word_embeddings=False),
        page_size=16, vector_std=0.05, seed=15),
}

# Random N(0, 0.02) weights at these widths give almost flat logits that hide faults;
# the tests draw matrices with a larger spread so that attention and the feed-forward
# matter to the result.
TEST_STD = 0.1


def make_model_dir(tmp_path, name: str, *, store_dtype: str = "bfloat16"):
    spec = TINY[name]
    folder = tmp_path / f"tiny_{name}_{store_dtype}"
    if not (folder / "model.safetensors").exists():
        write_random_model(spec["config"], folder, spec["seed"], std=TEST_STD, vector_std=spec["vector_std"],
                           store_dtype=store_dtype)
    return folder


def random_ids(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ---------------------------------------------------------------------------------------
# traces: lists of steps {"step", "entries": [{"id", "tokens", "want"}], "end"}
# ---------------------------------------------------------------------------------------

def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one step each, every position wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def trace_tail_decode(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, s = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        s += 1
        for i in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict[str, list[int]], seed: int = 0) -> list[dict]:
    """Portions of changing size, down to two tokens (and single ones)."""
    rnd = random.Random(seed)
    sizes = [7, 2, 5, 3, 2, 31, 1, 2, 17, 64, 2, 9]
    steps, s = [], 0
    for rid, toks in requests.items():
        i = 0
        while i < len(toks):
            n = min(len(toks) - i, rnd.choice(sizes))
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}],
                          "end": [rid] if i + n == len(toks) else []})
            i += n
            s += 1
    return steps


def trace_mixed(requests: dict[str, list[int]], seed: int = 0, max_live: int = 4, decode_tail: int = 12,
                admit: float = 0.7) -> list[dict]:
    """Up to ``max_live`` requests live at a time; every step holds portions of some beside
    single tokens of others; a request is sometimes left out of a step; requests end at
    different times so that their pages are handed to later ones.  ``admit``: the chance that
    one more pending request starts in a step that has room for it."""
    rnd = random.Random(seed)
    pending = list(requests.items())
    live: dict[str, int] = {}
    steps, s = [], 0
    while pending or live:
        while pending and len(live) < max_live and (not live or rnd.random() < admit):
            rid, _ = pending.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            toks, i = requests[rid], live[rid]
            if len(live) > 1 and rnd.random() < 0.2:
                continue  # sits this step out
            remaining = len(toks) - i
            if remaining <= decode_tail:
                n = 1
            else:
                n = min(remaining - decode_tail, rnd.choice([2, 3, 5, 8, 13, 21, 40]))
            entries.append({"id": rid, "tokens": toks[i:i + n], "want": list(range(n))})
            live[rid] = i + n
            if i + n == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": s, "entries": entries, "end": end})
            s += 1
    return steps


def peak_live(steps: list[dict]) -> int:
    """The most requests that are live at the same time in a trace."""
    live: set[str] = set()
    peak = 0
    for st in steps:
        live.update(e["id"] for e in st["entries"])
        peak = max(peak, len(live))
        live.difference_update(st["end"])
    return peak


def thin_wants(steps: list[dict], keep: int = 2) -> list[dict]:
    """The same trace asking for fewer logits: of every entry's wanted places only the first
    and the last ``keep - 1`` (large vocabularies make every wanted row expensive to compare)."""
    out = []
    for st in steps:
        entries = []
        for e in st["entries"]:
            w = sorted(e["want"])
            w = w if len(w) <= keep else [w[0], *w[len(w) - keep + 1:]]
            entries.append({**e, "want": w})
        out.append({**st, "entries": entries})
    return out


def peak_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: list[dict], outputs: dict[int, torch.Tensor]) -> dict[str, dict[int, torch.Tensor]]:
    """``{request: {position: logits row}}`` from per-step outputs."""
    pos: dict[str, int] = {}
    result: dict[str, dict[int, torch.Tensor]] = {}
    for st in steps:
        row = 0
        out = outputs.get(st["step"])
        for e in st["entries"]:
            start = pos.get(e["id"], 0)
            for w in e["want"]:
                result.setdefault(e["id"], {})[start + w] = out[row]
                row += 1
            pos[e["id"]] = start + len(e["tokens"])
        assert out is None or row == out.shape[0]
    return result


def run_trace(rt, steps: list[dict], *, poison: bool = False, check: bool = True) -> dict[str, dict[int, torch.Tensor]]:
    """Drive a Runtime (model + cache + step function) through a trace, in process,
    the way ``bin/trace_run`` does."""
    from qwen3_runtime_b200.engine.batch import StepEntry

    live = {}
    outputs = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            rc = live.get(e["id"])
            if rc is None:
                rc = live[e["id"]] = rt.cache.open(e["id"])
            rt.cache.reserve(rc, len(e["tokens"]))
            entries.append(StepEntry(rc, list(e["tokens"]), list(e["want"])))
        logits = rt.runner.run(entries)
        if logits is not None:
            outputs[st["step"]] = logits.float().cpu()
        for rid in st["end"]:
            rc = live.pop(rid)
            pages = [list(t) for t in rc.tables]
            rt.cache.close(rc)
            if poison:  # whatever a later request finds in a page that is used again must not matter
                for gi, pg in enumerate(pages):
                    rt.storage.poison_pages(gi, [p for p in pg if p >= 0])
        if check:
            rt.cache.check_invariants()
    return collect(steps, outputs)


def max_abs_diff(got: dict, want: dict[str, torch.Tensor]) -> float:
    worst = 0.0
    for rid, rows in got.items():
        for p, row in rows.items():
            worst = max(worst, float((row.double() - want[rid][p].double()).abs().max()))
    return worst


def first_mismatch(got: dict, want: dict[str, torch.Tensor], tol: float):
    """(request, position, diff) of the first place beyond ``tol`` -- for failure messages."""
    for rid, rows in got.items():
        for p in sorted(rows):
            d = float((rows[p].double() - want[rid][p].double()).abs().max())
            if not d <= tol:
                return rid, p, d
    return None
