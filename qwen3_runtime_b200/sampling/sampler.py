"""Choose the next token for the rows of a step that sample.

Greedy rows take the argmax kernel; rows with a temperature draw by inverse CDF on
the device with a uniform number from the request's own CPU generator (so a seed
gives the same draws on any device, qwen3_runtime/sampling.py:208-227, 293-298).
Rows that use logit bias, penalties, min_p, top_k or top_p first pass the processor
kernels, in the reference's order (sampling.py:120-135).  Token ids come back to the
host in one copy.
"""

from __future__ import annotations

import torch

from .params import SamplingParams


def draw_uniform(generator: torch.Generator | None) -> float:
    return float(torch.rand((), dtype=torch.float32, generator=generator))


class Sampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = device

    def sample(self, logits: torch.Tensor, requests: list) -> tuple[list[int], list[float | None]]:
        """``logits`` [R, V] float32, one row per request in ``requests``."""
        R = len(requests)
        if logits.shape[0] != R:
            raise ValueError(f"logits rows {logits.shape[0]} must equal {R} sampling requests")
        params: list[SamplingParams] = [r.sampling for r in requests]
        if any(p.logit_bias or p.has_penalties() or (not p.is_greedy() and p.needs_filter()) for p in params):
            logits = self._process(logits, requests)
        want_lp = any(p.logprobs for p in params)
        greedy = [i for i, p in enumerate(params) if p.is_greedy()]
        if len(greedy) == R:
            tok, lp = self.ops.argmax(logits, want_lp)
            return tok.tolist(), (lp.tolist() if want_lp else [None] * R)
        temps = torch.tensor([p.temperature if not p.is_greedy() else 1.0 for p in params], dtype=torch.float32)
        unis = torch.tensor([0.0 if p.is_greedy() else draw_uniform(r.rng) for p, r in zip(params, requests)],
                            dtype=torch.float32)
        host = torch.stack([temps, unis]).pin_memory() if logits.is_cuda else torch.stack([temps, unis])
        dev = host.to(self.device, non_blocking=True)
        tok_s, lp_s = self.ops.sample(logits, dev[0], dev[1], want_lp)
        if greedy:
            tok_g, lp_g = self.ops.argmax(logits, want_lp)
            mask = torch.zeros(R, dtype=torch.bool)
            mask[greedy] = True
            mask = mask.to(self.device, non_blocking=True)
            tok_s = torch.where(mask, tok_g, tok_s)
            if want_lp:
                lp_s = torch.where(mask, lp_g, lp_s)
        return tok_s.tolist(), (lp_s.tolist() if want_lp else [None] * R)

    def _process(self, logits: torch.Tensor, requests: list) -> torch.Tensor:
        out = logits.clone()
        for i, req in enumerate(requests):
            p: SamplingParams = req.sampling
            if p.logit_bias or p.has_penalties() or (not p.is_greedy() and p.needs_filter()):
                self.ops.process_logits_row(out[i], p, req.token_ids)
        return out
