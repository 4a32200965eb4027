"""Choose the next token for the rows of a step that sample.

Greedy rows take the argmax kernel; rows with a temperature draw by inverse CDF on
the device with a uniform number from the request's own CPU generator (so a seed
gives the same draws on any device, qwen3_runtime/sampling.py:208-227, 293-298).
Rows that use logit bias, penalties, min_p, top_k or top_p first pass the processor
kernels, in the reference's order (sampling.py:120-135).  Token ids come back to the
host in one copy, which :meth:`Sampler.launch` starts and :meth:`Sampler.read` waits for, so
that the engine can put the next step on the device in between.
"""

from __future__ import annotations

import torch

from .params import SamplingParams


def draw_uniform(generator: torch.Generator | None) -> float:
    return float(torch.rand((), dtype=torch.float32, generator=generator))


class Sampled:
    """What :meth:`Sampler.launch` leaves: the tokens on the device (the next step may read
    them there) and their copy to the host, under way."""

    __slots__ = ("tokens", "logprobs", "host_tokens", "host_logprobs", "event", "count")

    def __init__(self, tokens, logprobs, host_tokens, host_logprobs, event, count):
        self.tokens, self.logprobs = tokens, logprobs
        self.host_tokens, self.host_logprobs = host_tokens, host_logprobs
        self.event, self.count = event, count


class Sampler:
    RING = 4  # pinned result buffers; at most two steps are ever unread

    def __init__(self, ops, device):
        self.ops = ops
        self.device = device
        self.on_cuda = torch.device(device).type == "cuda"
        self._ring: list[tuple[torch.Tensor, torch.Tensor]] = []
        self._turn = 0

    def sample(self, logits: torch.Tensor, requests: list) -> tuple[list[int], list[float | None]]:
        """``logits`` [R, V] float32, one row per request in ``requests``."""
        return self.read(self.launch(logits, requests))

    def launch(self, logits: torch.Tensor, requests: list) -> Sampled:
        """Choose on the device and start the copy to the host; waits for nothing."""
        tok, lp = self._choose(logits, requests)
        R = len(requests)
        if not self.on_cuda:
            return Sampled(tok, lp, tok, lp, None, R)
        if not self._ring or self._ring[0][0].numel() < R:
            size = max(64, 1 << (R - 1).bit_length())
            self._ring = [(torch.zeros(size, dtype=torch.int32, pin_memory=True),
                           torch.zeros(size, dtype=torch.float32, pin_memory=True)) for _ in range(self.RING)]
        self._turn = (self._turn + 1) % self.RING
        host_tok, host_lp = self._ring[self._turn]
        host_tok[:R].copy_(tok, non_blocking=True)
        if lp is not None:
            host_lp[:R].copy_(lp, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return Sampled(tok, lp, host_tok, host_lp if lp is not None else None, event, R)

    def read(self, sampled: Sampled) -> tuple[list[int], list[float | None]]:
        if sampled.event is not None:
            sampled.event.synchronize()
        R = sampled.count
        toks = sampled.host_tokens[:R].tolist()
        lps = sampled.host_logprobs[:R].tolist() if sampled.host_logprobs is not None else [None] * R
        return toks, lps

    def _choose(self, logits: torch.Tensor, requests: list) -> tuple[torch.Tensor, torch.Tensor | None]:
        """int32 tokens [R] (and float32 log-probabilities, if any request asks) on the device."""
        R = len(requests)
        if logits.shape[0] != R:
            raise ValueError(f"logits rows {logits.shape[0]} must equal {R} sampling requests")
        params: list[SamplingParams] = [r.sampling for r in requests]
        want_lp = any(p.logprobs for p in params)
        greedy = [i for i, p in enumerate(params) if p.is_greedy()]
        touched = [i for i, p in enumerate(params)
                   if p.logit_bias or p.has_penalties() or (not p.is_greedy() and p.needs_filter())]
        if touched:
            logits = self._process(logits, requests, touched)
        if len(greedy) == R:
            tok, lp = self.ops.argmax(logits, want_lp)
            return tok, (lp if want_lp else None)
        # rows that went through the filters are already divided by their temperature
        filtered = {i for i in touched if not params[i].is_greedy() and params[i].needs_filter()}
        temps = [1.0 if (p.is_greedy() or i in filtered) else p.temperature for i, p in enumerate(params)]
        unis = [0.0 if p.is_greedy() else draw_uniform(r.rng) for p, r in zip(params, requests)]
        dev = self._to_device(torch.tensor([temps, unis], dtype=torch.float32))
        tok_s, lp_s = self.ops.sample(logits, dev[0], dev[1], want_lp)
        if greedy:
            tok_g, lp_g = self.ops.argmax(logits, want_lp)
            mask = torch.zeros(R, dtype=torch.bool)
            mask[greedy] = True
            mask = self._to_device(mask)
            tok_s = torch.where(mask, tok_g, tok_s)
            if want_lp:
                lp_s = torch.where(mask, lp_g, lp_s)
        return tok_s, (lp_s if want_lp else None)

    def _to_device(self, host: torch.Tensor) -> torch.Tensor:
        if torch.device(self.device).type == "cuda":
            host = host.pin_memory()
        return host.to(self.device, non_blocking=True)

    def _process(self, logits: torch.Tensor, requests: list, touched: list[int]) -> torch.Tensor:
        """Processor chain on a copy of the rows that need it (qwen3_runtime/sampling.py:120-135):
        bias and penalties per row, then one launch that divides by the temperature and applies
        min_p, top_k and top_p to the non-greedy rows."""
        out = logits.clone()
        biased = [i for i in touched if requests[i].sampling.logit_bias or requests[i].sampling.has_penalties()]
        if biased:  # one launch for all of them
            ps = [requests[i].sampling for i in biased]
            self.ops.bias_penalty_rows(out, biased, logit_bias=[p.logit_bias for p in ps],
                                       seen_ids=[requests[i].token_ids for i in biased],
                                       repetition_penalty=[p.repetition_penalty for p in ps],
                                       presence_penalty=[p.presence_penalty for p in ps],
                                       frequency_penalty=[p.frequency_penalty for p in ps])
        rows = [i for i in touched if not requests[i].sampling.is_greedy() and requests[i].sampling.needs_filter()]
        if rows:
            ps = [requests[i].sampling for i in rows]
            f = self._to_device(torch.tensor([[p.temperature for p in ps], [p.min_p for p in ps],
                                              [p.top_p for p in ps]], dtype=torch.float32))
            k = self._to_device(torch.tensor([p.top_k for p in ps], dtype=torch.int32))
            if len(rows) == logits.shape[0]:
                self.ops.filter_rows(out, f[0], f[1], k, f[2])
            else:
                idx = self._to_device(torch.tensor(rows, dtype=torch.long))
                sub = out.index_select(0, idx).contiguous()
                self.ops.filter_rows(sub, f[0], f[1], k, f[2])
                out.index_copy_(0, idx, sub)
        return out
