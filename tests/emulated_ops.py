"""Plain torch statements of what each CUDA kernel of the engine computes.

Two uses, both in tests only: (1) the per-kernel GPU tests compare every kernel with
the function of the same name here; (2) the CPU tests put this table in place of the
kernel table so that the engine's host logic (batching, cache, scheduler, replay) can
be exercised without a GPU.  Loops are deliberately simple; nothing here is fast.
"""

from __future__ import annotations


import torch


class TorchOps:
    name = "torch-emulation"

    def prepare(self, groups):
        pass

    # ---- norms ----------------------------------------------------------------------
    def fused_norm(self, out, weight, eps, *, resid=None, pending=None, ids=None, table=None, rows=None,
                   write_resid=True, num_rows=None):
        n = out.shape[0] if num_rows is None else num_rows
        src = rows[:n].long() if rows is not None else torch.arange(n, device=out.device)
        if ids is not None:
            v = table[ids.long()[src]].float()
        else:
            v = resid[src].float()
        if pending is not None and pending.dim() == 3:  # fp32 partial sums [parts, rows, H], added in order
            total = pending[0][src]
            for p in range(1, pending.shape[0]):
                total = total + pending[p][src]
            v = v + total
        elif pending is not None:
            v = v + pending[src].float()
        if write_resid:
            resid[src] = v
        var = v.pow(2).mean(-1, keepdim=True)
        out[:n] = ((v * torch.rsqrt(var + eps)) * weight.float()).to(out.dtype)
        return out

    def silu_mul(self, gate_up, out):
        I = out.shape[-1]
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
        out.copy_(((g / (1 + torch.exp(-g))) * u).to(out.dtype))
        return out

    # ---- position encoding + cache write -----------------------------------------------
    def rope_table(self, inv_freq, max_positions):
        ang = torch.arange(max_positions, dtype=torch.float32, device=inv_freq.device)[:, None] * inv_freq[None, :]
        return ang.cos(), ang.sin()

    def qk_norm_rope_store(self, qkv, *, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos, sin,
                           positions, token_seq, block_table, k_pages, v_pages, page_size, write_kv,
                           pairing="half"):
        T = qkv.shape[0]
        D = head_dim
        pos = positions.long()

        def norm_rope(x, w):  # x [T, n, D] float
            if w is not None:
                x = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)) * w.float()
            if cos is not None:
                half = cos.shape[1]
                c, s = cos[pos][:, None, :], sin[pos][:, None, :]
                rest = x[..., 2 * half:]
                if pairing == "interleaved":  # pair i = elements (2i, 2i + 1)
                    x1, x2 = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
                    rot = torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).flatten(-2)
                    x = torch.cat((rot, rest), dim=-1)
                else:  # pair i = elements (i, i + half)
                    x1, x2 = x[..., :half], x[..., half:2 * half]
                    x = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)
            return x

        nq, nkv = num_heads, num_kv_heads
        q = qkv[:, : nq * D].reshape(T, nq, D).float()
        qkv[:, : nq * D] = norm_rope(q, q_weight).reshape(T, nq * D).to(qkv.dtype)
        if not write_kv:
            return
        k = norm_rope(qkv[:, nq * D:(nq + nkv) * D].reshape(T, nkv, D).float(), k_weight).to(qkv.dtype)
        v = qkv[:, (nq + nkv) * D:(nq + 2 * nkv) * D].reshape(T, nkv, D)
        for t in range(T):
            p = int(pos[t])
            page = int(block_table[int(token_seq[t]), p // page_size])
            k_pages[page, :, p % page_size, :] = k[t]
            v_pages[page, :, p % page_size, :] = v[t]

    # ---- attention --------------------------------------------------------------------
    def paged_attention(self, q, q_stride, *, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table,
                        token_seq, positions, out, page_size, scale, window, step=None):
        T = out.shape[0]
        D = head_dim
        group = num_heads // num_kv_heads
        for t in range(T):
            p = int(positions[t])
            lo = max(0, p - window + 1) if window else 0
            table = block_table[int(token_seq[t])]
            js = torch.arange(lo, p + 1)
            pages = table[(js // page_size).to(table.device)].long()
            offs = (js % page_size).to(pages.device)
            keys = k_pages[pages, :, offs, :].float()  # [n, nkv, D]
            vals = v_pages[pages, :, offs, :].float()
            qt = q[t, : num_heads * D].reshape(num_heads, D).float()
            kh = keys.repeat_interleave(group, dim=1)  # [n, nq, D]
            vh = vals.repeat_interleave(group, dim=1)
            scores = torch.einsum("hd,nhd->hn", qt, kh) * scale
            probs = torch.softmax(scores, dim=-1)
            out[t] = torch.einsum("hn,nhd->hd", probs, vh).reshape(-1).to(out.dtype)
        return out

    # ---- matrix products ----------------------------------------------------------------
    partial_parts = 0  # > 1: linear(partial_sums=True) answers with that many planes

    def add_bias(self, out, bias):
        out.copy_((out.float() + bias.float()).to(out.dtype))
        return out

    def logit_scale_cap(self, logits, scale=1.0, cap=0.0):
        v = logits * scale
        logits.copy_(cap * torch.tanh(v / cap) if cap > 0 else v)
        return logits

    def linear(self, x, weight, out=None, out_dtype=None, partial_sums=False, bias=None):
        if bias is not None:
            return self.add_bias(self.linear(x, weight, out, out_dtype), bias)
        if partial_sums and self.partial_parts > 1 and out is None and out_dtype is None:
            cuts = torch.linspace(0, x.shape[1], self.partial_parts + 1).long().tolist()
            return torch.stack([x[:, a:b].float() @ weight[:, a:b].float().t() for a, b in zip(cuts, cuts[1:])])
        res = x.float() @ weight.float().t()
        res = res.to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def gated_linear(self, x, gate_up_weight, out):
        return self.silu_mul(self.linear(x, gate_up_weight), out)

    # ---- sampling ---------------------------------------------------------------------
    def argmax(self, logits, want_logprob=False):
        tok = logits.argmax(-1).to(torch.int32)
        lp = None
        if want_logprob:
            lp = torch.log_softmax(logits.float(), -1).gather(1, tok.long()[:, None])[:, 0]
        return tok, lp

    def sample(self, logits, temperature, uniform, want_logprob=False):
        probs = torch.softmax(logits.float() / temperature[:, None], -1)
        cdf = probs.cumsum(-1)
        idx = torch.searchsorted(cdf, uniform[:, None].contiguous(), right=True)[:, 0].clamp(0, logits.shape[1] - 1)
        lp = None
        if want_logprob:
            lp = torch.log(probs.gather(1, idx[:, None])[:, 0].clamp_min(1e-30))
        return idx.to(torch.int32), lp

    def bias_penalty_row(self, row, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                         frequency_penalty):
        for tok, val in (logit_bias or {}).items():
            row[int(tok)] += float(val)
        if seen_ids and not (repetition_penalty == 1.0 and presence_penalty == 0.0 and frequency_penalty == 0.0):
            V = row.numel()
            counts = torch.bincount(torch.tensor([t for t in seen_ids if 0 <= t < V], dtype=torch.long), minlength=V)
            counts = counts.to(row.device)
            seen = counts > 0
            rep = torch.where(row > 0, row / repetition_penalty, row * repetition_penalty)
            row.copy_(torch.where(seen, rep, row) - presence_penalty * seen.float() - frequency_penalty * counts.float())
        return row

    def bias_penalty_rows(self, logits, rows, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                          frequency_penalty):
        for i, b, s, rp, pp, fp in zip(rows, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                                       frequency_penalty):
            self.bias_penalty_row(logits[i], logit_bias=b, seen_ids=list(s), repetition_penalty=rp,
                                  presence_penalty=pp, frequency_penalty=fp)
        return logits

    def filter_rows(self, logits, temperature, min_p, top_k, top_p):
        lowest = torch.finfo(torch.float32).min
        for r in range(logits.shape[0]):
            x = logits[r] / temperature[r]
            if float(min_p[r]) > 0:
                p = torch.softmax(x, -1)
                x = torch.where(p < float(min_p[r]) * p.max(), torch.full_like(x, float("-inf")), x)
            k = int(top_k[r])
            if 0 < k < x.numel():
                kth = torch.topk(x, k).values[-1]
                x = torch.where(x < kth, torch.full_like(x, lowest), x)
            tp = float(top_p[r])
            if 0 < tp < 1:
                p = torch.softmax(x, -1)
                order = torch.argsort(x, descending=True, stable=True)
                before = p[order].cumsum(0) - p[order]  # mass ranked before each token
                keep = torch.zeros_like(x, dtype=torch.bool)
                keep[order] = before <= tp
                # tokens tied with a kept one are kept as well (the kernel cuts by value)
                keep |= x >= x[keep].min()
                x = torch.where(keep, x, torch.full_like(x, lowest))
            logits[r] = x
        return logits
