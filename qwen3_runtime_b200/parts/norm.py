"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in float32, one rounding at the end
(qwen3_runtime/layers/ops.py:17-20; residual form :28-37)."""

from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, ResidualStream, register_part


class RMSNorm(Part):
    category = "norm"
    adds_partial_sums = True

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), "vector")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def kernel_groups(self):
        return ["norm"]

    def add_norm(self, stream: ResidualStream, rows: torch.Tensor | None = None,
                 num_rows: int | None = None) -> torch.Tensor:
        """Fold what is pending into the residual sum and return its normalised rows.

        With ``rows`` only those rows are normalised and the residual sum is left as
        it is (the final norm before the output head)."""
        n = stream.num_tokens if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=self.ctx.device)
        keep = rows is None
        if stream.embed is not None:
            ids, table = stream.embed
            if keep:
                stream.resid = torch.empty((stream.num_tokens, self.size), dtype=torch.float32,
                                           device=self.ctx.device)
            self.ops.fused_norm(out, self.weight, self.eps, resid=stream.resid if keep else None,
                                pending=stream.pending, ids=ids, table=table, rows=rows, write_resid=keep,
                                num_rows=n)
            if keep:
                stream.embed = None
        else:
            self.ops.fused_norm(out, self.weight, self.eps, resid=stream.resid, pending=stream.pending,
                                rows=rows, write_resid=keep, num_rows=n)
        if keep:
            stream.pending = None
        return out


register_part("norm", "rmsnorm", RMSNorm)
