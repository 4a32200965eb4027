"""Dense gated feed-forward (SwiGLU): down(silu(gate x) * up x), no biases
(qwen3_runtime/models/qwen3.py:130-138; layers/ops.py:23-25)."""

from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, StepContext, register_part


class GatedMLP(Part):
    category = "feed_forward"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        activation = spec.get("activation", "silu")
        if activation != "silu":
            raise ValueError(f"gated_mlp has a silu kernel only, not {activation!r}")
        self.down_bias = bool(spec.get("down_bias", False))
        self.gate_up_weight = self.down_weight = self.down_bias_vec = None

    def param_specs(self):
        specs = {
            "gate_proj.weight": ParamSpec((self.intermediate_size, self.hidden_size)),
            "up_proj.weight": ParamSpec((self.intermediate_size, self.hidden_size)),
            "down_proj.weight": ParamSpec((self.hidden_size, self.intermediate_size)),
        }
        if self.down_bias:
            specs["down_proj.bias"] = ParamSpec((self.hidden_size,), "vector")
        return specs

    def load(self, tensors):
        # one product for gate and up: gate rows first (utils/loader.py:51-53)
        self.gate_up_weight = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.down_weight = tensors["down_proj.weight"].contiguous()
        self.down_bias_vec = tensors.get("down_proj.bias")

    def kernel_groups(self):
        if self.ctx.dtype == torch.float32:
            return ["norm", "gemm_f32"]
        return ["norm", "gemm_small_m", "gemm_stream", "gemm_tcgen05"]

    def forward(self, h: torch.Tensor, step: StepContext) -> torch.Tensor:
        mid = torch.empty((h.shape[0], self.intermediate_size), dtype=h.dtype, device=h.device)
        self.ops.gated_linear(h, self.gate_up_weight, mid)
        if self.down_bias_vec is not None:
            return self.ops.linear(mid, self.down_weight, bias=self.down_bias_vec)
        return self.ops.linear(mid, self.down_weight, partial_sums=self.partial_sums_ok)


register_part("feed_forward", "gated_mlp", GatedMLP)
