"""Grouped-query attention over the paged cache.

q/k/v projection (one fused product), optional per-head RMSNorm on q and k, position
encoding on q and k, store of k and v into the cache pages, causal attention of every
token over its sequence's pages (optionally only a window of them), output projection.
Parity: qwen3_runtime/models/qwen3.py:62-127 and attention/pytorch.py:18-47.
"""

from __future__ import annotations

import math

import torch

from ..cache.layout import KVLayerSpec
from ..config.spec import PartSpec
from .base import BuildContext, ParamSpec, Part, StepContext, build_part, register_part


class PagedAttention(Part):
    category = "mixer"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.qk_norm_eps = spec.get("qk_norm_eps")
        self.window = spec.get("window") or None
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.head_dim))
        self._slices_choice = ("decode_slices", self.num_kv_heads, self.head_dim, self.window)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ValueError(
                f"head_dim={self.head_dim} is not supported: the attention kernels take multiples of 16 up to 256")
        pos_spec = spec.get("position") or PartSpec("none")
        self.position = build_part("position", pos_spec, ctx)
        if self.position.style not in ("none", "rotary"):
            raise ValueError(f"the fused q/k kernel has no {self.position.style!r} position encoding")
        self.pairing = getattr(self.position, "pairing", "half")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotation pairs are 'half' or 'interleaved', not {self.pairing!r}")
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.o_bias = bool(spec.get("o_bias", False))
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qkv_weight = self.o_weight = self.q_norm_weight = self.k_norm_weight = None

    def param_specs(self):
        specs = {
            "q_proj.weight": ParamSpec((self.q_size, self.hidden_size)),
            "k_proj.weight": ParamSpec((self.kv_size, self.hidden_size)),
            "v_proj.weight": ParamSpec((self.kv_size, self.hidden_size)),
            "o_proj.weight": ParamSpec((self.hidden_size, self.q_size)),
        }
        if self.qk_norm_eps is not None:
            specs["q_norm.weight"] = ParamSpec((self.head_dim,), "vector")
            specs["k_norm.weight"] = ParamSpec((self.head_dim,), "vector")
        if self.qkv_bias:
            specs["q_proj.bias"] = ParamSpec((self.q_size,), "vector")
            specs["k_proj.bias"] = ParamSpec((self.kv_size,), "vector")
            specs["v_proj.bias"] = ParamSpec((self.kv_size,), "vector")
        if self.o_bias:
            specs["o_proj.bias"] = ParamSpec((self.hidden_size,), "vector")
        return specs

    def load(self, tensors):
        # one product for q, k and v: rows of q, then k, then v (utils/loader.py:44-47)
        self.qkv_weight = torch.cat(
            [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0).contiguous()
        self.o_weight = tensors["o_proj.weight"].contiguous()
        self.q_norm_weight = tensors.get("q_norm.weight")
        self.k_norm_weight = tensors.get("k_norm.weight")
        self.qkv_bias_vec = (torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]])
                             if self.qkv_bias else None)
        self.o_bias_vec = tensors.get("o_proj.bias")

    def kernel_groups(self):
        groups = ["rope_kv", "attention_generic", *self.position.kernel_groups()]
        if self.ctx.dtype == torch.bfloat16:
            groups += ["gemm_small_m", "gemm_stream"]
            # the specialised attention kernels that this head size can reach (ops.paged_attention)
            group = self.num_heads // self.num_kv_heads
            if self.head_dim in (64, 128, 256) and group <= 16:
                groups.append("attention_decode")
            if self.head_dim in (64, 128) and group <= 16:
                groups.append("attention_prefill")
            if self.head_dim == 128 and not self.window and 128 % group == 0:
                groups.append("attention_prefill_tc")
        if self.ctx.dtype == torch.float32:
            groups.append("gemm_f32")
        return groups

    def step_choosers(self):
        """Into how many slices the split-KV decode kernel cuts the longest sequence's keys."""
        model = getattr(self.ops, "decode_slices_for", None)
        if model is None or self.ctx.dtype != torch.bfloat16 or self.head_dim not in (64, 128, 256):
            return {}
        nkv, D, window = self.num_kv_heads, self.head_dim, self.window
        return {self._slices_choice: lambda kv_lens: model(kv_lens, nkv, D, window)}

    def cache_spec(self):
        return KVLayerSpec(self.num_kv_heads, self.head_dim, self.window)

    def position_limit(self):
        return self.position.position_limit()

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        ops = self.ops
        T = h.shape[0]
        weight = self.qkv_weight if cache.writes else self.qkv_weight[: self.q_size]
        if self.qkv_bias_vec is None:
            qkv = ops.linear(h, weight)
        else:
            qkv = ops.linear(h, weight, bias=self.qkv_bias_vec[: weight.shape[0]])
        tables = self.position.rotation_tables()
        cos, sin = tables if tables is not None else (None, None)
        block_table = step.block_tables[cache.paged_index]
        ctx_out = torch.empty((T, self.q_size), dtype=h.dtype, device=h.device)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        slices = step.choices.get(self._slices_choice)
        fusable = getattr(ops, "decode_new_token_ok", None)
        if (fusable is not None and step.decode_only and cache.writes
                and fusable(qkv, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                            cos=cos, q_weight=self.q_norm_weight, k_weight=self.k_norm_weight)):
            # one kernel: norm and rotation of the newest q and k, cache write, split-KV attention
            width = step.captured_width
            ops.paged_attention_decode(
                qkv, qkv.stride(0), num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                head_dim=self.head_dim, k_pages=cache.k_pages, v_pages=cache.v_pages, block_table=block_table,
                kv_lens=step.kv_lens, cu_seqlens=step.cu_seqlens, out=ctx_out, page_size=cache.page_size,
                scale=self.scale, window=self.window, num_seqs=step.num_seqs,
                max_kv_len=width * cache.page_size or step.max_kv_len,
                new_token=dict(q_weight=self.q_norm_weight, k_weight=self.k_norm_weight, eps=eps, cos=cos, sin=sin,
                               pairing=self.pairing),
                num_splits=slices, longest=step.kv_longest, step=step)
            return self._project_out(ctx_out)
        ops.qk_norm_rope_store(
            qkv, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
            q_weight=self.q_norm_weight, k_weight=self.k_norm_weight,
            eps=eps, cos=cos, sin=sin,
            positions=step.positions, token_seq=step.token_seq, block_table=block_table,
            k_pages=cache.k_pages, v_pages=cache.v_pages, page_size=cache.page_size, write_kv=cache.writes,
            pairing=self.pairing)
        ops.paged_attention(
            qkv, qkv.stride(0), num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
            head_dim=self.head_dim, k_pages=cache.k_pages, v_pages=cache.v_pages, block_table=block_table,
            token_seq=step.token_seq, positions=step.positions, out=ctx_out, page_size=cache.page_size,
            scale=self.scale, window=self.window, step=step, **({"decode_slices": slices} if slices else {}))
        return self._project_out(ctx_out)

    def _project_out(self, ctx_out: torch.Tensor) -> torch.Tensor:
        if self.o_bias_vec is not None:
            return self.ops.linear(ctx_out, self.o_weight, bias=self.o_bias_vec)
        return self.ops.linear(ctx_out, self.o_weight, partial_sums=self.partial_sums_ok)


register_part("mixer", "paged_attention", PagedAttention)
