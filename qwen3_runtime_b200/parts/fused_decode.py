"""All layers of a decode step as one kernel, for models whose layers have the one shape that
kernel is built for.

``plan_fused_decode(model)`` looks at the parts a model was put together from.  If every block
is a ``pre_norm`` arrangement of an RMSNorm, paged grouped-query attention (no window, no
biases, rotation over the whole head or none), another RMSNorm and a SwiGLU feed-forward
(no biases), all of one size, and the blocks run once each in order with a cache layer of
their own, it returns a :class:`FusedDecode`; otherwise None, and the model steps part by
part as always.  The parts themselves know nothing of this: it is a property of an
arrangement, found from outside.  :class:`DecoderModel` asks for it once after loading and
uses it for steps in which every sequence brings one token and there are at most as many
sequences as the kernel takes (csrc/decode_step.cu: 16).
"""

from __future__ import annotations

import torch

from .attention import PagedAttention
from .base import StepContext
from .block import PreNormBlock
from .feed_forward import GatedMLP
from .norm import RMSNorm


class FusedDecode:
    def __init__(self, model, sizes: dict, scratch_bytes: list[int]):
        self.model = model
        self.ops = model.ops
        self.sizes = sizes
        dev = model.ctx.device
        tokens = self.ops.DECODE_STEP_TOKENS
        H, I = sizes["hidden_size"], sizes["intermediate_size"]
        q_width = sizes["num_heads"] * sizes["head_dim"]
        qkv_width = q_width + 2 * sizes["num_kv_heads"] * sizes["head_dim"]

        def raw(nbytes, dtype=torch.float32):
            return torch.zeros(max(1, nbytes // torch.empty((), dtype=dtype).element_size()), dtype=dtype, device=dev)

        self.resid = torch.zeros((tokens, H), dtype=torch.float32, device=dev)
        self.qkv = torch.zeros((tokens, qkv_width), dtype=torch.bfloat16, device=dev)
        self.ctx = torch.zeros((tokens, q_width), dtype=torch.bfloat16, device=dev)
        self.mid = torch.zeros((tokens, I), dtype=torch.bfloat16, device=dev)
        self.att_o = raw(scratch_bytes[0])
        self.att_lse = raw(scratch_bytes[1])
        self.att_tickets = raw(scratch_bytes[2], torch.int32)
        self.sumsq = raw(scratch_bytes[3])
        self.map_bytes = scratch_bytes[4]
        self.barrier = torch.zeros(1, dtype=torch.int32, device=dev)
        self.enabled = True
        self.steps = 0

    def applies(self, step: StepContext) -> bool:
        return self.enabled and step.decode_only and 0 < step.num_seqs <= self.ops.DECODE_STEP_TOKENS

    def _layer_table(self, storage):
        """Device table of the layers' pointers and the tensor maps of their pages; the pages belong
        to one cache storage, so both are made once per storage (False: the kernel does not take
        this cache's page size)."""
        made = getattr(storage, "_fused_decode_layers", None)
        if made is None:
            rows, k_pages, v_pages = [], [], []
            for run, block in zip(self.model.spec.order, self.model.blocks):
                view = storage.view(run.cache, True)
                k_pages.append(view.k_pages)
                v_pages.append(view.v_pages)
                mixer, ff = block.mixer, block.feed_forward
                rows.append([mixer.qkv_weight.data_ptr(), mixer.o_weight.data_ptr(), ff.gate_up_weight.data_ptr(),
                             ff.down_weight.data_ptr(), block.mixer_norm.weight.data_ptr(),
                             block.feed_forward_norm.weight.data_ptr(),
                             0 if mixer.q_norm_weight is None else mixer.q_norm_weight.data_ptr(),
                             0 if mixer.k_norm_weight is None else mixer.k_norm_weight.data_ptr(),
                             view.k_pages.data_ptr(), view.v_pages.data_ptr()])
            dev = self.model.ctx.device
            maps = torch.zeros(len(rows) * self.map_bytes, dtype=torch.uint8, device=dev)
            ok = self.ops.decode_step_maps(k_pages, v_pages, num_kv_heads=self.sizes["num_kv_heads"],
                                           page_size=storage.page_size, head_dim=self.sizes["head_dim"], out=maps)
            made = (torch.tensor(rows, dtype=torch.int64).to(dev), maps) if ok else False
            storage._fused_decode_layers = made
        return made

    def run(self, step: StepContext, storage) -> torch.Tensor | None:
        """The residual sum after the last layer, fp32 ``[tokens, H]`` (a view of a buffer that the
        next step overwrites), or None if the kernel refused the step."""
        s = self.sizes
        made = self._layer_table(storage)
        if made is False:
            return None
        mixer = self.model.blocks[0].mixer
        view = storage.view(self.model.spec.order[0].cache, True)
        tables = mixer.position.rotation_tables()
        cos, sin = tables if tables is not None else (None, None)
        ok = self.ops.decode_step(
            layers=made[0], maps=made[1], num_layers=len(self.model.blocks), num_tokens=step.num_seqs,
            hidden_size=s["hidden_size"], intermediate_size=s["intermediate_size"], num_heads=s["num_heads"],
            num_kv_heads=s["num_kv_heads"], head_dim=s["head_dim"], page_size=view.page_size,
            token_ids=step.token_ids, embed=self.model.embed, kv_lens=step.kv_lens,
            block_table=step.block_tables[view.paged_index], cos=cos, sin=sin, pairing=mixer.pairing,
            eps=s["eps"], qk_eps=s["qk_eps"], scale=mixer.scale, resid=self.resid, sumsq=self.sumsq, qkv=self.qkv,
            ctx=self.ctx, mid=self.mid, att_o=self.att_o, att_lse=self.att_lse, att_tickets=self.att_tickets,
            barrier=self.barrier, cost=self._cost(step) if self.ops.timing is not None else None)
        if not ok:
            return None
        self.steps += 1
        return self.resid[: step.num_seqs]


    def _cost(self, step: StepContext) -> tuple[float, float]:
        """(bytes, flops) of the step's layers: every layer weight once, every cached key and value."""
        s = self.sizes
        q = s["num_heads"] * s["head_dim"]
        kv = s["num_kv_heads"] * s["head_dim"]
        per_layer = s["hidden_size"] * (q + 2 * kv) + q * s["hidden_size"] + 3 * s["hidden_size"] * s["intermediate_size"]
        L = len(self.model.blocks)
        held = sum(step.host_kv_lens)
        return 2.0 * L * (per_layer + 2 * kv * held), 2.0 * L * per_layer * step.num_seqs


def plan_fused_decode(model) -> FusedDecode | None:
    ops = model.ops
    if model.ctx.dtype != torch.bfloat16 or not hasattr(ops, "decode_step_scratch") or model.ctx.device.type != "cuda":
        return None
    spec = model.spec
    if len(spec.order) != len(model.blocks) or any(
            run.block != i or not run.writes or run.cache != spec.order[i].cache or
            sum(r.cache == run.cache for r in spec.order) != 1 for i, run in enumerate(spec.order)):
        return None
    sizes = None
    for block in model.blocks:
        if type(block) is not PreNormBlock:
            return None
        mixer, ff, n1, n2 = block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm
        if type(mixer) is not PagedAttention or type(ff) is not GatedMLP or type(n1) is not RMSNorm or type(n2) is not RMSNorm:
            return None
        if mixer.window or mixer.qkv_bias or mixer.o_bias or ff.down_bias or n1.eps != n2.eps:
            return None
        if mixer.position.style not in ("none", "rotary"):
            return None
        tables = mixer.position.rotation_tables() if mixer.position.style == "rotary" else None
        if tables is not None and 2 * tables[0].shape[1] != mixer.head_dim:
            return None
        if (mixer.q_norm_weight is None) != (mixer.k_norm_weight is None):
            return None
        mine = dict(hidden_size=mixer.hidden_size, intermediate_size=ff.intermediate_size, num_heads=mixer.num_heads,
                    num_kv_heads=mixer.num_kv_heads, head_dim=mixer.head_dim, eps=n1.eps,
                    qk_eps=mixer.qk_norm_eps if mixer.qk_norm_eps is not None else 0.0, scale=mixer.scale,
                    pairing=mixer.pairing, position=id(tables[0]) if tables is not None else None)
        if ff.hidden_size != mixer.hidden_size or n1.size != mixer.hidden_size or n2.size != mixer.hidden_size:
            return None
        if sizes is not None and mine != sizes:
            return None
        sizes = mine
    if sizes is None or model.cache_layout().paged_groups != [0] or len(model.cache_layout().groups) != 1:
        return None
    scratch = ops.decode_step_scratch(hidden_size=sizes["hidden_size"], intermediate_size=sizes["intermediate_size"],
                                      num_heads=sizes["num_heads"], num_kv_heads=sizes["num_kv_heads"],
                                      head_dim=sizes["head_dim"])
    if scratch is None:
        return None
    return FusedDecode(model, sizes, scratch)
