"""The decoder: embedding, blocks in their run order, final norm, output head.

Built from a :class:`ModelSpec`; knows no architecture by name.  Parity for the
Qwen3 instance: qwen3_runtime/models/qwen3.py:190-266.
"""

from __future__ import annotations

import torch

from ..cache.layout import CacheLayout
from ..config.spec import ModelSpec
from .base import BuildContext, ParamSpec, ResidualStream, StepContext, build_part


class DecoderModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        self.ops = ctx.ops
        self.blocks = [build_part("block", b, ctx) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        # tell each block which norms take its output: the entry norm of whatever runs after
        # it (a block may run more than once), or the final norm
        takers: dict[int, list] = {}
        for i, run in enumerate(spec.order):
            after = self.blocks[spec.order[i + 1].block] if i + 1 < len(spec.order) else None
            norm = self.final_norm if after is None else getattr(after, "entry_norm", None)
            takers.setdefault(run.block, []).append(norm)
        for index, norms in takers.items():
            block = self.blocks[index]
            if hasattr(block, "exit_to") and all(n is not None for n in norms):
                block.exit_to(norms)
        self.choosers: dict = {}
        for block in self.blocks:
            self.choosers.update(block.step_choosers())
        self.embed: torch.Tensor | None = None
        self.head: torch.Tensor | None = None
        self.loaded = False

    # ---- tensors ----------------------------------------------------------------------
    def expected_tensors(self) -> dict[str, ParamSpec]:
        """Every stored tensor by its checkpoint name, in a fixed order."""
        s = self.spec
        out: dict[str, ParamSpec] = {s.embed_name: ParamSpec((s.vocab_size, s.hidden_size))}
        for i, block in enumerate(self.blocks):
            prefix = s.block_prefix.format(index=i)
            for name, ps in block.param_specs().items():
                out[prefix + name] = ps
        for name, ps in self.final_norm.param_specs().items():
            out[s.final_norm_prefix + name] = ps
        if not s.tie_word_embeddings:
            out[s.head_name] = ParamSpec((s.vocab_size, s.hidden_size))
        return out

    def ignorable_tensors(self) -> set[str]:
        """Names a checkpoint may hold that the model does not read (a tied model's copy
        of the head, utils/loader.py:39-40)."""
        return {self.spec.head_name} if self.spec.tie_word_embeddings else set()

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """``tensors``: every expected name -> tensor already on the device."""
        self.load_from(tensors.__getitem__)

    def load_from(self, fetch) -> None:
        """``fetch(name)`` returns the named tensor on the device.  Tensors are asked for part by
        part and let go as soon as the part has taken (and possibly fused) them, so that beside
        the model's own tensors only one block's stored tensors are alive at any time."""
        s = self.spec
        self.embed = fetch(s.embed_name).contiguous()
        for i, block in enumerate(self.blocks):
            prefix = s.block_prefix.format(index=i)
            block.load({name: fetch(prefix + name) for name in block.param_specs()})
        self.final_norm.load({name: fetch(s.final_norm_prefix + name) for name in self.final_norm.param_specs()})
        self.head = self.embed if s.tie_word_embeddings else fetch(s.head_name).contiguous()
        self.loaded = True

    def kernel_groups(self) -> list[str]:
        groups = {"norm"}
        for part in [*self.blocks, self.final_norm]:
            groups.update(part.kernel_groups())
        return sorted(groups)

    def position_limit(self) -> int | None:
        """The longest sequence every part can serve (None: no part sets a limit)."""
        limits = [n for n in (b.position_limit() for b in self.blocks) if n is not None]
        return min(limits) if limits else None

    # ---- cache ------------------------------------------------------------------------
    def cache_layout(self) -> CacheLayout:
        specs = {}
        for run in self.spec.order:
            if run.writes:
                specs[run.cache] = self.blocks[run.block].cache_spec()
        for run in self.spec.order:
            if not run.writes and specs[run.cache] != self.blocks[run.block].cache_spec():
                raise ValueError(f"a run entry reads cache layer {run.cache} whose layout differs from its own")
        return CacheLayout(specs)

    def step_choices(self, kv_lens: list[int]) -> dict:
        """What the parts' choosers answer for a step of one-token sequences with these lengths."""
        return {name: fn(kv_lens) for name, fn in self.choosers.items()} if kv_lens else {}

    # ---- one step -----------------------------------------------------------------------
    def forward(self, step: StepContext, storage) -> torch.Tensor | None:
        """Run the step's tokens through every run entry; float32 logits ``[R, V]`` at
        ``step.logit_rows`` (None when no logits are wanted)."""
        s = self.spec
        stream = ResidualStream(step.num_tokens, s.hidden_size, ids=step.token_ids, table=self.embed)
        for run in s.order:
            self.blocks[run.block].forward(stream, step, storage.view(run.cache, run.writes))
        if step.num_logit_rows == 0:
            return None
        h = self.final_norm.add_norm(stream, rows=step.logit_rows, num_rows=step.num_logit_rows)
        logits = self.ops.linear(h, self.head, out_dtype=torch.float32)
        if s.logit_scale != 1.0 or s.logit_softcap is not None:
            self.ops.logit_scale_cap(logits, s.logit_scale, s.logit_softcap or 0.0)
        return logits
