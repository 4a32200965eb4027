"""Arrangement of parts in a block.  ``pre_norm``: x += mixer(norm(x)); x += ff(norm(x))
(qwen3_runtime/models/qwen3.py:159-187, where each add is fused with the next norm)."""

from __future__ import annotations

from .base import BuildContext, Part, ResidualStream, StepContext, build_part, register_part


class PreNormBlock(Part):
    category = "block"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.mixer = build_part("mixer", spec["mixer"], ctx)
        self.feed_forward = build_part("feed_forward", spec["feed_forward"], ctx)
        self.mixer_norm = build_part("norm", spec["mixer_norm"], ctx)
        self.feed_forward_norm = build_part("norm", spec["feed_forward_norm"], ctx)
        self.children = {
            spec.get("mixer_prefix", "mixer."): self.mixer,
            spec.get("feed_forward_prefix", "feed_forward."): self.feed_forward,
            spec.get("mixer_norm_prefix", "mixer_norm."): self.mixer_norm,
            spec.get("feed_forward_norm_prefix", "feed_forward_norm."): self.feed_forward_norm,
        }
        # the mixer's output meets this block's second norm; where the feed-forward's output
        # goes only the model knows (exit_to)
        self.entry_norm = self.mixer_norm
        self.mixer.partial_sums_ok = self.feed_forward_norm.adds_partial_sums

    def exit_to(self, norms) -> None:
        """``norms``: every norm that may fold this block's output into the residual sum."""
        self.feed_forward.partial_sums_ok = all(n.adds_partial_sums for n in norms)

    def param_specs(self):
        return {prefix + name: ps for prefix, part in self.children.items()
                for name, ps in part.param_specs().items()}

    def load(self, tensors):
        for prefix, part in self.children.items():
            part.load({name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)})

    def kernel_groups(self):
        return [g for part in self.children.values() for g in part.kernel_groups()]

    def step_choosers(self):
        return {name: fn for part in self.children.values() for name, fn in part.step_choosers().items()}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def position_limit(self):
        limits = [n for n in (part.position_limit() for part in self.children.values()) if n is not None]
        return min(limits) if limits else None

    def forward(self, stream: ResidualStream, step: StepContext, cache) -> None:
        h = self.mixer_norm.add_norm(stream)
        stream.pending = self.mixer.forward(h, step, cache)
        h = self.feed_forward_norm.add_norm(stream)
        stream.pending = self.feed_forward.forward(h, step)


register_part("block", "pre_norm", PreNormBlock)
