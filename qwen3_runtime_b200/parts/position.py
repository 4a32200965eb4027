"""Position encodings.  ``rope_neox``: rotate-half rotary embedding with fp32 tables
(qwen3_runtime/layers/rope.py:7-27).  ``none``: no position encoding.

A position part does not run a kernel of its own: the mixer applies it inside its
fused q/k kernel and asks the part for what that kernel needs.  The interface is

* ``style``: ``"none"`` or ``"rotary"``;
* for ``"rotary"``: :meth:`rotation_tables` -> ``(cos, sin)``, float32 ``[positions, pairs]``
  with the angle of rotation pair ``i`` at position ``p`` in ``[p, i]``; and ``pairing``, which
  two elements of a head pair ``i`` is: ``"half"`` -- ``(i, i + pairs)`` -- or
  ``"interleaved"`` -- ``(2i, 2i + 1)``.  ``2 * pairs`` may be less than the head size
  (partial rotary: the rest of the head is left as it is).

Any encoding that rotates pairs of elements by angles that depend on the absolute position
only (other frequency schedules, scaled or slowed positions, partial rotation, either
pairing) is such a part and needs no kernel change.
"""

from __future__ import annotations

import torch

from .base import BuildContext, Part, register_part


class NoPosition(Part):
    category = "position"
    style = "none"

    def rotation_tables(self):
        return None


class RotaryNeox(Part):
    category = "position"
    style = "rotary"
    pairing = "half"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be a positive even number")

    def kernel_groups(self):
        return ["rope_kv"]

    def position_limit(self):
        return self.max_positions

    def inverse_frequencies(self) -> torch.Tensor:
        """inv_j = 1 / theta^(2j / rotary_dim), computed on the host in float32 exactly as
        the reference does (layers/rope.py:18), so both sides rotate by the same angles."""
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float) / self.rotary_dim
        return 1.0 / (self.theta ** exponents)

    def rotation_tables(self):
        key = ("rope_neox", self.rotary_dim, self.theta, self.max_positions)
        if key not in self.ctx.shared:
            inv = self.inverse_frequencies().to(self.ctx.device)
            self.ctx.shared[key] = self.ops.rope_table(inv, self.max_positions)
        return self.ctx.shared[key]


register_part("position", "none", NoPosition)
register_part("position", "rope_neox", RotaryNeox)
