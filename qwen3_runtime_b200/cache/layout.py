"""From what each cache layer needs to groups, and from groups to device tensors.

A mixer declares what its cache layer needs with a :class:`KVLayerSpec` (paged
keys and values, optionally only a window of them) or a :class:`StateLayerSpec`
(a fixed-size slot per request).  Layers with the same needs form one group; a
paged group has one page pool and one block table per request for all its
layers, so one page id addresses that page in every layer of the group
(as in qwen3_runtime/kv/paged.py:63-72, where the only group is "all layers").

Device layout of a paged group: ``[layers, 2 (K,V), pages + 1, kv_heads,
page_size, head_dim]`` -- per (page, head) a contiguous ``[page_size, head_dim]``
tile, so one key/value tile of a head is a single contiguous read.  The extra
last page is a scratch page that padded rows of a captured decode step write to.
"""

from __future__ import annotations

from dataclasses import dataclass

from .manager import GroupSpec


@dataclass(frozen=True)
class KVLayerSpec:
    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateLayerSpec:
    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class GroupLayout:
    spec: GroupSpec
    layer_spec: object  # KVLayerSpec | StateLayerSpec
    cache_ids: tuple[int, ...]  # cache layers of this group, in order


class CacheLayout:
    """Groups for a model: ``layer_specs`` maps cache layer id -> its spec (or None)."""

    def __init__(self, layer_specs: dict[int, object]):
        buckets: dict[object, list[int]] = {}
        for cache_id in sorted(layer_specs):
            spec = layer_specs[cache_id]
            if spec is None:
                continue
            buckets.setdefault(spec, []).append(cache_id)
        self.groups: list[GroupLayout] = []
        for spec, ids in buckets.items():
            if isinstance(spec, KVLayerSpec):
                gs = GroupSpec("window", spec.window) if spec.window else GroupSpec("full")
            elif isinstance(spec, StateLayerSpec):
                gs = GroupSpec("state")
            else:
                raise TypeError(f"unknown cache layer spec {spec!r}")
            self.groups.append(GroupLayout(gs, spec, tuple(ids)))
        if not any(g.spec.paged for g in self.groups):
            # a model without paged layers still gets block tables of width zero
            pass
        self.where: dict[int, tuple[int, int]] = {}
        for gi, g in enumerate(self.groups):
            for li, cache_id in enumerate(g.cache_ids):
                self.where[cache_id] = (gi, li)
        self.paged_groups = [gi for gi, g in enumerate(self.groups) if g.spec.paged]

    @property
    def group_specs(self) -> list[GroupSpec]:
        return [g.spec for g in self.groups]

    def page_bytes(self, page_size: int, dtype_bytes: int) -> list[int]:
        """Bytes of one page (all layers, K and V) for each paged group."""
        out = []
        for gi in self.paged_groups:
            g = self.groups[gi]
            s: KVLayerSpec = g.layer_spec
            out.append(len(g.cache_ids) * 2 * s.num_kv_heads * s.head_dim * page_size * dtype_bytes)
        return out

    def token_bytes(self, dtype_bytes: int) -> int:
        """Bytes of keys and values one token adds over all paged groups
        (qwen3_runtime/engine/memory.py:8-10)."""
        return sum(self.page_bytes(1, dtype_bytes))

    def pages_for_budget(self, budget_bytes: int, page_size: int, dtype_bytes: int, *,
                         max_num_seqs: int | None = None, max_step_tokens: int | None = None) -> list[int]:
        """Pages for each paged group that together fit in ``budget_bytes``
        (qwen3_runtime/engine/memory.py:17-27 for the single group of the reference).

        A group that keeps every key needs pages in proportion to the tokens held, so such
        groups all get the same count.  A window group never holds more, per request, than
        its window plus the portion being computed; with ``max_num_seqs`` and
        ``max_step_tokens`` given it gets no more pages than that, and what it leaves goes to
        the groups that keep everything."""
        per = self.page_bytes(page_size, dtype_bytes)
        if not per or sum(per) <= 0:
            return [0 for _ in per]
        equal = int(budget_bytes // sum(per))
        counts = [equal] * len(per)
        if max_num_seqs is None or max_step_tokens is None:
            return counts
        spent, open_bytes = 0, 0
        for i, gi in enumerate(self.paged_groups):
            window = self.groups[gi].spec.window
            if window:
                cap = max_num_seqs * (-(-(window + max_step_tokens) // page_size) + 2)
                counts[i] = min(equal, cap)
                spent += counts[i] * per[i]
            else:
                open_bytes += per[i]
        if open_bytes:
            full = int((budget_bytes - spent) // open_bytes)
            counts = [c if self.groups[gi].spec.window else full for c, gi in zip(counts, self.paged_groups)]
        return counts
