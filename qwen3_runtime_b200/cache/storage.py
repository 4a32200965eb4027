"""Device tensors behind the cache groups (see layout.py for the layout)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .layout import CacheLayout, KVLayerSpec, StateLayerSpec


@dataclass
class CacheLayerView:
    """What a mixer sees of its cache layer during one step."""

    group: int  # index into CacheLayout.groups
    paged_index: int | None  # index among paged groups (selects the block table)
    page_size: int
    window: int | None
    k_pages: torch.Tensor | None  # [pages + 1, kv_heads, page_size, head_dim]
    v_pages: torch.Tensor | None
    state: torch.Tensor | None  # [slots + 1, *shape]
    writes: bool = True


class CacheStorage:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages: int | list[int], num_slots: int,
                 dtype: torch.dtype, device: torch.device | str):
        """``num_pages``: pages of every paged group, or one count per paged group."""
        self.layout = layout
        self.page_size = page_size
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(layout.paged_groups)
        if len(num_pages) != len(layout.paged_groups):
            raise ValueError("one page count per paged group is required")
        self.num_pages = list(num_pages)
        self.num_slots = num_slots
        # the extra page of each paged group, which padded rows write to
        self.scratch_page = tuple(self.num_pages)
        self.scratch_slot = num_slots
        self.tensors: list[torch.Tensor] = []
        for gi, g in enumerate(layout.groups):
            s = g.layer_spec
            if isinstance(s, KVLayerSpec):
                pages = self.num_pages[layout.paged_groups.index(gi)]
                shape = (len(g.cache_ids), 2, pages + 1, s.num_kv_heads, page_size, s.head_dim)
                self.tensors.append(torch.zeros(shape, dtype=dtype, device=device))
            else:
                assert isinstance(s, StateLayerSpec)
                shape = (len(g.cache_ids), num_slots + 1, *s.shape)
                self.tensors.append(torch.zeros(shape, dtype=getattr(torch, s.dtype), device=device))

    def view(self, cache_id: int, writes: bool = True) -> CacheLayerView | None:
        if cache_id not in self.layout.where:
            return None
        gi, li = self.layout.where[cache_id]
        g = self.layout.groups[gi]
        t = self.tensors[gi]
        if g.spec.paged:
            return CacheLayerView(gi, self.layout.paged_groups.index(gi), self.page_size, g.spec.window,
                                  t[li, 0], t[li, 1], None, writes)
        return CacheLayerView(gi, None, self.page_size, None, None, None, t[li], writes)

    def zero_state_slots(self, slots: list[int]) -> None:
        """Fixed-size state starts from zero when a request starts or restarts."""
        if not slots:
            return
        idx = None
        for g, t in zip(self.layout.groups, self.tensors):
            if g.spec.paged:
                continue
            if idx is None:
                idx = torch.tensor(slots, dtype=torch.long, device=t.device)
            t.index_fill_(1, idx, 0)

    def poison_pages(self, paged_index: int, pages: list[int], value: float = float("nan")) -> None:
        """Overwrite pages (tests: a page that is used again must not leak old contents)."""
        t = self.tensors[self.layout.paged_groups[paged_index]]
        if pages:
            t[:, :, torch.tensor(pages, dtype=torch.long, device=t.device)] = value

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)
