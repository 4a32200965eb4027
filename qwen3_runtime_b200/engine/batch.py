"""From ``(request, its next tokens, wanted places)`` to the device arrays of a step.

All integer metadata of a step is packed into one pinned host buffer and copied to
the device with a single transfer; the parts see slices of that device buffer.
Parity: qwen3_runtime/engine/batch.py:45-60 (ids, positions, cu_seqlens, kv_lens,
block tables, rows that get logits) -- here as int32 arrays on the device, and with
explicit wanted places instead of "the last row if the request caught up".
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..parts.base import StepContext


class BatchError(ValueError):
    pass


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` (they follow what the cache
    already holds for it) and ``want``, indices into ``tokens`` whose logits are asked for."""

    cache: RequestCache
    tokens: list[int]
    want: list[int]


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class BatchBuilder:
    RING = 4  # pinned staging buffers in flight

    def __init__(self, cache: CacheManager, device, *, vocab_size: int, max_positions: int):
        self.cache = cache
        self.device = device
        self.vocab_size = vocab_size
        self.max_positions = max_positions
        self._host: list[torch.Tensor] = []
        self._events: list[torch.cuda.Event | None] = []
        self._dev: torch.Tensor | None = None
        self._turn = 0
        self._capacity = 0
        self.pin = torch.device(device).type == "cuda"
        self._last_decode: dict | None = None  # what the last captured-size decode step packed
        # device view of the real token ids of the step packed last: whoever has those ids on the
        # device only (tokens sampled by a step whose result the host has not read yet) writes
        # them here after packing and before the step runs
        self.last_token_ids: torch.Tensor | None = None

    def _buffers(self, need: int):
        if need > self._capacity:
            self._capacity = max(4096, 1 << (need - 1).bit_length())
            self._host = [torch.zeros(self._capacity, dtype=torch.int32, pin_memory=self.pin)
                          for _ in range(self.RING)]
            self._events = [None] * self.RING
            self._dev = torch.empty(self._capacity, dtype=torch.int32, device=self.device)
        self._turn = (self._turn + 1) % self.RING
        ev = self._events[self._turn]
        if ev is not None:
            ev.synchronize()
        return self._host[self._turn], self._dev

    def _continue_decode(self, entries, pad_to, table_width, scratch_page, scratch_slot, device_buffer) -> bool:
        """The same requests as in the last packed step, one more token each, into the same
        device buffer: only token ids, positions, lengths and block-table rows that grew
        change.  Updates the kept image of the buffer and copies it; False if the step is not
        such a continuation (the caller then packs it in full)."""
        last = self._last_decode
        if (last is None or last["device_buffer"] is not device_buffer or len(entries) != len(last["caches"])
                or last["key"] != (pad_to, table_width, scratch_page, scratch_slot)):
            return False
        for e, c in zip(entries, last["caches"]):
            if e.cache is not c or len(e.tokens) != 1:
                return False
        n = len(entries)
        toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=n)
        starts = np.fromiter((e.cache.num_computed for e in entries), dtype=np.int32, count=n)
        reserved = np.fromiter((e.cache.num_reserved for e in entries), dtype=np.int32, count=n)
        if not np.array_equal(starts, last["starts"] + 1):
            return False  # not exactly one token further than the step this image was packed for
        if (toks.min() < 0 or toks.max() >= self.vocab_size or (starts + 1 > reserved).any()
                or int(starts.max()) + 1 > self.max_positions or any(e.want not in ([0], []) for e in entries)):
            return False  # the full path words the error
        image, sections, width, B = last["image"], last["sections"], last["width"], last["B"]

        def sec(name):
            o, s = sections[name]
            return image[o:o + s]

        sec("ids")[:n] = toks
        sec("pos")[:n] = starts
        sec("kv")[:n] = starts + 1
        sec("kvmax")[0] = int(starts.max()) + 1
        for g, windowed in enumerate(last["windowed"]):
            bt = None
            for b, e in enumerate(entries):
                size = len(e.cache.tables[g])
                if windowed or size != last["table_lens"][b][g]:
                    if size > width:
                        return False
                    if bt is None:
                        bt = sec(f"bt{g}").reshape(B, width)
                    bt[b, :] = scratch_page[g]
                    bt[b, :size] = e.cache.table_array(g)
                    last["table_lens"][b][g] = size
        last["starts"] = starts
        off = last["off"]
        host, _ = self._buffers(off)
        views = last.setdefault("views", {})
        view = views.get(self._turn)
        if view is None or view[0] is not host:  # slices of the staging buffers, made once
            view = views[self._turn] = (host, host.numpy()[:off], host[:off], device_buffer[:off])
        view[1][:] = image
        view[3].copy_(view[2], non_blocking=True)
        self.last_token_ids = last["ids_view"]
        if self.pin:
            ev = self._events[self._turn] or torch.cuda.Event()
            ev.record()
            self._events[self._turn] = ev
        return True

    def build(self, entries: list[StepEntry], *, pad_to: int | None = None, table_width: int | None = None,
              scratch_page: int | tuple[int, ...] = 0, scratch_slot: int = 0,
              device_buffer: torch.Tensor | None = None,
              all_rows: bool = False, need_context: bool = True) -> StepContext | None:
        """Pack a step.  ``pad_to`` appends dummy one-token sequences (writing to the
        scratch page and the scratch state slot) so that a decode batch fills a captured batch
        size; with no entries at all the step consists of such rows only.  ``table_width``
        fixes the block-table width; ``device_buffer`` is a preallocated int32 buffer that
        the metadata is copied into (captured steps read from fixed addresses).
        ``scratch_page``: the page that padded rows and unused block-table entries name, one id
        for every paged group or one per group.
        ``need_context=False``: the caller only wants the device buffer filled (a replayed
        graph reads it) and gets no :class:`StepContext`."""
        if not entries and not pad_to:
            raise BatchError("a step needs at least one entry")
        if not isinstance(scratch_page, tuple):  # one scratch page id per paged group
            scratch_page = (int(scratch_page),) * len(self.cache.paged_groups)
        if not need_context and device_buffer is not None and all_rows:
            if self._continue_decode(entries, pad_to, table_width, scratch_page, scratch_slot, device_buffer):
                return None
        ps = self.cache.page_size
        n_paged = len(self.cache.paged_groups)
        B_real = len(entries)
        B = max(B_real, pad_to or 0)
        ids: list[int] = []
        lens = []
        for e in entries:
            n = len(e.tokens)
            if n < 1:
                raise BatchError(f"request {e.cache.request_id!r} brings no tokens")
            start = e.cache.num_computed
            if start + n > e.cache.num_reserved:
                raise BatchError(f"request {e.cache.request_id!r}: pages are reserved for "
                                 f"{e.cache.num_reserved} tokens, the step needs {start + n}")
            if start + n > self.max_positions:
                raise BatchError(f"request {e.cache.request_id!r} would reach position {start + n - 1}; "
                                 f"the model's position encoding covers {self.max_positions}")
            for w in e.want:
                if not 0 <= w < n:
                    raise BatchError(f"request {e.cache.request_id!r}: wanted place {w} is outside its {n} tokens")
            ids.extend(e.tokens)
            lens.append(n)
        T_real = len(ids)
        T = T_real + (B - B_real)
        ids_np = np.asarray(ids, dtype=np.int64)
        if ids_np.size and (ids_np.min() < 0 or ids_np.max() >= self.vocab_size):
            bad = int(ids_np[(ids_np < 0) | (ids_np >= self.vocab_size)][0])
            raise BatchError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        width = max(1, max((len(t) for e in entries for t in e.cache.tables), default=1))
        if table_width is not None:
            if table_width < width:
                raise BatchError("fixed block-table width is smaller than a request's table")
            width = table_width
        else:
            width = _round_up(width, 8)
        rows: list[int] = []
        # section offsets inside the int32 buffer (each 4-int aligned => 16-byte aligned)
        off, sections = 0, {}
        for name, size in (("ids", T), ("pos", T), ("seq", T), ("cu", B + 1), ("kv", B), ("kvmax", 1), ("slot", B),
                           ("rows", T), ("single", B), *[(f"bt{g}", B * width) for g in range(n_paged)]):
            sections[name] = (off, size)
            off += _round_up(size, 4)
        host, dev = self._buffers(off)
        if device_buffer is not None:
            if device_buffer.numel() < off:
                raise BatchError("preallocated step buffer is too small")
            dev = device_buffer
        h = host.numpy()

        def sec(name):
            o, s = sections[name]
            return h[o:o + s]

        sec("ids")[:T_real] = ids_np
        sec("ids")[T_real:] = 0
        pos, seq, cu, kv, slot = sec("pos"), sec("seq"), sec("cu"), sec("kv"), sec("slot")
        starts = np.fromiter((e.cache.num_computed for e in entries), dtype=np.int32, count=B_real)
        lens_np = np.asarray(lens, dtype=np.int32)
        cu[0] = 0
        np.cumsum(lens_np, out=cu[1:B_real + 1])
        kv[:B_real] = starts + lens_np
        slot[:B_real] = np.fromiter((e.cache.slot for e in entries), dtype=np.int32, count=B_real)
        if T_real == B_real:  # every entry brings one token
            pos[:T_real] = starts
            seq[:T_real] = np.arange(B_real, dtype=np.int32)
        else:
            seq[:T_real] = np.repeat(np.arange(B_real, dtype=np.int32), lens_np)
            pos[:T_real] = np.arange(T_real, dtype=np.int32) - np.repeat(cu[:B_real] - starts, lens_np)
        for e, first in zip(entries, cu[:B_real].tolist()):
            if e.want:
                rows.extend(first + w for w in e.want)
        for g in range(n_paged):
            bt = sec(f"bt{g}").reshape(B, width)
            bt[:] = scratch_page[g]
            for b, e in enumerate(entries):
                arr = e.cache.table_array(g)
                bt[b, : arr.size] = arr
        t = T_real
        for b in range(B_real, B):  # padding rows: one token at position 0 of the scratch page
            pos[t] = 0
            seq[t] = b
            t += 1
            cu[b + 1] = t
            kv[b] = 1
            slot[b] = scratch_slot
        sec("kvmax")[0] = kv[:B].max()
        singles = [b for b, n in enumerate(lens) if n == 1] + list(range(B_real, B))
        sec("single")[:len(singles)] = singles
        if all_rows:
            rows_np = np.arange(T, dtype=np.int32)
        else:
            rows_np = np.asarray(rows, dtype=np.int32)
        R = int(rows_np.size)
        sec("rows")[:R] = rows_np
        dev[:off].copy_(host[:off], non_blocking=True)
        self.last_token_ids = dev[sections["ids"][0]:sections["ids"][0] + T_real]
        if self.pin:
            ev = self._events[self._turn] or torch.cuda.Event()
            ev.record()
            self._events[self._turn] = ev
        self._last_decode = None
        if device_buffer is not None and all_rows and T_real == B_real and B_real > 0:
            windowed = [self.cache.groups[g].window is not None for g in self.cache.paged_groups]
            self._last_decode = dict(
                caches=[e.cache for e in entries], key=(pad_to, table_width, scratch_page, scratch_slot),
                device_buffer=device_buffer, off=off, width=width, B=B, sections=sections, image=h[:off].copy(),
                table_lens=[[len(t) for t in e.cache.tables] for e in entries], windowed=windowed, starts=starts.copy(),
                ids_view=self.last_token_ids)
        if not need_context:
            return None

        def dsec(name, size=None):
            o, s = sections[name]
            return dev[o:o + (s if size is None else size)]

        return StepContext(
            num_tokens=T, num_seqs=B,
            token_ids=dsec("ids"), positions=dsec("pos"), token_seq=dsec("seq"), cu_seqlens=dsec("cu"),
            kv_lens=dsec("kv"), kv_longest=dsec("kvmax"), state_slots=dsec("slot"),
            block_tables=[dsec(f"bt{g}").view(B, width) for g in range(n_paged)],
            logit_rows=dsec("rows", R), num_logit_rows=R,
            max_query_len=max(lens, default=1), max_kv_len=int(kv[:B].max()),
            decode_only=all(n == 1 for n in lens),
            single_seqs=dsec("single", len(singles)), num_single=len(singles),
            host_cu_seqlens=[int(x) for x in cu], host_kv_lens=[int(x) for x in kv[:B]],
        )
