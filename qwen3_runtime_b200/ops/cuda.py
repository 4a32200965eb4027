"""The kernel table of the engine: thin Python wrappers over the ``extern "C"``
launchers in ``csrc/``.

There is one implementation per operation and no fallback: constructing
:class:`CudaOps` without a CUDA device, or without a working nvcc to build the
kernels, raises.  Wrappers check sizes and refuse, with a clear message, what a
kernel does not support; they never substitute another code path silently.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import build

_CODES = {1: "unsupported size or option", 2: "CUDA launch failed", 3: "bad argument"}


class KernelError(RuntimeError):
    pass


class KernelsUnavailable(RuntimeError):
    pass


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


def _check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: {_CODES.get(code, code)}")


_SIGNATURES = {
    "norm": {
        "q3_fused_norm": [c_int, c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "q3_silu_mul": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "q3_add_bias": [c_int, c_void_p, c_long, c_void_p, c_int, c_int, c_void_p],
        "q3_logit_scale_cap": [c_void_p, c_long, c_float, c_float, c_void_p],
    },
    "rope_kv": {
        "q3_qk_norm_rope_store": [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                  c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "q3_rope_table": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    },
    "attention_generic": {
        "q3_paged_attention_generic": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                       c_void_p],
    },
    "attention_decode": {
        "q3_paged_attention_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "q3_paged_attention_decode_fused": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                            c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_float,
                                            c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    },
    "attention_prefill": {
        "q3_paged_attention_prefill": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                       c_void_p],
    },
    "attention_prefill_tc": {
        "q3_paged_attention_prefill_tc": [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_long, c_void_p, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_int, c_void_p, c_void_p],
    },
    "gemm_f32": {
        "q3_gemm_f32": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_small_m": {
        "q3_gemm_small_m": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_stream": {
        "q3_gemm_stream": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p],
        "q3_gemm_stream_parts": [c_int, c_int, c_int],
        "q3_gemm_stream_partial": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p],
    },
    "gemm_tcgen05": {
        "q3_gemm_tcgen05": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                            c_void_p],
        "q3_gemm_tcgen05_pair": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p],
    },
    "sampling": {
        "q3_argmax": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "q3_sample": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_void_p],
        "q3_bias_penalty": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_float,
                            c_float, c_void_p],
        "q3_bias_penalty_rows": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p],
        "q3_filter": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    },
}


class _Span:
    """CUDA events around one launch, appended to the kernel table's timing records."""

    def __init__(self, ops, what: str):
        self.ops, self.what = ops, what

    def __enter__(self):
        self.start, self.stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.stop.record()
        nbytes, flops, tag = self.ops._cost
        self.ops._cost = (0, 0, "")
        self.ops.timing.append((self.what + tag, self.start, self.stop, nbytes, flops))
        return False


class CudaOps:
    """Kernels on the current CUDA device.  ``groups`` are compiled up front (in
    parallel); any other group is compiled when first used."""

    name = "cuda-sm100a"

    def __init__(self, groups: list[str] | None = None, large_gemm: str = "auto"):
        """``large_gemm`` picks the bfloat16 product for more than 16 tokens: ``"tcgen05"`` -- this
        engine's tcgen05/TMEM kernel for every such product; ``"library"`` -- the library's;
        ``"auto"`` (default) -- the tcgen05 kernel where it is at least as fast as the library
        on a B200 (the fused SwiGLU product of prompt-sized batches), the library elsewhere."""
        if large_gemm not in ("auto", "tcgen05", "library"):
            raise ValueError("large_gemm must be auto, tcgen05 or library")
        self.large_gemm = large_gemm
        self.prefill_attention = "tcgen05"  # "mma" keeps every prompt portion on the mma.sync kernel
        self.tcgen05_pairs = True           # False: the tcgen05 product never pairs SMs (cta_group::1 only)
        self.fuse_decode_new_token = True   # False: always the separate q/k norm + rotation + store kernel
        self._tickets: torch.Tensor | None = None
        self._argmax_tickets: torch.Tensor | None = None
        # products of at most 16 tokens: "auto" -- the shared-memory stream (csrc/gemm_stream.cu) for the
        # large ones, the register stream (csrc/gemm_small_m.cu) for the rest; "stream" -- the first
        # for everything it supports; "registers" -- always the second
        self.small_gemm = "auto"
        # True: a product whose result a norm folds into the residual sum may come as fp32 partial
        # sums over ranges of K (linear(partial_sums=True)); False: always a finished product
        self.partial_sums = True
        self._parts_cache: dict[tuple, int] = {}
        self._slices_cache: dict[tuple, int] = {}
        if not torch.cuda.is_available():
            raise KernelsUnavailable(
                "qwen3_runtime_b200 runs on a CUDA device only (built for NVIDIA B200, sm_100a); "
                "no CUDA device is visible and there is no CPU path"
            )
        major, _minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelsUnavailable(
                f"the kernels are compiled for sm_100a; this device reports sm_{major}{_minor}"
            )
        self._device_index = torch.cuda.current_device()
        self.SM_COUNT = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        self._fn: dict[str, ctypes._CFuncPtr] = {}
        self.launches = 0  # kernels of this engine launched (or captured) through this table
        # Per-kernel timing, off by default: a list makes every launch through this table record
        # (kernel, start event, stop event, algorithmic bytes, flops) into it; see timed_kernels().
        self.timing: list | None = None
        self._cost = (0, 0, "")
        if groups:
            build.compile_groups([g for g in groups])

    def prepare(self, groups: list[str]) -> None:
        """Compile (in parallel) the kernel groups a model is going to use."""
        build.compile_groups([g for g in groups if g in _SIGNATURES])

    # ---- plumbing -------------------------------------------------------------------
    def _get(self, group: str, name: str):
        fn = self._fn.get(name)
        if fn is None:
            lib = build.load_group(group)
            fn = getattr(lib, name)
            fn.argtypes = _SIGNATURES[group][name]
            fn.restype = c_int
            self._fn[name] = fn
        return fn

    def _stream(self) -> int:
        """The current stream's handle.  Asked for at every launch (a captured step runs on another
        stream than an eager one), so through the raw query: ``torch.cuda.current_stream()`` builds
        a Stream object and looks the device up again each time, several microseconds a call."""
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream().cuda_stream

    def _call(self, group: str, name: str, what: str, *args) -> None:
        self.launches += 1
        if self.timing is not None:
            with self._timed(what):
                _check(self._get(group, name)(*args, self._stream()), what)
            return
        _check(self._get(group, name)(*args, self._stream()), what)

    # ---- per-kernel timing (a debugging and reporting aid; never on in a timed run) ------------
    def _costs(self, nbytes: float, flops: float = 0.0, tag: str = "") -> None:
        """What the next launch has to move and compute (and a tag that tells launches of one
        kernel apart, e.g. the sizes of a product), for the timing records."""
        self._cost = (float(nbytes), float(flops), tag)

    def _timed(self, what: str):
        return _Span(self, what)

    def timed_kernels(self) -> list[dict]:
        """Sum the records of :attr:`timing` per kernel: launches, microseconds (CUDA events around
        each launch, so kernels do not overlap their neighbours as they do in a captured step),
        algorithmic bytes and flops.  Waits for the device."""
        torch.cuda.synchronize()
        table: dict[str, dict] = {}
        for what, start, stop, nbytes, flops in self.timing or []:
            row = table.setdefault(what, dict(name=what, launches=0, us=0.0, bytes=0.0, flops=0.0))
            row["launches"] += 1
            row["us"] += start.elapsed_time(stop) * 1e3
            row["bytes"] += nbytes
            row["flops"] += flops
        return sorted(table.values(), key=lambda r: -r["us"])

    # ---- norms ----------------------------------------------------------------------
    def fused_norm(self, out, weight, eps, *, resid=None, pending=None, ids=None, table=None, rows=None,
                   write_resid=True, num_rows=None):
        """RMSNorm of ``resid (+ pending)`` or of ``table[ids] (+ pending)``; see csrc/norm.cu.
        ``pending`` is ``[rows, H]`` of the output's type, or fp32 ``[parts, rows, H]``: the
        partial sums of a product (:meth:`linear` with ``partial_sums``), added in order."""
        H = weight.numel()
        n = out.shape[0] if num_rows is None else num_rows
        vocab = table.shape[0] if table is not None else 0
        parts = stride = 0
        if pending is not None and pending.dim() == 3:
            if pending.dtype != torch.float32 or pending.stride(2) != 1 or pending.stride(1) != H:
                raise KernelError("fused_norm: partial sums are fp32 [parts, rows, H] with dense rows")
            parts, stride = pending.shape[0], pending.stride(0)
        elif pending is not None and pending.dtype != out.dtype:
            raise KernelError(f"fused_norm: pending is {pending.dtype}, the output {out.dtype}")
        if self.timing is not None:
            e = out.element_size()
            self._costs(n * H * (e + (4 if resid is not None else 0) + (4 if write_resid else 0)
                                 + (4 * parts if parts else (e if pending is not None else 0))
                                 + (table.element_size() if table is not None else 0)))
        self._call("norm", "q3_fused_norm", "fused_norm",
                   _dtype_code(out.dtype), _ptr(pending), parts, stride, _ptr(resid), _ptr(ids), _ptr(table), _ptr(rows),
                  _ptr(weight), _ptr(out), n, H, float(eps), int(bool(write_resid)), vocab)
        return out

    def add_bias(self, out, bias):
        """``out[r] += bias`` in place (``bias`` float32): the bias of a projection."""
        N = out.shape[-1]
        if bias.dtype != torch.float32 or bias.numel() != N or out.stride(-1) != 1:
            raise KernelError("add_bias: a float32 bias of the output's width, rows dense")
        self._call("norm", "q3_add_bias", "add_bias", _dtype_code(out.dtype), _ptr(out), out.stride(0), _ptr(bias),
                   out.shape[0], N)
        return out

    def logit_scale_cap(self, logits, scale=1.0, cap=0.0):
        """``logits *= scale`` and, with ``cap > 0``, ``cap * tanh(logits / cap)``, in place (float32)."""
        if logits.dtype != torch.float32 or not logits.is_contiguous():
            raise KernelError("logit_scale_cap: contiguous float32 logits")
        self._call("norm", "q3_logit_scale_cap", "logit_scale_cap", _ptr(logits), logits.numel(), float(scale),
                   float(cap))
        return logits

    def silu_mul(self, gate_up, out):
        I = out.shape[-1]
        if self.timing is not None:
            self._costs(3 * out.shape[0] * I * out.element_size())
        self._call("norm", "q3_silu_mul", "silu_mul",
                   _dtype_code(out.dtype), _ptr(gate_up), _ptr(out), out.shape[0], I)
        return out

    # ---- position encoding + cache write -----------------------------------------------
    def rope_table(self, inv_freq: torch.Tensor, max_positions: int):
        half = inv_freq.numel()
        cos = torch.empty((max_positions, half), dtype=torch.float32, device=inv_freq.device)
        sin = torch.empty_like(cos)
        self._call("rope_kv", "q3_rope_table", "rope_table",
                   _ptr(inv_freq), _ptr(cos), _ptr(sin), max_positions, half)
        return cos, sin

    PAIRINGS = {"half": 0, "interleaved": 1}

    def qk_norm_rope_store(self, qkv, *, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos, sin,
                           positions, token_seq, block_table, k_pages, v_pages, page_size, write_kv,
                           pairing="half"):
        """Per-head q/k norm, rotation by ``cos/sin[position]`` and the write of k and v into their
        pages (csrc/rope_kv.cu).  ``pairing`` says which two elements of a head rotation pair i
        is made of: ``"half"`` (i, i + rotary_dim/2) or ``"interleaved"`` (2i, 2i + 1)."""
        T = qkv.shape[0]
        rot_half = cos.shape[1] if cos is not None else 0
        max_pos = cos.shape[0] if cos is not None else 0
        max_pages = block_table.shape[1] if block_table is not None else 0
        if cos is not None and (max_pos < 1 or sin is None or sin.shape != cos.shape):
            raise KernelError("qk_norm_rope_store: bad argument: rotation tables need at least one position "
                              "and cos and sin of one shape")
        if head_dim * 16 > 48 * 1024:
            raise KernelError(f"qk_norm_rope_store: head_dim={head_dim} is too large (limit 3072)")
        if self.timing is not None:
            self._costs(2 * T * (num_heads + 2 * num_kv_heads) * head_dim * qkv.element_size())
        self._call("rope_kv", "q3_qk_norm_rope_store", "qk_norm_rope_store",
                   _dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), num_heads, num_kv_heads, head_dim,
                  _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rot_half, max_pos,
                  _ptr(positions), _ptr(token_seq), _ptr(block_table), max_pages, _ptr(k_pages), _ptr(v_pages),
                  page_size, T, int(bool(write_kv)), self.PAIRINGS[pairing], _ptr(self._error_word(qkv.device)))

    # ---- attention --------------------------------------------------------------------
    def paged_attention(self, q, q_stride, *, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table,
                        token_seq, positions, out, page_size, scale, window, step=None, decode_slices=None):
        """Causal attention of every token of the step over its sequence's pages."""
        T = out.shape[0]
        if head_dim % 8 or head_dim > 256:
            raise KernelError(
                f"paged_attention: head_dim={head_dim} is not supported (multiples of 8 up to 256 are)")
        if (step is not None and step.decode_only and out.dtype == torch.bfloat16 and head_dim in (64, 128, 256)
                and num_heads // num_kv_heads <= 16 and q_stride % 8 == 0):
            return self.paged_attention_decode(
                q, q_stride, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, k_pages=k_pages,
                v_pages=v_pages, block_table=block_table, kv_lens=step.kv_lens, cu_seqlens=step.cu_seqlens,
                out=out, page_size=page_size, scale=scale, window=window, num_seqs=step.num_seqs,
                max_kv_len=step.captured_width * page_size or step.max_kv_len, step=step,
                num_splits=decode_slices, longest=getattr(step, "kv_longest", None))
        if (step is not None and out.dtype == torch.bfloat16 and head_dim in (64, 128)
                and num_heads // num_kv_heads <= 16 and q_stride % 8 == 0):
            # portions of prompts on the tensor-core kernel, one-token sequences on the split-KV kernel
            group = num_heads // num_kv_heads
            cu = step.host_cu_seqlens
            qlens = [cu[b + 1] - cu[b] for b in range(step.num_seqs)]
            work = sum(-(-n * group // 128) for n in qlens if n > 1)
            done = False
            if (work and head_dim == 128 and not window and 128 % group == 0 and page_size in (8, 16, 32, 64)
                    and self.prefill_attention == "tcgen05"):
                # tcgen05/TMEM kernel; it answers "unsupported" for what it does not take
                self.launches += 1
                pairs = sum(-(-(-(-n * group // 128)) // 2) for n in qlens if n > 1)  # two row blocks per work item
                launch = lambda: self._get("attention_prefill_tc", "q3_paged_attention_prefill_tc")(  # noqa: E731
                    _ptr(q), q_stride, q.shape[0], _ptr(k_pages), _ptr(v_pages),
                    k_pages.shape[0] * num_kv_heads * page_size, _ptr(block_table), block_table.shape[1],
                    _ptr(step.kv_lens), _ptr(step.cu_seqlens), _ptr(out), step.num_seqs, pairs, num_heads,
                    num_kv_heads, head_dim, page_size, float(scale), 1, _ptr(self._error_word(out.device)),
                    self._stream())
                if self.timing is not None:
                    self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=True))
                    with self._timed("paged_attention_prefill_tc"):
                        code = launch()
                else:
                    code = launch()
                if code == 0:
                    done = True
                elif code != 1:
                    _check(code, "paged_attention_prefill_tc")
            if work and not done:
                if self.timing is not None:
                    self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=True))
                self._call("attention_prefill", "q3_paged_attention_prefill", "paged_attention_prefill",
                           _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                           block_table.shape[1], _ptr(step.kv_lens), _ptr(step.cu_seqlens), _ptr(out),
                           step.num_seqs, work, num_heads, num_kv_heads, head_dim, page_size, float(scale),
                           int(window or 0), 1)
            if step.num_single:
                singles = [kv for kv, n in zip(step.host_kv_lens, qlens) if n == 1]
                longest = max(singles)
                self.paged_attention_decode(
                    q, q_stride, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                    k_pages=k_pages, v_pages=v_pages, block_table=block_table, kv_lens=step.kv_lens,
                    cu_seqlens=step.cu_seqlens, out=out, page_size=page_size, scale=scale, window=window,
                    num_seqs=step.num_single, max_kv_len=longest, seq_list=step.single_seqs, step=step,
                    num_splits=self.decode_slices_for(singles, num_kv_heads, head_dim, window))
            return out
        if self.timing is not None and step is not None:
            self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out))
        self._call("attention_generic", "q3_paged_attention_generic", "paged_attention",
                   _dtype_code(out.dtype), _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                  block_table.shape[1], _ptr(token_seq), _ptr(positions), _ptr(out), T, num_heads, num_kv_heads,
                  head_dim, page_size, float(scale), int(window or 0))
        return out

    @staticmethod
    def _attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=None):
        """(bytes, flops) of a step's attention: every key and value of each sequence read once, q
        read and the result written; 4 * heads * head_dim flops per (query, key) pair.
        ``prompts``: True counts only sequences that bring more than one token, False only those
        that bring one, None all."""
        e = out.element_size()
        keys = pairs = rows = 0
        cu = step.host_cu_seqlens
        for b, kv in enumerate(step.host_kv_lens):
            n = cu[b + 1] - cu[b] if len(cu) > b + 1 else 1
            if prompts is not None and (n > 1) != prompts:
                continue
            keys += kv
            rows += n
            pairs += n * kv - n * (n - 1) // 2
        return (2 * keys * num_kv_heads * head_dim * e + 2 * rows * num_heads * head_dim * e,
                4 * num_heads * head_dim * pairs)

    SM_COUNT = 148  # of a B200; replaced by the device's own count when the table is built
    TICKETS = 1 << 16  # ticket words for the merge by the last block: sequences x kv heads of one launch
    # blocks of the split-KV kernel that an SM holds, by head size (registers allow 4 / 3 / 2,
    # shared memory 6 / 3 / 1)
    DECODE_BLOCKS_PER_SM = {64: 4, 128: 3, 256: 1}

    def decode_splits(self, num_seqs: int, num_kv_heads: int, max_kv_len: int, head_dim: int = 128) -> int:
        """How many slices each sequence's keys are cut into when all that is known is their number
        and an upper bound of their length (a captured step without :meth:`decode_slices_for`)."""
        return self._decode_slices([-(-max(1, max_kv_len) // 64)] * max(1, num_seqs), num_kv_heads, head_dim)

    def decode_slices_for(self, kv_lens: list[int], num_kv_heads: int, head_dim: int, window: int | None) -> int:
        """Into how many slices the split-KV kernel cuts the longest of these sequences (asked once
        per decode step by the attention parts' chooser; answers are kept by the sequences' lengths
        in tiles of 64 keys)."""
        cap = (int(window) + 63) if window else None
        tiles = tuple(-(-(n if cap is None or n < cap else cap) // 64) for n in kv_lens)
        key = (num_kv_heads, head_dim, tiles)
        slices = self._slices_cache.get(key)
        if slices is None:
            if len(self._slices_cache) > 8192:
                self._slices_cache.clear()
            slices = self._slices_cache[key] = self._decode_slices(tiles, num_kv_heads, head_dim)
        return slices

    def _decode_slices(self, tiles, num_kv_heads: int, head_dim: int) -> int:
        """The slice count for sequences of ``tiles`` x 64 keys.  With ``s`` slices the longest
        sequence is cut into slices of ``ceil(longest / s)`` tiles and every other sequence into as
        many slices of that length as it needs (the kernel's rule), which gives the number of
        blocks.  The cost of a choice, in units of the time one key takes to stream when every block
        slot (3 per SM at head size 128) is busy: while all blocks fit the slots, keys per slice + 12 per slice (the
        last block of a pair merges them); beyond that, waves x (keys per slice + 384), the 384 being
        what a block pays besides its keys (lengths, block table and first tile at the start, the
        warps' merge and the ticket at the end), which a full machine no longer hides; waves are
        whole up to six and blocks / slots + 1/2 beyond (blocks of equal length start and end
        together at first and drift apart later).  Slices are at least 192 keys long, 64 with at most
        32 (sequence, kv head) pairs.  The constants are fitted to a sweep of 1..128 sequences x
        256..16384 keys x 1..64 slices on a B200 (8 kv heads of 128,
        ``python -m qwen3_runtime_b200.ops.tune decode_splits``): the choice is within 0.6 % of the
        best one on average and 13 % at worst for sequences of one length, and within a few percent
        for the mixed batches tried.  The reference's rule for an RTX 4090 looks at the number of
        sequences and the longest one (qwen3_runtime/kernels/triton_decode.py:122-133)."""
        import numpy as np

        t = np.asarray(tiles, dtype=np.int64)
        t = t[t > 0]
        if t.size == 0:
            return 1
        longest = int(t.max())
        slots = self.DECODE_BLOCKS_PER_SM.get(head_dim, 3) * self.SM_COUNT
        # a key of a smaller head streams faster, what a block pays besides its keys stays; merging a
        # slice costs in proportion to the head size, like a key
        fixed, per_slice = 384.0 * 128.0 / head_dim, 12.0
        floor = 1 if t.size * num_kv_heads <= 32 else 3  # tiles
        counts = np.arange(1, min(64, longest) + 1)
        slice_tiles = -(-longest // counts)
        counts = counts[(slice_tiles >= floor) | (counts == 1)]
        slice_tiles = -(-longest // counts)
        blocks = num_kv_heads * (-(-t[None, :] // slice_tiles[:, None])).sum(axis=1)
        per = 64.0 * slice_tiles
        waves = blocks / slots
        waves = np.where(waves <= 6, np.ceil(waves), waves + 0.5)
        cost = np.where(blocks <= slots, per, waves * (per + fixed)) + per_slice * counts
        return int(counts[int(np.argmin(cost))])

    def decode_new_token_ok(self, qkv, *, num_heads, num_kv_heads, head_dim, cos, q_weight, k_weight) -> bool:
        """Whether the split-KV kernel can make q, k and v of the newest token itself (per-head
        norm, rotation, cache write) for a step in which every sequence brings one token."""
        return (self.fuse_decode_new_token and qkv.dtype == torch.bfloat16 and head_dim in (64, 128, 256)
                and num_heads // num_kv_heads <= 16 and qkv.stride(0) % 8 == 0
                and (cos is None or 2 * cos.shape[1] == head_dim)
                and (q_weight is None) == (k_weight is None))

    def paged_attention_decode(self, q, q_stride, *, num_heads, num_kv_heads, head_dim, k_pages, v_pages,
                               block_table, kv_lens, cu_seqlens, out, page_size, scale, window, num_seqs,
                               max_kv_len, seq_list=None, num_splits=None, new_token=None, step=None,
                               merge_kernel=False, longest=None):
        """Split-KV attention for sequences that bring one token each (csrc/attention_decode.cu).
        ``new_token`` (q_weight, k_weight, eps, cos, sin, optionally pairing): ``q`` is the raw q/k/v
        projection and the kernel also does the work of :meth:`qk_norm_rope_store` for the newest
        position of each sequence, ``kv_lens - 1``.  The slices of a sequence and kv head are merged
        by whichever of their blocks finishes last (a ticket word per pair); ``merge_kernel=True``
        asks for the second kernel that callers without ticket words get (the bits are the same).
        ``num_splits`` is the slice count of the longest sequence (a shorter one gets fewer slices of
        about the same length); ``longest``: a device int32 holding the longest of the sequences'
        lengths, when the caller has it (else every block works it out from ``kv_lens``)."""
        if out.dtype != torch.bfloat16 or head_dim not in (64, 128, 256) or num_heads // num_kv_heads > 16:
            raise KernelError("paged_attention_decode: bfloat16, head_dim 64/128/256 and groups of at most 16 only")
        if window:
            max_kv_len = min(max_kv_len, int(window) + 63)
        splits = num_splits or self.decode_splits(num_seqs, num_kv_heads, max_kv_len, head_dim)
        mid_o = mid_lse = None
        tickets = None
        if splits > 1:
            mid_o = torch.empty((num_seqs, num_heads, splits, head_dim), dtype=torch.float32, device=out.device)
            mid_lse = torch.empty((num_seqs, num_heads, splits), dtype=torch.float32, device=out.device)
            if not merge_kernel and num_seqs * num_kv_heads <= self.TICKETS:
                if self._tickets is None:  # zero between launches: the kernel leaves them so
                    self._tickets = torch.zeros(self.TICKETS, dtype=torch.int32, device=out.device)
                tickets = self._tickets
            else:
                self.launches += 1  # the merge kernel
        err = _ptr(self._error_word(out.device))
        if self.timing is not None and step is not None:
            self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=False))
        if new_token is not None:
            cos, sin = new_token["cos"], new_token["sin"]
            self._call("attention_decode", "q3_paged_attention_decode_fused", "paged_attention_decode_fused",
                       _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                       _ptr(kv_lens), _ptr(cu_seqlens), _ptr(seq_list), _ptr(out), _ptr(mid_o), _ptr(mid_lse),
                       num_seqs, num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
                       splits, _ptr(new_token["q_weight"]), _ptr(new_token["k_weight"]), float(new_token["eps"]),
                       _ptr(cos), _ptr(sin), cos.shape[0] if cos is not None else 0,
                       self.PAIRINGS[new_token.get("pairing", "half")], err, _ptr(tickets), _ptr(longest))
            return out
        self._call("attention_decode", "q3_paged_attention_decode", "paged_attention_decode",
                   _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                   _ptr(kv_lens), _ptr(cu_seqlens), _ptr(seq_list), _ptr(out), _ptr(mid_o), _ptr(mid_lse),
                   num_seqs, num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0), splits,
                   _ptr(tickets), _ptr(longest))
        return out

    # ---- matrix products ----------------------------------------------------------------
    def linear(self, x, weight, out=None, out_dtype=None, partial_sums=False, bias=None):
        """See :meth:`_product`; ``bias`` (float32 ``[N]``) is added to the finished product, which
        then never comes as partial sums."""
        if bias is None:
            return self._product(x, weight, out, out_dtype, partial_sums)
        return self.add_bias(self._product(x, weight, out, out_dtype, False), bias)

    def _product(self, x, weight, out=None, out_dtype=None, partial_sums=False):
        """``x[M, K] @ weight[N, K]^T``.  float32: this engine's FMA kernel (no TF32).
        bfloat16, at most 16 tokens: one of this engine's two weight-streaming kernels
        (:meth:`_small_product`).  bfloat16, more tokens: the library product with fp32
        accumulation, as the reference's ``nn.Linear`` (qwen3_runtime/models/qwen3.py:76-77,
        134-135), or this engine's tcgen05 kernel with ``large_gemm="tcgen05"``.

        ``partial_sums``: the caller also takes float32 ``[parts, M, N]`` whose sum over the
        first axis is the product (what :meth:`fused_norm` accepts as ``pending``).  It gets
        that when the streaming kernel would cut K into ranges: the blocks then need not
        wait for one another to add their parts up."""
        M, K = x.shape
        N = weight.shape[0]
        if weight.shape[1] != K:
            raise KernelError(f"linear: x is [{M},{K}] but weight is {list(weight.shape)}")
        if self.timing is not None:
            e = x.element_size()
            oe = 4 if out_dtype == torch.float32 else e
            self._costs(N * K * e + M * K * e + M * N * oe, 2.0 * M * N * K, f" {M}x{K}->{N}")
        if (partial_sums and self.partial_sums and out is None and out_dtype is None and M > 0
                and self.small_gemm != "registers" and self._small_m_ok(x, weight)):
            parts = self._stream_parts(M, N, K)
            if parts > 1:
                planes = torch.empty((parts, M, N), dtype=torch.float32, device=x.device)
                self._call("gemm_stream", "q3_gemm_stream_partial", "gemm_stream_partial", _ptr(x), x.stride(0),
                           _ptr(weight), weight.stride(0), _ptr(planes), parts, M, N, K,
                           _ptr(self._error_word(x.device)))
                return planes
        if x.dtype == torch.float32:
            if out is None:
                out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            self._call("gemm_f32", "q3_gemm_f32", "gemm_f32", _ptr(x), x.stride(0), _ptr(weight),
                       weight.stride(0), _ptr(out), out.stride(0), M, N, K)
            return out
        if self._small_m_ok(x, weight):
            odt = out_dtype or x.dtype
            if out is None:
                out = torch.empty((M, N), dtype=odt, device=x.device)
            self._small_product(1 if odt == torch.float32 else 0, x, weight, out, M, N, K)
            return out
        if self.large_gemm == "tcgen05" and self._tcgen05_ok(x, weight):
            return self.linear_tcgen05(x, weight, out=out, out_dtype=out_dtype)
        if self.timing is not None:
            with self._timed("library_mm"):
                return self._library_mm(x, weight, out, out_dtype)
        return self._library_mm(x, weight, out, out_dtype)

    @staticmethod
    def _library_mm(x, weight, out, out_dtype):
        if out_dtype is not None and out_dtype != x.dtype:
            return torch.mm(x, weight.t(), out_dtype=out_dtype)
        if out is None:
            return torch.mm(x, weight.t())
        return torch.mm(x, weight.t(), out=out)

    def _tcgen05_ok(self, x, weight) -> bool:
        return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
                and weight.stride(0) % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    ERR_POSITION = 16  # csrc/rope_kv.cu, csrc/attention_decode.cu: a position outside the rotation tables

    def _error_word(self, device) -> torch.Tensor:
        if getattr(self, "_err", None) is None:
            self._err = torch.zeros(1, dtype=torch.int32, device=device)
        return self._err

    def raise_if_kernel_error(self) -> None:
        """A bounded wait inside a kernel expired (it gave up and returned).  Reads one int from
        the device, so call it where the host waits for the device anyway."""
        err = getattr(self, "_err", None)
        code = int(err.item()) if err is not None else 0
        if code == self.ERR_POSITION:
            err.zero_()
            raise KernelError("a token's position lies outside the rotation tables of the position encoding: "
                              "its query and key were left unrotated and the step's output is invalid")
        if code != 0:
            err.zero_()
            if self._tickets is not None:  # a kernel that gave up may have left tickets drawn
                self._tickets.zero_()
            if self._argmax_tickets is not None:
                self._argmax_tickets.zero_()
            raise KernelError("a bounded wait inside a kernel expired (tcgen05 product or attention, or the "
                              "streaming product): the kernel gave up and its output is invalid")

    def watch_kernel_errors(self) -> None:
        """Enqueue a copy of the error word to pinned host memory, without waiting for it.
        :meth:`raise_if_watched_error` looks at the copy once the host has waited for the
        device for a reason of its own (the sampled tokens), so a step pays no extra wait."""
        err = getattr(self, "_err", None)
        if err is None:
            return
        if getattr(self, "_err_host", None) is None:
            self._err_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._err_host.copy_(err, non_blocking=True)

    def raise_if_watched_error(self) -> None:
        host = getattr(self, "_err_host", None)
        if host is not None and int(host[0]) != 0:
            host.zero_()
            self.raise_if_kernel_error()

    def linear_tcgen05(self, x, weight, out=None, out_dtype=None, mode=None, pair=None):
        """``x @ weight^T`` on tcgen05 tensor cores (csrc/gemm_tcgen05.cu).  ``mode=2``: SwiGLU with
        ``weight = [W_gate; W_up]``, ``out`` is ``[M, I]``.  ``pair``: the kernel that runs each
        256-token tile on two SMs (cta_group::2); default: when there are more than 128 tokens."""
        M, K = x.shape
        if not self._tcgen05_ok(x, weight):
            raise KernelError("gemm_tcgen05: bfloat16 operands with 16-byte aligned rows (K multiple of 8) only")
        if mode == 2:
            N = weight.shape[0] // 2
            odt = x.dtype
        else:
            N = weight.shape[0]
            odt = out_dtype or x.dtype
            mode = 1 if odt == torch.float32 else 0
        if out is None:
            out = torch.empty((M, N), dtype=odt, device=x.device)
        if pair is None:
            pair = self.tcgen05_pairs and M > 128 and self._tcgen05_plan(M, N)[0]
        self._call("gemm_tcgen05", "q3_gemm_tcgen05_pair" if pair else "q3_gemm_tcgen05", "gemm_tcgen05", mode,
                   _ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K,
                   _ptr(self._error_word(x.device)))
        return out

    def _tcgen05_plan(self, M: int, N: int) -> tuple[bool, float, float]:
        """(whether pairs of SMs should run the tiles, share of the token rows of the tiles that holds
        real tokens, share of the tile slots of all rounds that holds real work).  Both kernels work
        through their tiles in rounds over all SMs: 128 tokens x 128 features (of each of gate and up
        for SwiGLU) per SM, or 256 x 128 per pair.  A token count just above a multiple of the tile
        leaves most of the last token tile empty, a tile count just above a multiple of the SMs most of
        the last round."""
        cols = -(-N // 128)
        pairs = self.SM_COUNT // 2
        fill_1, fill_2 = M / (-(-M // 128) * 128), M / (-(-M // 256) * 256)
        single = (M / 128) * cols / (-(-(-(-M // 128) * cols) // self.SM_COUNT) * self.SM_COUNT)
        paired = (M / 256) * cols / (-(-(-(-M // 256) * cols) // pairs) * pairs)
        return (True, fill_2, paired) if paired >= single else (False, fill_1, single)

    SMALL_M = 16
    # The fused gate_up + SwiGLU product goes to the tcgen05 kernel when its token tiles are at least
    # this full and its rounds at least that full; else to the library product and a SwiGLU pass.
    # Measured at 129..4096 tokens x three model sizes: the library, with finer token tiles, wins
    # clearly (20-50 %) when the last token tile is mostly empty or the work fills less than a round
    # and a half; where only the last round is thin the two are within a few percent and the fused
    # kernel saves a launch and a pass over [tokens, 2 x intermediate].
    TCGEN05_MIN_TOKEN_FILL = 0.9
    TCGEN05_MIN_SHARE = 0.65

    def _stream_parts(self, M: int, N: int, K: int) -> int:
        """Ranges of K in the streaming kernel's partial-sum mode (0: it does not take the product)."""
        key = (M > 8, N, K)
        parts = self._parts_cache.get(key)
        if parts is None:
            parts = self._parts_cache[key] = int(self._get("gemm_stream", "q3_gemm_stream_parts")(M, N, K))
        return parts

    def _small_product(self, mode: int, x, weight, out, M, N, K) -> None:
        """A product of at most 16 tokens: the streaming kernel (csrc/gemm_stream.cu), or the
        register-streaming one (csrc/gemm_small_m.cu) for what the first refuses."""
        if self.small_gemm != "registers":
            self.launches += 1
            cost, span = self._cost, None
            if self.timing is not None:
                span = self._timed("gemm_stream").__enter__()
            code = self._get("gemm_stream", "q3_gemm_stream")(
                mode, _ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K,
                int(self.small_gemm == "auto"), _ptr(self._error_word(x.device)), self._stream())
            if code == 0:
                if span is not None:
                    span.__exit__()
                return
            self._cost = cost  # refused before any launch: the register kernel takes the product
            self.launches -= 1
            if code != 1:
                _check(code, "gemm_stream")
        self._call("gemm_small_m", "q3_gemm_small_m", "gemm_small_m", mode, _ptr(x), x.stride(0), _ptr(weight),
                   weight.stride(0), _ptr(out), out.stride(0), M, N, K)

    def _small_m_ok(self, x, weight) -> bool:
        return (x.dtype == torch.bfloat16 and x.shape[0] <= self.SMALL_M and x.shape[1] % 8 == 0
                and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.stride(1) == 1
                and weight.stride(1) == 1 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    def gated_linear(self, x, gate_up_weight, out):
        """``out = silu(x @ W_gate^T) * (x @ W_up^T)`` with ``gate_up_weight = [W_gate; W_up]``:
        one kernel for a handful of tokens, else the product followed by the SwiGLU kernel."""
        M, K = x.shape
        I = out.shape[1]
        if self.timing is not None:
            e = x.element_size()
            self._costs((2 * I * K + M * K + M * I) * e, 4.0 * M * I * K, f" {M}x{K}->2x{I} swiglu")
        if self._small_m_ok(x, gate_up_weight):
            self._small_product(2, x, gate_up_weight, out, M, I, K)
            return out
        if self.large_gemm != "library" and self._tcgen05_ok(x, gate_up_weight):
            _pair, token_fill, share = self._tcgen05_plan(M, I)
            if self.large_gemm == "tcgen05" or (token_fill >= self.TCGEN05_MIN_TOKEN_FILL
                                                and share >= self.TCGEN05_MIN_SHARE):
                return self.linear_tcgen05(x, gate_up_weight, out=out, mode=2)
        return self.silu_mul(self.linear(x, gate_up_weight), out)

    # ---- sampling ---------------------------------------------------------------------
    def argmax(self, logits, want_logprob=False):
        R, V = logits.shape
        if self.timing is not None:
            self._costs(R * V * 4)
        token = torch.empty(R, dtype=torch.int32, device=logits.device)
        logprob = torch.empty(R, dtype=torch.float32, device=logits.device) if want_logprob else None
        slices, scratch, tickets = self._row_slices(logits)
        self._call("sampling", "q3_argmax", "argmax",
                   _ptr(logits), R, V, _ptr(token), _ptr(logprob), _ptr(scratch), _ptr(tickets), slices)
        return token, logprob

    def _row_slices(self, logits):
        """Few long rows: cut each into slices so that about two blocks per SM share the work; the
        slices' results meet in a scratch, and a ticket word per row tells the last block."""
        R, V = logits.shape
        slices = max(0, min(1024, 2 * self.SM_COUNT // max(R, 1), V // 2048))
        if slices <= 1 or R > self.TICKETS:
            return 0, None, None
        if self._argmax_tickets is None:  # zero between launches: the kernels leave them so
            self._argmax_tickets = torch.zeros(self.TICKETS, dtype=torch.int32, device=logits.device)
        scratch = torch.empty((R, slices, 4), dtype=torch.float32, device=logits.device)
        return slices, scratch, self._argmax_tickets

    def sample(self, logits, temperature, uniform, want_logprob=False):
        R, V = logits.shape
        token = torch.empty(R, dtype=torch.int32, device=logits.device)
        logprob = torch.empty(R, dtype=torch.float32, device=logits.device) if want_logprob else None
        slices, scratch, tickets = self._row_slices(logits)
        if self.timing is not None:
            self._costs(R * V * 4)
        self._call("sampling", "q3_sample", "sample", _ptr(logits), R, V, _ptr(temperature), _ptr(uniform),
                   _ptr(token), _ptr(logprob), _ptr(scratch), _ptr(tickets), slices)
        return token, logprob


    def bias_penalty_row(self, row, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                         frequency_penalty):
        """Logit bias and repetition / presence / frequency penalties, in place on one fp32 row
        (qwen3_runtime/sampling.py:36-72)."""
        V = row.numel()
        dev = row.device
        bias_ids = bias_vals = seen = counts = None
        n_bias = n_seen = 0
        if logit_bias:
            n_bias = len(logit_bias)
            bias_ids = torch.tensor([int(k) for k in logit_bias], dtype=torch.int32, device=dev)
            bias_vals = torch.tensor([float(v) for v in logit_bias.values()], dtype=torch.float32, device=dev)
        if seen_ids and not (repetition_penalty == 1.0 and presence_penalty == 0.0 and frequency_penalty == 0.0):
            n_seen = len(seen_ids)
            seen = torch.tensor(seen_ids, dtype=torch.int32, device=dev)
            counts = torch.empty(V, dtype=torch.int32, device=dev)
        self._call("sampling", "q3_bias_penalty", "bias_penalty", _ptr(row), V, _ptr(bias_ids), _ptr(bias_vals),
                   n_bias, _ptr(seen), n_seen, _ptr(counts), float(repetition_penalty), float(presence_penalty),
                   float(frequency_penalty))
        return row

    def bias_penalty_rows(self, logits, rows, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                          frequency_penalty):
        """:meth:`bias_penalty_row` for several rows of ``logits`` at once (lists with one entry per
        row of ``rows``): everything the rows need goes to the device as one integer and one float
        buffer, and one launch with a block per row works on them."""
        n, V, dev = len(rows), logits.shape[1], logits.device
        biases = [b or {} for b in logit_bias]
        ints, bias_off, seen_off = list(int(r) for r in rows), [0], [0]
        for b in biases:
            bias_off.append(bias_off[-1] + len(b))
        for s, rp, pp, fp in zip(seen_ids, repetition_penalty, presence_penalty, frequency_penalty):
            live = bool(s) and not (rp == 1.0 and pp == 0.0 and fp == 0.0)
            seen_off.append(seen_off[-1] + (len(s) if live else 0))
        packed = ints + bias_off + seen_off
        packed += [int(k) for b in biases for k in b]
        packed += [int(t) for s, a, z in zip(seen_ids, seen_off, seen_off[1:]) if z > a for t in s]
        floats = [float(v) for triple in zip(repetition_penalty, presence_penalty, frequency_penalty) for v in triple]
        floats += [float(v) for b in biases for v in b.values()]
        host_i = torch.tensor(packed, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        host_f = torch.tensor(floats, dtype=torch.float32).pin_memory().to(dev, non_blocking=True)
        counts = torch.empty((n, V), dtype=torch.int32, device=dev)
        o_bias, o_seen = n, 2 * n + 1
        o_bias_ids = 3 * n + 2
        o_seen_ids = o_bias_ids + bias_off[-1]
        self._call("sampling", "q3_bias_penalty_rows", "bias_penalty_rows", _ptr(logits), V, n, _ptr(host_i),
                   _ptr(host_i[o_bias:]), _ptr(host_i[o_bias_ids:]) if bias_off[-1] else None,
                   _ptr(host_f[3 * n:]) if bias_off[-1] else None, _ptr(host_i[o_seen:]),
                   _ptr(host_i[o_seen_ids:]) if seen_off[-1] else None, _ptr(counts), _ptr(host_f))
        return logits

    def filter_rows(self, logits, temperature, min_p, top_k, top_p):
        """Divide by the temperature, then min_p, top_k and top_p masks, in place on fp32 rows
        (qwen3_runtime/sampling.py:75-109, 130-135).  The four arguments are per-row device tensors."""
        R, V = logits.shape
        self._call("sampling", "q3_filter", "filter", _ptr(logits), R, V, _ptr(temperature), _ptr(min_p),
                   _ptr(top_k), _ptr(top_p))
        return logits


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
